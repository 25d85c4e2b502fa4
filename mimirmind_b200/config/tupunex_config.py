"""Typed configuration of a Tupunex decoder, read from its ``config.json``.

The file gives every size and every constant that differs between models of the design, layer by layer::

    {"architecture": "Tupunex", "vocab": V, "width": D, "norm": {"eps": e}, "embedding": {"scale": s}, "streams": S,
     "loop": {"start": a, "stop": b, "times": n},
     "layers": [{"type": "attention",
                 "mixer": {"heads", "kv_heads", "dim", "vdim", "scale", "softcap", "diff", "conv", "mask": {"size"}}, "mlp": ...},
                {"type": "latent_attention",
                 "mixer": {"heads", "dim", "rot_dim", "vdim", "kv_rank", "scale", "rot": {"base", "dims"}}, "mlp": ...}]}

with ``mlp`` either null or ``{"kind": "dense", "ff": F}``.  Required keys fail with the key's path.  Keys that may be
absent mean "the model has none of it": ``streams`` (one residual stream, the ordinary sum), ``loop`` (every layer runs
once), ``embedding`` (scale 1), and in an attention layer ``mask`` (every earlier token is seen), ``softcap`` and ``conv``.
Same "required key throws" manner as the reference's config readers (src/model/LlmConfig.cpp:64-93).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Optional, Tuple

from .bigerax_config import _At
from .model_config import ConfigError

ARCHITECTURE = "Tupunex"


@dataclass(frozen=True)
class DifferentialLayer:
    """Two softmax maps per head over the same values, the second subtracted from the first."""
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    diff: float
    softcap: float = 0.0         # 0: scores are not capped
    window: int = 0              # 0: every earlier token
    conv: int = 0                # taps of the short convolution on q, k and v; 0: none


@dataclass(frozen=True)
class LatentLayer:
    """Keys and values of every head made from one cached latent vector per token, plus one rotated key part."""
    heads: int
    dim: int
    rot_dim: int
    vdim: int
    kv_rank: int
    scale: float
    rot_dims: int
    rot_base: float


@dataclass(frozen=True)
class DenseFeedForward:
    ff: int


@dataclass(frozen=True)
class TupunexLayer:
    type: str                               # "attention" or "latent_attention"
    mixer: Any
    mlp: Optional[DenseFeedForward]


@dataclass(frozen=True)
class Loop:
    start: int
    stop: int
    times: int


@dataclass(frozen=True)
class TupunexConfig:
    architecture: str
    vocab: int
    width: int
    norm_eps: float
    embedding_scale: float
    streams: int                            # 0: one residual stream and the ordinary sum
    loop: Optional[Loop]
    layers: Tuple[TupunexLayer, ...]
    max_positions: int
    eos_token_ids: Tuple[int, ...] = ()

    def order(self) -> Tuple[int, ...]:
        """The layers in the order they run: those of the loop ``times`` times in a row."""
        n = len(self.layers)
        if self.loop is None:
            return tuple(range(n))
        a, b = self.loop.start, self.loop.stop
        return tuple(range(a)) + tuple(range(a, b)) * self.loop.times + tuple(range(b, n))


def _optional_number(at: _At, key: str, default: float) -> float:
    return at.number(key) if at.obj.get(key) is not None else default


def parse_tupunex_config(obj: Dict[str, Any], where: str = "config.json") -> TupunexConfig:
    top = _At(obj, "", where)
    width = top.integer("width")
    raw_layers = top.need("layers")
    if not isinstance(raw_layers, list) or not raw_layers:
        raise ConfigError(f"{where}: 'layers' must be a non-empty list")
    layers = []
    for i, raw in enumerate(raw_layers):
        at = _At(raw, f"layers[{i}]", where)
        kind = at.need("type")
        m = at.child("mixer")
        if kind == "attention":
            heads, kv = m.integer("heads"), m.integer("kv_heads")
            if heads % kv:
                raise ConfigError(f"{where}: '{m._name('heads')}' = {heads} is not a multiple of kv_heads = {kv}")
            mask = m.maybe("mask")
            mixer = DifferentialLayer(
                heads=heads, kv_heads=kv, dim=m.integer("dim"), vdim=m.integer("vdim"), scale=m.number("scale"), diff=m.number("diff"),
                softcap=_optional_number(m, "softcap", 0.0), window=mask.integer("size") if mask is not None else 0,
                conv=m.integer("conv") if m.obj.get("conv") is not None else 0)
            if mixer.softcap < 0:
                raise ConfigError(f"{where}: '{m._name('softcap')}' must not be negative")
        elif kind == "latent_attention":
            rot = m.child("rot")
            rot_dim, rot_dims = m.integer("rot_dim"), rot.integer("dims", 0)
            if rot_dims % 2 or rot_dims > rot_dim:
                raise ConfigError(f"{where}: '{m._name('rot.dims')}' = {rot_dims} must be even and at most rot_dim = {rot_dim}")
            mixer = LatentLayer(heads=m.integer("heads"), dim=m.integer("dim"), rot_dim=rot_dim, vdim=m.integer("vdim"),
                                kv_rank=m.integer("kv_rank"), scale=m.number("scale"), rot_dims=rot_dims,
                                rot_base=rot.number("base") if rot_dims else 1.0)
        else:
            raise ConfigError(f"{where}: layers[{i}].type = {kind!r} is not one of 'attention', 'latent_attention'")
        mlp_at = at.maybe("mlp")
        mlp = None
        if mlp_at is not None:
            if mlp_at.need("kind") != "dense":
                raise ConfigError(f"{where}: layers[{i}].mlp.kind = {mlp_at.obj['kind']!r} is not 'dense'")
            mlp = DenseFeedForward(ff=mlp_at.integer("ff"))
        layers.append(TupunexLayer(type=kind, mixer=mixer, mlp=mlp))
    loop = None
    loop_at = top.maybe("loop")
    if loop_at is not None:
        loop = Loop(start=loop_at.integer("start", 0), stop=loop_at.integer("stop", 0), times=loop_at.integer("times", 1))
        if not (loop.start <= loop.stop <= len(layers)):
            raise ConfigError(f"{where}: 'loop' runs layers {loop.start} .. {loop.stop - 1}, the model has {len(layers)}")
    streams = top.integer("streams") if obj.get("streams") is not None else 0
    if streams > 8:
        raise ConfigError(f"{where}: 'streams' = {streams}: at most 8 residual streams are supported")
    emb = top.maybe("embedding")
    eos = obj.get("eos_token_id")
    eos_ids = tuple(eos) if isinstance(eos, list) else ((eos,) if isinstance(eos, int) else ())
    max_pos = obj.get("max_positions")
    return TupunexConfig(architecture=str(obj.get("architecture", ARCHITECTURE)), vocab=top.integer("vocab"), width=width,
                         norm_eps=top.child("norm").number("eps"), embedding_scale=_optional_number(emb, "scale", 1.0) if emb is not None else 1.0,
                         streams=streams, loop=loop, layers=tuple(layers),
                         max_positions=int(max_pos) if isinstance(max_pos, int) and max_pos > 0 else 1 << 20, eos_token_ids=eos_ids)
