"""Typed configuration of a Zubarax decoder, read from its ``config.json``.

The file gives every size and every constant that differs between models of the design, layer by layer::

    {"architecture": "Zubarax", "vocab": V, "width": D, "norm": {"eps": e}, "postln_alpha": a, "embedding": {"scale": s},
     "layers": [{"type": "parallel",
                 "mixer": {"left": {"heads", "kv_heads", "dim", "vdim", "scale", "conv", "rot": {"base", "dims"}},
                           "right": {"heads", "dim", "vdim"}, "left_scale", "right_scale"},
                 "mlp": {"kind": "moe", "expert": {"ff", "limit"}, "router": {"experts", "top"}, "shared": {"ff", "limit"}},
                 "weights_of": j}, ...]}

``mlp`` may be null (the layer has no feed-forward); ``shared``, ``rot``, ``conv`` and ``embedding`` may be absent and then
mean "none of it" (a scale of 1).  A layer with ``weights_of: j`` runs with layer j's tensors and a cache and state of its
own; the rest of its entry must equal layer j's.  Required keys fail with the key's path, in the manner of the reference's
config readers (src/model/LlmConfig.cpp:64-93).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Optional, Tuple

from .bigerax_config import _At
from .model_config import ConfigError

ARCHITECTURE = "Zubarax"


@dataclass(frozen=True)
class TalkingSide:
    """Softmax attention with short convolutions, q/k norm, partial rotation, unit values, mixed heads and a sink."""
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    conv: int = 0
    rot_dims: int = 0
    rot_base: float = 1.0


@dataclass(frozen=True)
class ForgetGateSide:
    """Linear attention with a forget gate per key channel whose complement is the write strength."""
    heads: int
    dim: int
    vdim: int


@dataclass(frozen=True)
class ParallelMixer:
    left: TalkingSide
    right: ForgetGateSide
    left_scale: float
    right_scale: float


@dataclass(frozen=True)
class ClampedExpert:
    ff: int
    limit: float


@dataclass(frozen=True)
class ExpertsFeedForward:
    expert: ClampedExpert
    experts: int
    top: int
    shared: Optional[ClampedExpert]


@dataclass(frozen=True)
class ZubaraxLayer:
    type: str                               # "parallel"
    mixer: ParallelMixer
    mlp: Optional[ExpertsFeedForward]
    weights_of: Optional[int] = None        # the layer whose tensors this one runs with


@dataclass(frozen=True)
class ZubaraxConfig:
    architecture: str
    vocab: int
    width: int
    norm_eps: float
    alpha: float
    embedding_scale: float
    layers: Tuple[ZubaraxLayer, ...]
    max_positions: int
    eos_token_ids: Tuple[int, ...] = ()

    def owner(self, i: int) -> int:
        """The layer whose tensors layer ``i`` runs with."""
        j = self.layers[i].weights_of
        return i if j is None else j


def _expert(at: _At) -> ClampedExpert:
    limit = at.number("limit")
    if limit <= 0:
        raise ConfigError(f"{at.where}: '{at._name('limit')}' must be positive, got {limit!r}")
    return ClampedExpert(ff=at.integer("ff"), limit=limit)


def _layer(raw: Any, i: int, where: str) -> ZubaraxLayer:
    at = _At(raw, f"layers[{i}]", where)
    kind = at.need("type")
    if kind != "parallel":
        raise ConfigError(f"{where}: layers[{i}].type = {kind!r} is not 'parallel'")
    m = at.child("mixer")
    left, right = m.child("left"), m.child("right")
    heads, kv = left.integer("heads"), left.integer("kv_heads")
    if heads % kv:
        raise ConfigError(f"{where}: '{left._name('heads')}' = {heads} is not a multiple of kv_heads = {kv}")
    dim = left.integer("dim")
    rot = left.maybe("rot")
    rot_dims = rot.integer("dims", 0) if rot is not None else 0
    if rot_dims % 2 or rot_dims > dim:
        raise ConfigError(f"{where}: '{left._name('rot.dims')}' = {rot_dims} must be even and at most dim = {dim}")
    conv = left.integer("conv", 0) if left.obj.get("conv") is not None else 0
    mixer = ParallelMixer(
        left=TalkingSide(heads=heads, kv_heads=kv, dim=dim, vdim=left.integer("vdim"), scale=left.number("scale"), conv=conv,
                         rot_dims=rot_dims, rot_base=rot.number("base") if rot is not None and rot_dims else 1.0),
        right=ForgetGateSide(heads=right.integer("heads"), dim=right.integer("dim"), vdim=right.integer("vdim")),
        left_scale=m.number("left_scale"), right_scale=m.number("right_scale"))
    mlp_at = at.maybe("mlp")
    mlp = None
    if mlp_at is not None:
        if mlp_at.need("kind") != "moe":
            raise ConfigError(f"{where}: layers[{i}].mlp.kind = {mlp_at.obj['kind']!r} is not 'moe'")
        router = mlp_at.child("router")
        experts, top = router.integer("experts"), router.integer("top")
        if top > experts:
            raise ConfigError(f"{where}: layers[{i}].mlp.router: {top} of {experts} experts cannot be chosen")
        shared = mlp_at.maybe("shared")
        mlp = ExpertsFeedForward(expert=_expert(mlp_at.child("expert")), experts=experts, top=top,
                                 shared=_expert(shared) if shared is not None else None)
    weights_of = at.integer("weights_of", 0) if raw.get("weights_of") is not None else None
    return ZubaraxLayer(type=kind, mixer=mixer, mlp=mlp, weights_of=weights_of)


def parse_zubarax_config(obj: Dict[str, Any], where: str = "config.json") -> ZubaraxConfig:
    top = _At(obj, "", where)
    raw_layers = top.need("layers")
    if not isinstance(raw_layers, list) or not raw_layers:
        raise ConfigError(f"{where}: 'layers' must be a non-empty list")
    layers = [_layer(raw, i, where) for i, raw in enumerate(raw_layers)]
    for i, layer in enumerate(layers):
        j = layer.weights_of
        if j is None:
            continue
        if not (0 <= j < len(layers)) or j == i or layers[j].weights_of is not None:
            raise ConfigError(f"{where}: layers[{i}].weights_of = {j} must name another layer that has tensors of its own")
        if (layer.mixer, layer.mlp) != (layers[j].mixer, layers[j].mlp):
            raise ConfigError(f"{where}: layers[{i}] runs with the tensors of layers[{j}] but describes another mixer or feed-forward")
    emb = top.maybe("embedding")
    eos = obj.get("eos_token_id")
    eos_ids = tuple(eos) if isinstance(eos, list) else ((eos,) if isinstance(eos, int) else ())
    max_pos = obj.get("max_positions")
    return ZubaraxConfig(architecture=str(obj.get("architecture", ARCHITECTURE)), vocab=top.integer("vocab"), width=top.integer("width"),
                         norm_eps=top.child("norm").number("eps"), alpha=top.number("postln_alpha") if obj.get("postln_alpha") is not None else 1.0,
                         embedding_scale=emb.number("scale") if emb is not None and emb.obj.get("scale") is not None else 1.0,
                         layers=tuple(layers), max_positions=int(max_pos) if isinstance(max_pos, int) and max_pos > 0 else 1 << 20,
                         eos_token_ids=eos_ids)
