"""Tupunex: a decoder over several copies of the residual stream whose layers mix two kinds of attention, laid out from parts.

A layer is two pre-norm sublayers, a mixer and a gated feed-forward, each reading the residual streams through a
connection of its own and writing back through it (``parts/connections.py``; every result is scaled per channel first).
Mixers, by the layer's ``type``:

* ``attention``: differential attention over a sliding window: a short causal convolution on every channel of q, k and
  v, two softmax maps per head over the same values with capped scores, the second map taken off the first ``lambda``
  times, each head divided by its root mean square, a sigmoid gate per head.  No position encoding.
* ``latent_attention``: causal attention whose keys and values are made from one normed latent vector per token, with
  one rotated key part shared by all heads; only the latent and that part are cached; a sigmoid gate per head.

``loop`` lets a run of consecutive layers execute several times in a row with the same weights; every pass is a schedule
entry of its own and so has its own cache and state.  Then the final norm over the sum of the streams, and the head.
Tensor names: ``embed``, ``l<i>.norm1|norm2``, ``l<i>.ls1|ls2``, ``l<i>.hc1|hc2.in|mix|out``, ``l<i>.mix.*``, ``l<i>.mlp.*``,
``final.norm``, ``head``.

This module only *describes* the model; it holds no arithmetic.
"""
from __future__ import annotations

from ..config.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry
from ..config.tupunex_config import ARCHITECTURE, TupunexConfig, parse_tupunex_config
from ..registry import register_architecture


def build_spec(cfg: TupunexConfig) -> ModelSpec:
    d, eps, S = cfg.width, cfg.norm_eps, cfg.streams

    def norm(name: str, streams: int = 1) -> PartSpec:
        return PartSpec("rmsnorm", {"width": d, "eps": eps, "weight": name, "streams": streams}, category="norm")

    def connection(q: int) -> PartSpec:
        return PartSpec("hyper_connection", {"width": d, "streams": S, "read": f"hc{q}.in", "mix": f"hc{q}.mix", "write": f"hc{q}.out",
                                             "scale": f"ls{q}"}, category="connection")

    layers = []
    for i, layer in enumerate(cfg.layers):
        m = layer.mixer
        if layer.type == "attention":
            mixer = PartSpec("differential_attention", {
                "hidden": d, "heads": m.heads, "kv_heads": m.kv_heads, "key_dim": m.dim, "value_dim": m.vdim, "window": m.window,
                "scale": m.scale, "softcap": m.softcap, "diff": m.diff, "eps": eps, "conv": m.conv, "conv_suffix": ".conv",
                "bias": True, "bias_suffix": ".b", "q": "mix.q", "k": "mix.k", "v": "mix.v", "g": "mix.g", "o": "mix.o",
                "lq1": "mix.lq1", "lk1": "mix.lk1", "lq2": "mix.lq2", "lk2": "mix.lk2"})
        else:
            mixer = PartSpec("latent_attention", {
                "hidden": d, "heads": m.heads, "key_dim": m.dim, "rot_dim": m.rot_dim, "value_dim": m.vdim, "rank": m.kv_rank,
                "scale": m.scale, "eps": eps, "rotary": {"dims": m.rot_dims, "base": m.rot_base} if m.rot_dims else None,
                "q": "mix.q", "down": "mix.dkv", "down_norm": "mix.dkv.norm", "up_k": "mix.uk", "up_v": "mix.uv", "g": "mix.g", "o": "mix.o"})
        extras = {"mixer_connection": connection(1)}
        if layer.mlp is not None:
            ffn = PartSpec("swiglu", {"hidden": d, "intermediate": layer.mlp.ff, "gate": "mlp.gate", "up": "mlp.up", "down": "mlp.down"})
            ffn_norm = norm("norm2")
            extras["ffn_connection"] = connection(2)
        else:
            ffn, ffn_norm = PartSpec("none", {}), PartSpec("none", {})
            spare = [("norm2", (d,)), ("ls2", (d,))] + ([("hc2.in", (S,)), ("hc2.out", (S,)), ("hc2.mix", (S, S))] if S else [])
            extras["unused"] = PartSpec("unused_sublayer", {"tensors": spare}, category="connection")
        layers.append(LayerSpec(prefix=f"l{i}.", block=PartSpec("stream_connections", {}), mixer=mixer, feed_forward=ffn,
                                mixer_norm=norm("norm1"), ffn_norm=ffn_norm, extras=extras))
    return ModelSpec(
        architecture=cfg.architecture, hidden_size=d, vocab_size=cfg.vocab, max_positions=cfg.max_positions,
        embedding=PartSpec("token_embedding", {"vocab": cfg.vocab, "width": d, "scale": cfg.embedding_scale, "weight": "embed",
                                               "copies": max(1, S)}),
        layers=tuple(layers), schedule=tuple(ScheduleEntry(i) for i in cfg.order()),
        final_norm=norm("final.norm", max(1, S)),
        head=PartSpec("lm_head", {"vocab": cfg.vocab, "width": d, "weight": "head", "tied_to": None}),
        eos_token_ids=cfg.eos_token_ids)


register_architecture(ARCHITECTURE, parse_tupunex_config, build_spec)
