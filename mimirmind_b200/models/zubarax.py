"""Zubarax: a decoder with the norm after the sum, whose layers run two mixers side by side and a mixture of experts.

A layer: ``x <- norm1(alpha x + mixer(x))``, ``x <- norm2(alpha x + experts(x))``; the sublayers read the stream itself, both
norms are RMS norms whose weight is stored around zero (``1 + w`` multiplies).  The mixer, of the layer's ``type``
``parallel``, is ``left_scale * left + right_scale * right`` over the same input:

* left: causal softmax attention with grouped heads: a short causal convolution on every channel of q, k and v, an RMS norm
  per head on q and k (one weight for all heads), rotation of the first ``rot.dims`` numbers of every head (half-split
  pairs), values divided by their root mean square per head, the heads' scaled scores mixed by a learned matrix before
  the softmax, and a learned sink per head;
* right: HGRN2, a matrix state per head with a forget gate per key channel (above a learned lower bound) whose complement is the
  strength of the write; silu on q, an RMS norm per head with one weight for all heads.

Feed-forward: routed experts with sigmoid scores that are not renormed and multiply the expert's *input*, experts of the
clamped form ``g sigmoid(1.702 g) (u + 1)``, and one more such expert that no router gates.  A layer may run with
another layer's tensors (``weights_of``): it is then a schedule entry of that layer, with a cache and state of its own.
The embedding is scaled; the head is the embedding table itself.
Tensor names: ``embed``, ``l<i>.norm1|norm2``, ``l<i>.mix.left.*``, ``l<i>.mix.right.*``, ``l<i>.mlp.*``, ``final.norm``.

This module only *describes* the model; it holds no arithmetic.
"""
from __future__ import annotations

from ..config.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry
from ..config.zubarax_config import ARCHITECTURE, ClampedExpert, ZubaraxConfig, parse_zubarax_config
from ..registry import register_architecture


def _shared(d: int, e: ClampedExpert) -> PartSpec:
    return PartSpec("gated_mlp", {"hidden": d, "intermediate": e.ff, "activation": "clamped", "limit": e.limit,
                                  "gate": "mlp.shared.gate", "up": "mlp.shared.up", "down": "mlp.shared.down"})


def build_spec(cfg: ZubaraxConfig) -> ModelSpec:
    d, eps = cfg.width, cfg.norm_eps

    def norm(name: str) -> PartSpec:
        return PartSpec("rmsnorm", {"width": d, "eps": eps, "weight": name, "offset": 1.0}, category="norm")

    layers, index = [], {}            # index: the config's layer number -> its place among the layers that own tensors
    for i, layer in enumerate(cfg.layers):
        if layer.weights_of is not None:
            continue
        L, R = layer.mixer.left, layer.mixer.right
        left = PartSpec("talking_attention", {
            "hidden": d, "heads": L.heads, "kv_heads": L.kv_heads, "key_dim": L.dim, "value_dim": L.vdim, "window": 0, "scale": L.scale,
            "eps": eps, "conv": L.conv, "conv_suffix": ".conv", "qk_norm": True, "q_norm": "mix.left.q.norm", "k_norm": "mix.left.k.norm",
            "rotary": {"dims": L.rot_dims, "base": L.rot_base} if L.rot_dims else None, "v_unit": True, "talk": "mix.left.talk",
            "sink": "mix.left.sink", "q": "mix.left.q", "k": "mix.left.k", "v": "mix.left.v", "o": "mix.left.o"})
        right = PartSpec("linear_state", {
            "hidden": d, "heads": R.heads, "qk_heads": R.heads, "key_dim": R.dim, "value_dim": R.vdim, "eps": eps, "decay": "forget_gate",
            "f_bias": "mix.right.f.b", "lower": "mix.right.lower", "delta": None, "conv": 0, "activation": "silu", "rotary": None,
            "unit_eps": None, "out_norm": "head", "out_weight": "mix.right.norm", "g": None,
            "q": "mix.right.q", "k": "mix.right.f", "v": "mix.right.v", "o": "mix.right.o"})
        mixer = PartSpec("parallel_mixers", {"hidden": d, "combine": "sum", "left": left, "right": right,
                                             "left_scale": layer.mixer.left_scale, "right_scale": layer.mixer.right_scale})
        extras = {}
        if layer.mlp is not None:
            f = layer.mlp
            ffn = PartSpec("routed_experts", {
                "hidden": d, "ff": f.expert.ff, "experts": f.experts, "top": f.top, "groups": 1, "keep": 1, "router": "mlp.router",
                "expert": "mlp.e{}", "scoring": "sigmoid", "weight_on": "input", "activation": "clamped", "limit": f.expert.limit,
                "shared": _shared(d, f.shared) if f.shared is not None else None})
            ffn_norm = norm("norm2")
        else:
            ffn, ffn_norm = PartSpec("none", {}), PartSpec("none", {})
            extras["unused"] = PartSpec("unused_sublayer", {"tensors": [("norm2", (d,))]}, category="connection")
        index[i] = len(layers)
        layers.append(LayerSpec(prefix=f"l{i}.", block=PartSpec("post_norm", {"alpha": cfg.alpha}), mixer=mixer, feed_forward=ffn,
                                mixer_norm=norm("norm1"), ffn_norm=ffn_norm, extras=extras))
    return ModelSpec(
        architecture=cfg.architecture, hidden_size=d, vocab_size=cfg.vocab, max_positions=cfg.max_positions,
        embedding=PartSpec("token_embedding", {"vocab": cfg.vocab, "width": d, "scale": cfg.embedding_scale, "weight": "embed"}),
        layers=tuple(layers), schedule=tuple(ScheduleEntry(index[cfg.owner(i)]) for i in range(len(cfg.layers))),
        final_norm=norm("final.norm"),
        head=PartSpec("lm_head", {"vocab": cfg.vocab, "width": d, "weight": "head", "tied_to": "embed"}),
        eos_token_ids=cfg.eos_token_ids)


register_architecture(ARCHITECTURE, parse_zubarax_config, build_spec)
