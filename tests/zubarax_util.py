"""Small Zubarax configurations and weights for the tests.  The tensor list is derived here from the configuration
(the names a checkpoint of the design uses), independently of the package's own list."""
import copy
import json
import os

import numpy as np


def moe(ff, limit, experts, top, shared=None):
    out = {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": {"experts": experts, "top": top}}
    if shared:
        out["shared"] = {"ff": shared[0], "limit": shared[1]}
    return out


def parallel(left, right, scales, mlp=None):
    """left: (heads, kv_heads, dim, vdim, scale, conv or None, rot (dims, base) or None); right: (heads, dim, vdim)"""
    H, G, dk, dv, scale, conv, rot = left
    L = {"heads": H, "kv_heads": G, "dim": dk, "vdim": dv, "scale": scale}
    if conv is not None:
        L["conv"] = conv
    if rot is not None:
        L["rot"] = {"dims": rot[0], "base": rot[1]}
    return {"type": "parallel", "mlp": mlp,
            "mixer": {"left": L, "right": {"heads": right[0], "dim": right[1], "vdim": right[2]}, "left_scale": scales[0], "right_scale": scales[1]}}


def again(layers, j):
    """A layer that runs with layer j's tensors: its entry repeats layer j's."""
    out = copy.deepcopy(layers[j])
    out["weights_of"] = j
    return out


def config(vocab, width, eps, alpha, emb_scale, layers):
    out = {"architecture": "Zubarax", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}
    if alpha is not None:
        out["postln_alpha"] = alpha
    if emb_scale is not None:
        out["embedding"] = {"scale": emb_scale}
    return out


def _with_repeats(layers, order):
    """order: for every layer of the model an index into ``layers`` (a first mention owns the tensors) -> the config's list."""
    out, first = [], {}
    for idx in order:
        if idx in first:
            out.append(again(out, first[idx]))
        else:
            first[idx] = len(out)
            out.append(layers[idx])
    return out


CONFIGS = {
    # grouped heads, keys wider and narrower than values, part of the head rotated, three and four taps, two experts of six
    # with a shared one, a layer without a feed-forward, without convolution and without rotation, layers run twice in
    # another order than they stand
    "A": config(101, 64, 1e-5, 2.0, 4.0, _with_repeats([
        parallel((4, 2, 24, 16, 0.2, 3, (12, 100.0)), (3, 16, 8), (0.7, 1.2), moe(40, 1.5, 6, 2, (24, 0.8))),
        parallel((2, 1, 16, 40, 0.25, 4, (16, 10000.0)), (2, 8, 16), (1.0, 0.5), moe(24, 1.0, 4, 1)),
        parallel((3, 3, 10, 7, 0.3, None, None), (1, 10, 12), (1.3, 1.0)),
    ], [0, 1, 0, 2, 1])),
    # sizes that tensor-core kernels take (key sizes 64 and 96, depths that are multiples of 8), three experts of eight
    "B": config(320, 256, 1e-6, 3.0, 8.0, _with_repeats([
        parallel((8, 2, 64, 64, 0.125, 4, (32, 1000000.0)), (4, 64, 32), (0.8, 1.1), moe(64, 2.0, 8, 3, (128, 1.0))),
        parallel((4, 4, 96, 32, 0.1, 2, (96, 500.0)), (2, 32, 64), (1.0, 1.0), moe(64, 1.0, 8, 3)),
    ], [0, 1, 1, 0])),
    # sizes that fit no tile: odd width, odd key and value sizes, one tap, every expert chosen, one head, no alpha and no
    # embedding scale in the file, a vocabulary of 77
    "C": config(77, 54, 1e-6, None, None, _with_repeats([
        parallel((5, 5, 9, 7, 0.33, 2, (4, 50.0)), (3, 10, 5), (0.9, 0.9), moe(33, 0.7, 5, 5, (17, 3.0))),
        parallel((6, 2, 10, 12, 0.3, 1, None), (1, 12, 6), (1.0, 2.0), moe(17, 1.0, 3, 1)),
    ], [0, 0, 1])),
    # a wider model whose attention sizes the tensor-core kernel takes in its other forms: twelve heads of wide values (a head
    # per warp), a key size that is an odd multiple of 16, three heads over one key head, part of a head rotated, values wider
    # than keys
    "D": config(1000, 384, 1e-5, 2.5, 12.0, _with_repeats([
        parallel((12, 4, 80, 96, 0.11, 4, (40, 500000.0)), (3, 48, 80), (0.8, 1.1), moe(160, 1.0, 6, 2, (96, 1.0))),
        parallel((3, 1, 144, 32, 0.08, 3, (144, 10000.0)), (2, 64, 64), (1.0, 0.7), moe(64, 2.0, 4, 1)),
        parallel((8, 8, 32, 128, 0.18, 2, (16, 1000.0)), (4, 32, 32), (1.2, 1.0), moe(96, 1.5, 5, 3, (64, 0.5))),
    ], [0, 1, 2, 0, 1, 2])),
}
LENGTHS = {"A": [1, 9, 77, 300], "B": [5, 70, 280], "C": [2, 33, 150, 270], "D": [3, 120, 333]}


def every_expert_chosen(cfg):
    """The same model with ``top = experts`` in every feed-forward: the choice of experts cannot flip on a near tie, and the
    weights move smoothly with the scores."""
    out = copy.deepcopy(cfg)
    for layer in out["layers"]:
        if layer["mlp"] is not None:
            layer["mlp"]["router"]["top"] = layer["mlp"]["router"]["experts"]
    return out


def tensor_shapes(cfg):
    d, v = cfg["width"], cfg["vocab"]
    out = {"embed": (v, d), "final.norm": (d,)}
    for i, layer in enumerate(cfg["layers"]):
        if layer.get("weights_of") is not None:
            continue
        p, m = f"l{i}.", layer["mixer"]
        out[p + "norm1"] = (d,)
        L, R = m["left"], m["right"]
        H, G, dk, dv = L["heads"], L["kv_heads"], L["dim"], L["vdim"]
        out.update({p + "mix.left.q": (H * dk, d), p + "mix.left.k": (G * dk, d), p + "mix.left.v": (G * dv, d),
                    p + "mix.left.q.norm": (dk,), p + "mix.left.k.norm": (dk,), p + "mix.left.talk": (H, H), p + "mix.left.sink": (H,),
                    p + "mix.left.o": (d, H * dv)})
        if L.get("conv"):
            out.update({p + "mix.left.q.conv": (H * dk, L["conv"]), p + "mix.left.k.conv": (G * dk, L["conv"]), p + "mix.left.v.conv": (G * dv, L["conv"])})
        H, dk, dv = R["heads"], R["dim"], R["vdim"]
        out.update({p + "mix.right.q": (H * dk, d), p + "mix.right.f": (H * dk, d), p + "mix.right.f.b": (H * dk,), p + "mix.right.lower": (H * dk,),
                    p + "mix.right.v": (H * dv, d), p + "mix.right.norm": (dv,), p + "mix.right.o": (d, H * dv)})
        if layer["mlp"] is not None:
            f, E = layer["mlp"]["expert"]["ff"], layer["mlp"]["router"]["experts"]
            out[p + "norm2"] = (d,)
            out[p + "mlp.router"] = (E, d)
            for e in range(E):
                out.update({p + f"mlp.e{e}.gate": (f, d), p + f"mlp.e{e}.up": (f, d), p + f"mlp.e{e}.down": (d, f)})
            if layer["mlp"].get("shared"):
                f = layer["mlp"]["shared"]["ff"]
                out.update({p + "mlp.shared.gate": (f, d), p + "mlp.shared.up": (f, d), p + "mlp.shared.down": (d, f)})
    return out


def random_weights(cfg, seed, gain=1.0):
    """Weights large enough that every mechanism moves the logits: matrices ~ N(0, gain / sqrt(in)); the norms stored
    around zero ~ 0.1 N; the plain norm weights ~ 1 + 0.1 N; sinks and forget biases ~ N(0, 1); lower bounds inside (0, 1);
    the head-mixing matrix near the identity; taps ~ 0.5 N; the router spread wide, so that a choice of experts is seldom a
    near tie."""
    rng = np.random.RandomState(seed)
    out = {}
    for name, shape in tensor_shapes(cfg).items():
        leaf = name.split(".")[-1]
        if leaf in ("norm1", "norm2") or name == "final.norm":
            w = 0.1 * rng.randn(*shape)
        elif leaf == "norm":
            w = 1.0 + 0.1 * rng.randn(*shape)
        elif leaf in ("sink", "b"):
            w = rng.randn(*shape)
        elif leaf == "lower":
            w = 1.0 / (1.0 + np.exp(-rng.randn(*shape)))
        elif leaf == "talk":
            w = np.eye(shape[0]) + 0.3 * rng.randn(*shape)
        elif leaf == "conv":
            w = 0.5 * rng.randn(*shape)
        elif leaf == "router":
            w = rng.randn(*shape) * 4.0 / np.sqrt(shape[1])
        elif name == "embed":
            w = rng.randn(*shape) / np.sqrt(cfg.get("embedding", {}).get("scale", 1.0))
        else:
            w = rng.randn(*shape) * gain / np.sqrt(shape[1])
        out[name] = w.astype(np.float32)
    return out


def write_model(folder, cfg, seed, gain=1.0, overrides=None):
    """config.json + model.safetensors (bfloat16) in ``folder``."""
    import torch
    from mimirmind_b200.weights.safetensors_io import write_safetensors
    w = random_weights(cfg, seed, gain)
    w.update(overrides or {})
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f)
    write_safetensors(os.path.join(folder, "model.safetensors"), {k: torch.from_numpy(np.asarray(v)).to(torch.bfloat16) for k, v in w.items()})
    return folder
