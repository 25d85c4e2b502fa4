"""Small Tupunex configurations and weights for the tests.  The tensor list is derived here from the configuration
(the names a checkpoint of the design uses), independently of the package's own list."""
import copy
import json
import os

import numpy as np


def dense(ff):
    return {"kind": "dense", "ff": ff}


def attention(heads, kv_heads, dim, vdim, scale, diff, window=None, softcap=None, conv=None, mlp=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "diff": diff}
    if window is not None:
        m["mask"] = {"size": window}
    if softcap is not None:
        m["softcap"] = softcap
    if conv is not None:
        m["conv"] = conv
    return {"type": "attention", "mixer": m, "mlp": mlp}


def latent(heads, dim, rot_dim, vdim, rank, scale, base, mlp=None):
    return {"type": "latent_attention", "mlp": mlp,
            "mixer": {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": rank, "scale": scale,
                      "rot": {"base": base, "dims": rot_dim}}}


def config(vocab, width, eps, layers, streams=None, loop=None, scale=None):
    cfg = {"architecture": "Tupunex", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}
    if streams is not None:
        cfg["streams"] = streams
    if loop is not None:
        cfg["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    if scale is not None:
        cfg["embedding"] = {"scale": scale}
    return cfg


CONFIGS = {
    # three streams, a loop over the two middle layers that runs three times, grouped heads, keys narrower than values,
    # a window that decoding passes over, a soft cap small enough to bend the scores, a layer without a feed-forward
    "A": config(101, 64, 1e-5, [
        attention(4, 2, 16, 24, 0.4, 0.3, window=23, softcap=4.0, conv=4, mlp=dense(96)),
        latent(3, 8, 12, 10, 20, 0.35, 300.0, mlp=dense(40)),
        attention(2, 1, 24, 8, 0.3, 0.6, window=50, softcap=9.0, conv=2),
        latent(2, 16, 8, 24, 48, 0.2, 10000.0, mlp=dense(72)),
    ], streams=3, loop=(1, 3, 3), scale=1.5),
    # sizes the tensor-core kernels take (keys and values of 64/64 and 32/96, a width and depths that the weight-streaming
    # products take), two streams, a loop over one layer that runs twice
    "B": config(320, 256, 1e-6, [
        latent(4, 32, 32, 64, 96, 0.125, 20000.0, mlp=dense(256)),
        attention(8, 2, 64, 64, 0.125, 0.5, window=70, softcap=30.0, conv=3, mlp=dense(256)),
        attention(4, 4, 32, 96, 0.18, 0.2, window=130, softcap=20.0, conv=4, mlp=dense(128)),
    ], streams=2, loop=(1, 2, 2), scale=2.0),
    # sizes that fit no tile: odd width, odd key and value sizes, one stream (with its own tensors), no loop, no embedding
    # scale, one head, one tap, a layer without window, cap or convolution, a window of one token, a vocabulary of 77
    "C": config(77, 54, 1e-6, [
        attention(3, 3, 10, 7, 0.33, 0.0, window=1, conv=1, mlp=dense(33)),
        latent(1, 6, 10, 9, 14, 0.5, 50.0, mlp=dense(17)),
        attention(6, 2, 9, 11, 0.3, 0.8, mlp=dense(33)),
        latent(5, 7, 2, 3, 9, 0.41, 7.0),
        attention(1, 1, 12, 5, 0.25, 0.45, window=300, softcap=2.5, conv=8, mlp=dense(20)),
    ], streams=1),
    # no streams at all (the ordinary residual sum with a scale per channel), every layer inside a loop that runs twice
    "D": config(90, 48, 1e-5, [
        attention(2, 1, 8, 16, 0.35, 0.5, window=17, softcap=6.0, conv=3, mlp=dense(64)),
        latent(2, 8, 4, 8, 16, 0.3, 100.0, mlp=dense(32)),
    ], loop=(0, 2, 2)),
}
LENGTHS = {"A": [1, 9, 77, 300], "B": [5, 70, 280], "C": [2, 33, 150, 270], "D": [3, 40, 290]}


def layer_order(cfg):
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return list(range(n))
    return list(range(loop["start"])) + list(range(loop["start"], loop["stop"])) * loop["times"] + list(range(loop["stop"], n))


def tensor_shapes(cfg):
    d, v, S = cfg["width"], cfg["vocab"], cfg.get("streams")
    out = {"embed": (v, d), "final.norm": (d,), "head": (v, d)}
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        subs = [1] + ([2] if layer["mlp"] is not None else [])
        for q in subs:
            out[p + f"norm{q}"] = (d,)
            out[p + f"ls{q}"] = (d,)
            if S:
                out.update({p + f"hc{q}.in": (S,), p + f"hc{q}.out": (S,), p + f"hc{q}.mix": (S, S)})
        if layer["type"] == "attention":
            H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            rows = {"q": H * 2 * dk, "k": G * 2 * dk, "v": G * dv}
            for n, r in rows.items():
                out[p + "mix." + n] = (r, d)
                out[p + "mix." + n + ".b"] = (r,)
                if m.get("conv"):
                    out[p + "mix." + n + ".conv"] = (r, m["conv"])
            out.update({p + "mix.lq1": (dk,), p + "mix.lk1": (dk,), p + "mix.lq2": (dk,), p + "mix.lk2": (dk,), p + "mix.g": (H, d),
                        p + "mix.o": (d, H * dv)})
        else:
            H, dk, dr, dv, r = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
            out.update({p + "mix.q": (H * (dk + dr), d), p + "mix.dkv": (r + dr, d), p + "mix.dkv.norm": (r,), p + "mix.uk": (H * dk, r),
                        p + "mix.uv": (H * dv, r), p + "mix.g": (H, d), p + "mix.o": (d, H * dv)})
        if layer["mlp"] is not None:
            f = layer["mlp"]["ff"]
            out.update({p + "mlp.gate": (f, d), p + "mlp.up": (f, d), p + "mlp.down": (d, f)})
    return out


def random_weights(cfg, seed, gain=1.0):
    """Weights large enough that every mechanism moves the logits: matrices ~ N(0, gain / sqrt(in)); norm weights and
    per-channel scales ~ 1 + 0.1 N; how the streams are read ~ 1/S + 0.2 N, carried on ~ I + 0.2 N, written ~ 1 + 0.2 N;
    taps ~ 0.5 N; biases ~ 0.2 N; the vectors behind lambda ~ 0.3 N; q and k three times as large, so that scores are spread
    and the soft cap bends them."""
    rng = np.random.RandomState(seed)
    S = cfg.get("streams") or 1
    out = {}
    for name, shape in tensor_shapes(cfg).items():
        parts = name.split(".")
        leaf = parts[-1]
        if leaf in ("norm1", "norm2", "ls1", "ls2", "norm") or name == "final.norm":
            w = 1.0 + 0.1 * rng.randn(*shape)
        elif leaf == "in" and "hc" in parts[-2]:
            w = 1.0 / S + 0.2 * rng.randn(*shape)
        elif leaf == "mix" and "hc" in parts[-2]:
            w = np.eye(S) + 0.2 * rng.randn(*shape)
        elif leaf == "out" and "hc" in parts[-2]:
            w = 1.0 + 0.2 * rng.randn(*shape)
        elif leaf == "conv":
            w = 0.5 * rng.randn(*shape)
        elif leaf == "b":
            w = 0.2 * rng.randn(*shape)
        elif leaf in ("lq1", "lk1", "lq2", "lk2"):
            w = 0.3 * rng.randn(*shape)
        elif name == "embed":
            w = rng.randn(*shape)
        elif leaf in ("q", "k") and len(shape) == 2:
            w = rng.randn(*shape) * 3.0 * gain / np.sqrt(shape[1])
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
        json.dump(copy.deepcopy(cfg), f)
    write_safetensors(os.path.join(folder, "model.safetensors"), {k: torch.from_numpy(np.asarray(v)).to(torch.bfloat16) for k, v in w.items()})
    return folder
