"""Plain, slow implementation of the Zubarax decoder in numpy float64: whole sequences, no cache, one function per
mechanism.  It is the oracle of the Zubarax tests and shares no code with the package.

Notation: ``T`` tokens, width ``D``; a linear map stored ``[out, in]`` is applied as ``x @ W.T``.
"""
from __future__ import annotations

import json
import math
import os
import struct
from typing import Dict, List, Optional

import numpy as np


# ---- container --------------------------------------------------------------------------------------------------
def read_safetensors(path: str) -> Dict[str, np.ndarray]:
    with open(path, "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        header = json.loads(f.read(n).decode("utf-8"))
        data = f.read()
    out = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        lo, hi = info["data_offsets"]
        raw, shape, dt = data[lo:hi], tuple(info["shape"]), info["dtype"]
        if dt == "BF16":
            u = np.frombuffer(raw, dtype="<u2").astype(np.uint32) << 16
            out[name] = u.view(np.float32).astype(np.float64).reshape(shape)
        elif dt == "F32":
            out[name] = np.frombuffer(raw, dtype="<f4").astype(np.float64).reshape(shape)
        elif dt == "I32":
            out[name] = np.frombuffer(raw, dtype="<i4").astype(np.int64).reshape(shape)
        else:
            raise ValueError(f"dtype {dt} of '{name}' is not read by the oracle")
    return out


def load_folder(folder: str):
    with open(os.path.join(folder, "config.json")) as f:
        cfg = json.load(f)
    return cfg, read_safetensors(os.path.join(folder, "model.safetensors"))


# ---- small functions ----------------------------------------------------------------------------------------------
def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def rms(x, eps):
    """x divided by its root mean square over the last axis, eps inside the root."""
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def norm_one_plus(x, w, eps):
    return rms(x, eps) * (1.0 + w)


# ---- mechanisms ---------------------------------------------------------------------------------------------------
def short_conv(u, taps):
    """u [T, C], taps [C, K]: y_t = sum_j taps[:, j] * u_(t - K + 1 + j), zeros before the start."""
    T, C = u.shape
    K = taps.shape[1]
    padded = np.concatenate([np.zeros((K - 1, C)), u], axis=0)
    y = np.zeros_like(u)
    for j in range(K):
        y += padded[j:j + T] * taps[:, j][None, :]
    return y


def rotate_half(x, positions, dims, base):
    """x [T, heads, d]: the first ``dims`` numbers of a head turn by position; number i pairs with i + dims/2."""
    if not dims:
        return x
    half = dims // 2
    freq = np.array([base ** (-2.0 * i / dims) for i in range(half)])
    ang = np.asarray(positions, dtype=np.float64)[:, None] * freq[None, :]           # [T, half]
    c, s = np.cos(ang)[:, None, :], np.sin(ang)[:, None, :]
    out = x.copy()
    a, b = x[..., :half], x[..., half:dims]
    out[..., :half] = a * c - b * s
    out[..., half:dims] = b * c + a * s
    return out


def talking_sink_attention_core(q, k, v, talk, sink, scale):
    """q [T, H, dk], k [T, G, dk], v [T, G, dv]; the scaled scores of all heads of one (query, key) pair are mixed by
    ``talk`` [H, H] before the softmax; causal; every head's denominator also holds exp(sink_h).  Returns [T, H, dv]."""
    T, H, _ = q.shape
    G = k.shape[1]
    rep = H // G
    raw = np.zeros((H, T, T))
    for h in range(H):
        raw[h] = (q[:, h, :] @ k[:, h // rep, :].T) * scale
    mixed = np.einsum("hg,gij->hij", talk, raw)
    out = np.zeros((T, H, v.shape[2]))
    for h in range(H):
        for i in range(T):
            s = mixed[h, i, :i + 1]
            m = max(float(s.max()), float(sink[h]))
            e = np.exp(s - m)
            den = e.sum() + math.exp(float(sink[h]) - m)
            out[i, h] = (e / den) @ v[:i + 1, h // rep, :]
    return out


def talking_attention(h, w, prefix, m, eps, positions):
    """The left side: projections, short convolutions, q/k norm, rotation, unit values, mixed scores, sink, output."""
    T = h.shape[0]
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q, k, v = h @ w[prefix + "q"].T, h @ w[prefix + "k"].T, h @ w[prefix + "v"].T
    if m.get("conv"):
        q, k, v = (short_conv(t, w[prefix + n + ".conv"]) for t, n in ((q, "q"), (k, "k"), (v, "v")))
    q, k, v = q.reshape(T, H, dk), k.reshape(T, G, dk), v.reshape(T, G, dv)
    q = rms(q, eps) * w[prefix + "q.norm"]
    k = rms(k, eps) * w[prefix + "k.norm"]
    rot = m.get("rot")
    if rot and rot.get("dims"):
        q = rotate_half(q, positions, rot["dims"], rot["base"])
        k = rotate_half(k, positions, rot["dims"], rot["base"])
    v = rms(v, eps)
    o = talking_sink_attention_core(q, k, v, w[prefix + "talk"], w[prefix + "sink"], m["scale"])
    return o.reshape(T, H * dv) @ w[prefix + "o"].T


def hgrn2_core(q, f, v):
    """q, f [T, H, dk], v [T, H, dv]: S_t = diag(f_t) S_(t-1) + (1 - f_t) v_t^T, o_t = S_t^T q_t, from S = 0."""
    T, H, dk = q.shape
    dv = v.shape[2]
    S = np.zeros((H, dk, dv))
    o = np.zeros((T, H, dv))
    for t in range(T):
        S = f[t][:, :, None] * S + (1.0 - f[t])[:, :, None] * v[t][:, None, :]
        o[t] = np.einsum("hkv,hk->hv", S, q[t])
    return o


def hgrn2(h, w, prefix, m, eps):
    T = h.shape[0]
    H, dk, dv = m["heads"], m["dim"], m["vdim"]
    q = silu(h @ w[prefix + "q"].T).reshape(T, H, dk)
    v = (h @ w[prefix + "v"].T).reshape(T, H, dv)
    low = w[prefix + "lower"]
    f = (low + (1.0 - low) * sigmoid(h @ w[prefix + "f"].T + w[prefix + "f.b"])).reshape(T, H, dk)
    o = hgrn2_core(q, f, v)
    o = rms(o, eps) * w[prefix + "norm"]
    return o.reshape(T, H * dv) @ w[prefix + "o"].T


def parallel_mixer(h, w, prefix, m, eps, positions):
    left = talking_attention(h, w, prefix + "left.", m["left"], eps, positions)
    right = hgrn2(h, w, prefix + "right.", m["right"], eps)
    return m["left_scale"] * left + m["right_scale"] * right


def clamped_expert(h, w, stem, limit):
    g = np.minimum(h @ w[stem + ".gate"].T, limit)
    u = np.clip(h @ w[stem + ".up"].T, -limit, limit)
    return (g * sigmoid(1.702 * g) * (u + 1.0)) @ w[stem + ".down"].T


def router_choice(h, w_router, top):
    """Sigmoid scores; the ``top`` largest (lowest index first on ties); returns indices [T, top] and their scores."""
    s = sigmoid(h @ w_router.T)
    idx = np.argsort(-s, axis=-1, kind="stable")[:, :top]
    return idx, np.take_along_axis(s, idx, axis=-1)


def experts_feed_forward(h, w, prefix, f):
    """Sum over the chosen experts of expert(score * h), plus a shared expert on h itself."""
    idx, wts = router_choice(h, w[prefix + "router"], f["router"]["top"])
    out = np.zeros((h.shape[0], w[prefix + "e0.down"].shape[0]))
    for t in range(h.shape[0]):
        for e, s in zip(idx[t], wts[t]):
            out[t] += clamped_expert(s * h[t:t + 1], w, prefix + f"e{int(e)}", f["expert"]["limit"])[0]
    if f.get("shared"):
        out += clamped_expert(h, w, prefix + "shared", f["shared"]["limit"])
    return out


# ---- the model ----------------------------------------------------------------------------------------------------
def forward(cfg, w, tokens, positions=None, collect: Optional[List[np.ndarray]] = None):
    """Logits [T, vocab] of one sequence; ``collect`` receives the stream after every layer run."""
    eps, alpha = cfg["norm"]["eps"], cfg.get("postln_alpha", 1.0)
    T = len(tokens)
    positions = list(range(T)) if positions is None else positions
    x = w["embed"][np.asarray(tokens)] * cfg.get("embedding", {}).get("scale", 1.0)
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{layer.get('weights_of', i) if layer.get('weights_of') is not None else i}."
        if layer["type"] != "parallel":
            raise ValueError(f"layer type {layer['type']!r}")
        x = norm_one_plus(alpha * x + parallel_mixer(x, w, p + "mix.", layer["mixer"], eps, positions), w[p + "norm1"], eps)
        if layer.get("mlp") is not None:
            x = norm_one_plus(alpha * x + experts_feed_forward(x, w, p + "mlp.", layer["mlp"]), w[p + "norm2"], eps)
        if collect is not None:
            collect.append(x.copy())
    x = norm_one_plus(x, w["final.norm"], eps)
    return x @ w["embed"].T
