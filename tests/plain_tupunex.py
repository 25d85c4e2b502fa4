"""Plain, slow implementation of the Tupunex decoder in numpy float64: whole sequences, no cache, one function per
mechanism.  It is the oracle of the Tupunex tests and shares no code with the package.

Notation: ``T`` tokens, width ``D``; a linear map stored ``[out, in]`` is applied as ``x @ W.T``.
"""
from __future__ import annotations

import json
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


def rms_norm(x, w, eps):
    return rms(x, eps) * w


def softmax_rows(s, visible):
    """Softmax over the last axis of ``s`` restricted to ``visible`` (same shape, bool); a row sees at least one key."""
    s = np.where(visible, s, -np.inf)
    e = np.exp(s - s.max(axis=-1, keepdims=True))
    return e / e.sum(axis=-1, keepdims=True)


# ---- mechanisms ---------------------------------------------------------------------------------------------------
def causal_conv(u, taps):
    """u [T, C], taps [C, K]: y_t = sum_j taps[:, j] * u_(t - K + 1 + j), zeros before the sequence."""
    T, C = u.shape
    K = taps.shape[1]
    padded = np.concatenate([np.zeros((K - 1, C)), u], axis=0)
    y = np.zeros((T, C))
    for j in range(K):
        y += padded[j:j + T] * taps[:, j][None, :]
    return y


def soft_cap(s, cap):
    return cap * np.tanh(s / cap)


def window_visible(T: int, window: int):
    """[T, T] bool: query i sees key j with 0 <= i - j < window (window 0: every j <= i)."""
    i = np.arange(T)[:, None]
    j = np.arange(T)[None, :]
    vis = j <= i
    if window:
        vis &= (i - j) < window
    return vis


def differential_lambda(lq1, lk1, lq2, lk2, diff):
    return float(np.exp(np.sum(lq1 * lk1)) - np.exp(np.sum(lq2 * lk2)) + diff)


def differential_attention_core(q, k, v, scale, cap, window, lam, diff, eps):
    """q [T, H, 2, dk], k [T, G, 2, dk], v [T, G, dv]: two softmax maps per head over the same values, the second taken
    off the first ``lam`` times; each head's result divided by its root mean square and scaled by ``1 - diff``.
    Returns [T, H, dv]."""
    T, H = q.shape[0], q.shape[1]
    G, dv = k.shape[1], v.shape[2]
    vis = window_visible(T, window)
    out = np.zeros((T, H, dv))
    for h in range(H):
        g = h // (H // G)
        maps = []
        for m in range(2):
            s = (q[:, h, m, :] @ k[:, g, m, :].T) * scale
            if cap:
                s = soft_cap(s, cap)
            maps.append(softmax_rows(s, vis) @ v[:, g, :])
        o = maps[0] - lam * maps[1]
        out[:, h, :] = rms(o, eps) * (1.0 - diff)
    return out


def differential_attention(h, w: Dict[str, np.ndarray], m: dict, eps: float):
    """The mixer of an ``attention`` layer: projections with biases, a short convolution over time on every channel of
    q, k and v, two maps per head, a sigmoid gate per head, the output projection."""
    T = h.shape[0]
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    proj = {}
    for name in ("q", "k", "v"):
        u = h @ w[name].T
        if name + ".b" in w:
            u = u + w[name + ".b"]
        if m.get("conv"):
            u = causal_conv(u, w[name + ".conv"])
        proj[name] = u
    q = proj["q"].reshape(T, H, 2, dk)
    k = proj["k"].reshape(T, G, 2, dk)
    v = proj["v"].reshape(T, G, dv)
    lam = differential_lambda(w["lq1"], w["lk1"], w["lq2"], w["lk2"], m["diff"])
    window = (m.get("mask") or {}).get("size", 0)
    o = differential_attention_core(q, k, v, m["scale"], m.get("softcap", 0.0), window, lam, m["diff"], eps)
    gate = sigmoid(h @ w["g"].T)                                  # [T, H]
    o = o * gate[:, :, None]
    return o.reshape(T, H * dv) @ w["o"].T


def rotate_half(x, positions, dims, base):
    """x [T, ..., d]: the first ``dims`` dimensions turn, dimension i paired with i + dims/2, by position * base^(-2i/dims)."""
    half = dims // 2
    f = base ** (-2.0 * np.arange(half) / dims)
    a = positions[:, None] * f[None, :]                           # [T, half]
    shape = (x.shape[0],) + (1,) * (x.ndim - 2) + (half,)
    c, s = np.cos(a).reshape(shape), np.sin(a).reshape(shape)
    u, v = x[..., :half], x[..., half:dims]
    out = x.copy()
    out[..., :half] = u * c - v * s
    out[..., half:dims] = v * c + u * s
    return out


def latent_attention(h, w: Dict[str, np.ndarray], m: dict, eps: float, positions=None):
    """The mixer of a ``latent_attention`` layer: keys and values of all heads are made from one normed latent vector per
    token; one rotated key part is shared by the heads."""
    T = h.shape[0]
    H, dk, dr, dv, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    pos = np.arange(T, dtype=np.float64) if positions is None else np.asarray(positions, dtype=np.float64)
    q = (h @ w["q"].T).reshape(T, H, dk + dr)
    down = h @ w["dkv"].T
    c = rms_norm(down[:, :rank], w["dkv.norm"], eps)
    k_rot = rotate_half(down[:, rank:], pos, m["rot"]["dims"], m["rot"]["base"])          # [T, dr]
    q_rot = rotate_half(q[:, :, dk:], pos, m["rot"]["dims"], m["rot"]["base"])            # [T, H, dr]
    k_plain = (c @ w["uk"].T).reshape(T, H, dk)
    v = (c @ w["uv"].T).reshape(T, H, dv)
    vis = window_visible(T, 0)
    out = np.zeros((T, H, dv))
    for i in range(H):
        s = (q[:, i, :dk] @ k_plain[:, i, :].T + q_rot[:, i, :] @ k_rot.T) * m["scale"]
        out[:, i, :] = softmax_rows(s, vis) @ v[:, i, :]
    gate = sigmoid(h @ w["g"].T)
    out = out * gate[:, :, None]
    return out.reshape(T, H * dv) @ w["o"].T


def dense_feed_forward(h, w: Dict[str, np.ndarray]):
    return (silu(h @ w["gate"].T) * (h @ w["up"].T)) @ w["down"].T


def hyper_in(streams, w_in):
    """streams [S, T, D]: the sublayer's input, sum_s in[s] x_s."""
    return np.tensordot(w_in, streams, axes=(0, 0))


def hyper_out(streams, y, w_mix, w_out):
    """x_t <- sum_s mix[s, t] x_s + out[t] y, all streams at once from the old ones."""
    mixed = np.tensordot(w_mix.T, streams, axes=(1, 0))           # [to, T, D]
    return mixed + w_out[:, None, None] * y[None, :, :]


# ---- the model ----------------------------------------------------------------------------------------------------
def _sub(weights: Dict[str, np.ndarray], prefix: str) -> Dict[str, np.ndarray]:
    return {k[len(prefix):]: v for k, v in weights.items() if k.startswith(prefix)}


def mixer(kind: str, h, w, m, eps):
    if kind == "attention":
        return differential_attention(h, w, m, eps)
    if kind == "latent_attention":
        return latent_attention(h, w, m, eps)
    raise ValueError(kind)


def layer_order(cfg: dict) -> List[int]:
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return list(range(n))
    a, b, times = loop["start"], loop["stop"], loop["times"]
    return list(range(a)) + list(range(a, b)) * times + list(range(b, n))


def forward(cfg: dict, weights: Dict[str, np.ndarray], tokens: List[int], layers_out: Optional[list] = None) -> np.ndarray:
    """Logits [T, vocab] of a whole sequence; ``layers_out`` collects the residual stream (the sum of the streams) after
    every layer run."""
    eps = cfg["norm"]["eps"]
    x = weights["embed"][np.asarray(tokens)] * (cfg.get("embedding") or {}).get("scale", 1.0)
    S = cfg.get("streams")
    streams = np.stack([x] * S) if S else None
    for i in layer_order(cfg):
        layer = cfg["layers"][i]
        p = f"l{i}."
        subs = [(1, lambda h: mixer(layer["type"], h, _sub(weights, p + "mix."), layer["mixer"], eps))]
        if layer.get("mlp") is not None:
            subs.append((2, lambda h: dense_feed_forward(h, _sub(weights, p + "mlp."))))
        for q, fn in subs:
            u = hyper_in(streams, weights[f"{p}hc{q}.in"]) if S else x
            y = fn(rms_norm(u, weights[f"{p}norm{q}"], eps))
            if f"{p}ls{q}" in weights:
                y = y * weights[f"{p}ls{q}"]
            if S:
                streams = hyper_out(streams, y, weights[f"{p}hc{q}.mix"], weights[f"{p}hc{q}.out"])
            else:
                x = x + y
        if layers_out is not None:
            layers_out.append(streams.sum(axis=0) if S else x.copy())
    if S:
        x = streams.sum(axis=0)
    return rms_norm(x, weights["final.norm"], eps) @ weights["head"].T
