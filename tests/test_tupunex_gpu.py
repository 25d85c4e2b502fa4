"""Tupunex on the GPU against the plain implementation (tests/plain_tupunex.py): each mechanism alone, keys that stand out
at the edges of windows and pages, then whole models under every way of cutting, decoding from the first token, slots
and pages used again, generation through the engine's own entry point, the replay program and the command line."""
import numpy as np
import pytest
import torch

import plain_tupunex as pt
import replay_util as ru
import tupunex_util as tu
from conftest import random_tokens

pytestmark = pytest.mark.gpu

DEV = "cuda"
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}
# relative root-mean-square error of a logits row against float64: fp32 sums of a few hundred terms; bfloat16 rounds the
# activations to 8 bits between kernels
ROW_TOL = {"float32": 3e-5, "bfloat16": 4e-2}


def rel_rms(got, want):
    d = np.asarray(got, dtype=np.float64) - want
    return np.sqrt((d * d).mean(axis=-1)) / max(np.sqrt((want * want).mean()), 1e-9)


def dev(a, dtype=torch.float32):
    return torch.from_numpy(np.ascontiguousarray(a)).to(DEV).to(dtype)


def bf16_round(a):
    return torch.from_numpy(np.asarray(a, dtype=np.float32)).to(torch.bfloat16).float().numpy().astype(np.float64)


class Ctx:
    """What an attention kernel reads of a step: one request, queries lo..hi-1, keys 0..hi-1 cached."""

    def __init__(self, lo, hi):
        n = hi - lo
        self.positions = torch.arange(lo, hi, dtype=torch.int32, device=DEV)
        self.token_req = torch.zeros(n, dtype=torch.int32, device=DEV)
        self.max_q_len, self.max_kv_len, self.n_requests, self.q_start, self.q_len, self.kv_len = n, hi, 1, [0], [n], [hi]
        self.derived, self.plans = {}, {}


def paged(rows, page_size, rng, dtype, extra=3, table=None):
    """Per-token rows [T, G, d] of one request scattered over shuffled pages (or those of ``table``): the pool
    [pages, G, page, d] and the table."""
    T, G, d = rows.shape
    n_pages = (T + page_size - 1) // page_size
    order = rng.permutation(n_pages + extra)[:n_pages] if table is None else table[0].cpu().numpy().astype(np.int64)
    pool = torch.zeros((n_pages + extra, G, page_size, d), dtype=dtype, device=DEV)
    full = np.zeros((n_pages * page_size, G, d))
    full[:T] = rows
    pool[torch.from_numpy(order).to(DEV)] = dev(full.reshape(n_pages, page_size, G, d).transpose(0, 2, 1, 3), dtype)
    return pool, torch.tensor(order[None, :].astype(np.int32), device=DEV)


# ---- mechanisms alone ---------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("S,d", [(1, 54), (2, 64), (3, 200), (5, 33), (8, 1024), (4, 4096)])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_stream_connections_read_and_write(S, d, dtype):
    from mimirmind_b200.kernels import ops
    rng = np.random.RandomState(S * 7 + d)
    n, eps = 6, 1e-5
    x0 = rng.randn(n, d).astype(np.float32).astype(np.float64)
    streams = np.stack([x0 * (1 + 0.3 * s) + 0.1 * s for s in range(S)]).astype(np.float32).astype(np.float64)      # [S, n, D]
    flat = dev(streams.transpose(1, 0, 2).reshape(n, S * d))
    a, b, mix = [rng.randn(S).astype(np.float32) for _ in range(2)] + [(np.eye(S) + 0.3 * rng.randn(S, S)).astype(np.float32)]
    w = bf16_round(1 + 0.2 * rng.randn(d))
    scale = (1 + 0.2 * rng.randn(d)).astype(np.float32)
    y = bf16_round(rng.randn(n, d)) if dtype == "bfloat16" else rng.randn(n, d).astype(np.float32).astype(np.float64)
    tol = 3e-6 if dtype == "float32" else 8e-3
    # the copies at the start
    c = ops.stream_copies(dev(x0), S).cpu().numpy().reshape(n, S, d)
    assert all(np.array_equal(c[:, s], x0.astype(np.float32)) for s in range(S))
    # read with the norm, read without (the sum of the streams)
    got = ops.hc_read(flat, S, dev(a), dev(w, DT[dtype]), eps, DT[dtype]).float().cpu().numpy()
    want = pt.rms_norm(pt.hyper_in(streams, a.astype(np.float64)), w, eps)
    assert np.abs(got - want).max() <= tol * np.abs(want).max()
    total = ops.hc_read(flat, S, torch.ones(S, device=DEV), None, 0.0, torch.float32).cpu().numpy()
    assert np.abs(total - streams.sum(0)).max() <= 3e-6 * np.abs(streams).max() * S
    # write alone; write with the next read and norm in the same pass
    want_streams = pt.hyper_out(streams, y * scale, mix.astype(np.float64), b.astype(np.float64))
    x1 = flat.clone()
    assert ops.hc_write(x1, S, dev(y, DT[dtype]), dev(scale), dev(mix), dev(b)) is None
    got_streams = x1.cpu().numpy().reshape(n, S, d).transpose(1, 0, 2)
    assert np.abs(got_streams - want_streams).max() <= 3e-6 * np.abs(want_streams).max()
    x2 = flat.clone()
    h = ops.hc_write(x2, S, dev(y, DT[dtype]), dev(scale), dev(mix), dev(b), dev(a), dev(w, DT[dtype]), eps, DT[dtype])
    assert torch.equal(x1, x2)
    want = pt.rms_norm(pt.hyper_in(want_streams, a.astype(np.float64)), w, eps)
    assert np.abs(h.float().cpu().numpy() - want).max() <= tol * np.abs(want).max()
    # without a scale per channel
    x3 = flat.clone()
    ops.hc_write(x3, S, dev(y, DT[dtype]), None, dev(mix), dev(b))
    want3 = pt.hyper_out(streams, y, mix.astype(np.float64), b.astype(np.float64))
    assert np.abs(x3.cpu().numpy().reshape(n, S, d).transpose(1, 0, 2) - want3).max() <= 3e-6 * np.abs(want3).max()


def test_the_mix_matrix_is_indexed_from_to():
    """One stream feeds another and nothing else happens: mix[0, 1] = 1 moves stream 0 into stream 1."""
    from mimirmind_b200.kernels import ops
    n, d = 3, 16
    x = np.zeros((n, 2, d), dtype=np.float32)
    x[:, 0] = 1.0
    x[:, 1] = 5.0
    mix = np.array([[0.0, 1.0], [0.0, 0.0]], dtype=np.float32)
    t = dev(x.reshape(n, 2 * d))
    ops.hc_write(t, 2, torch.zeros((n, d), device=DEV), None, dev(mix), torch.zeros(2, device=DEV))
    got = t.cpu().numpy().reshape(n, 2, d)
    assert (got[:, 0] == 0).all() and (got[:, 1] == 1).all()


@pytest.mark.parametrize("H,dv", [(4, 64), (3, 7), (1, 200), (6, 24), (16, 128)])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_head_finish(H, dv, dtype):
    from mimirmind_b200.kernels import ops
    rng = np.random.RandomState(H + dv)
    n, lam, eps, diff = 9, 0.73, 1e-5, 0.3
    att = bf16_round(rng.randn(n, 2, H, dv)) if dtype == "bfloat16" else rng.randn(n, 2, H, dv).astype(np.float32).astype(np.float64)
    gate = rng.randn(n, H + 3).astype(np.float32)
    tol = 1e-5 if dtype == "float32" else 1e-2
    wide = dev(gate)
    got = ops.head_finish(dev(att.reshape(n, 2 * H * dv), DT[dtype]), H, dv, pair=True, lam=lam, eps=eps, post=1 - diff, gate=wide[:, 2:2 + H])
    o = att[:, 0] - lam * att[:, 1]
    want = pt.rms(o, eps) * (1 - diff) * pt.sigmoid(gate[:, 2:2 + H].astype(np.float64))[:, :, None]
    assert np.abs(got.float().cpu().numpy().reshape(n, H, dv) - want).max() <= tol * np.abs(want).max()
    # a gate only
    got = ops.head_finish(dev(att[:, 0].reshape(n, H * dv), DT[dtype]), H, dv, gate=wide[:, :H])
    want = att[:, 0] * pt.sigmoid(gate[:, :H].astype(np.float64))[:, :, None]
    assert np.abs(got.float().cpu().numpy().reshape(n, H, dv) - want).max() <= tol * np.abs(want).max()
    # the difference and the norm without a gate
    got = ops.head_finish(dev(att.reshape(n, 2 * H * dv), DT[dtype]), H, dv, pair=True, lam=-0.2, eps=eps)
    want = pt.rms(att[:, 0] + 0.2 * att[:, 1], eps)
    assert np.abs(got.float().cpu().numpy().reshape(n, H, dv) - want).max() <= tol * np.abs(want).max()


@pytest.mark.parametrize("H,K,N,wide", [(4, 32, 128, 160), (3, 8, 20, 32), (2, 48, 24, 24), (1, 14, 9, 9), (16, 128, 512, 576), (5, 9, 3, 5)])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_matrix_per_head(H, K, N, wide, dtype):
    from mimirmind_b200.kernels import ops
    rng = np.random.RandomState(H * K + N)
    for n in (1, 5, 70):
        x, m = bf16_round(rng.randn(n, H, K)), bf16_round(rng.randn(H, K, N) / np.sqrt(K))
        out = torch.full((n, H * wide), 7.0, dtype=DT[dtype], device=DEV)
        ops.head_matmul(dev(x.reshape(n, H * K), DT[dtype]), dev(m, DT[dtype]), out, H)
        got = out.float().cpu().numpy().reshape(n, H, wide)
        want = np.einsum("thk,hkn->thn", x, m)
        assert np.abs(got[:, :, :N] - want).max() <= (1e-5 if dtype == "float32" else 1e-2) * np.abs(want).max()
        assert (got[:, :, N:] == 7.0).all(), "places behind a head's result were touched"


@pytest.mark.parametrize("dims,base", [(32, 20000.0), (12, 300.0), (2, 7.0), (64, 1e6)])
def test_rotation_angles_are_exact_far_out(dims, base):
    from mimirmind_b200.kernels import ops
    from mimirmind_b200.parts.latent_attention import split_frequencies
    pos = np.array([0, 1, 2, 63, 64, 1000, 65537, 1 << 19], dtype=np.int32)
    hi, lo = split_frequencies(base, dims, DEV)
    got = ops.rope_half_table(dev(pos, torch.int32), hi, lo).cpu().numpy()
    a = pos[:, None].astype(np.float64) * base ** (-2.0 * np.arange(dims // 2) / dims)
    # an angle kept as a float32 would be off by up to 0.03 at the last of these positions
    err = np.maximum(np.abs(got[..., 0] - np.cos(a)), np.abs(got[..., 1] - np.sin(a))).max(axis=1)
    assert (err[:6] < 5e-7).all() and (err[6:] < 5e-5).all(), err


def _two_maps(q, kp, vp, table, page, lo, hi, H, G, dk, dv, window, scale, cap, lam, diff, eps, dtype):
    """Queries lo..hi-1 (rows [T, 2, H, dk]: all first maps before all second maps) through the attention kernels and
    ``head_finish``, as the mixer runs them."""
    from mimirmind_b200.kernels import attention, ops
    from mimirmind_b200.parts.base import LayerCache
    n = hi - lo
    att = torch.empty((n, 2 * H * dv), dtype=torch.float32, device=DEV)
    cache = LayerCache(arrays={"k": kp, "v": vp}, block_table=table, page_size=page)
    attention.paged_sink_attention(dev(q[lo:hi].reshape(n, 2 * H * dk), DT[dtype]), cache, att, Ctx(lo, hi), 2 * H, 2 * G, dk, dv, window, scale, False,
                                   softcap=cap, value_heads=G)
    return ops.head_finish(att, H, dv, pair=True, lam=lam, eps=eps, post=1 - diff, out_dtype=DT[dtype]).float().cpu().numpy().reshape(n, H, dv)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,G,dk,dv,window,cap,page", [(8, 2, 32, 64, 44, 25.0, 16), (4, 2, 16, 24, 23, 4.0, 16), (3, 3, 10, 7, 1, 0.0, 8),
                                                       (8, 2, 64, 64, 70, 2.0, 32), (6, 2, 9, 11, 0, 5.0, 16), (2, 1, 128, 96, 129, 50.0, 64),
                                                       (1, 1, 96, 32, 64, 0.0, 16)])
def test_two_maps_over_the_same_values(H, G, dk, dv, window, cap, page, dtype):
    """The capped, windowed scores of both maps, their difference, the unit norm per head: prompts, portions that start
    and end anywhere, and single tokens, against the plain implementation."""
    rng = np.random.RandomState(H * 100 + dk + window)
    T, scale, lam, diff, eps = 300, 2.5 / np.sqrt(dk), 0.61, 0.35, 1e-6
    q, k, v = bf16_round(rng.randn(T, H, 2, dk)), bf16_round(rng.randn(T, G, 2, dk)), bf16_round(rng.randn(T, G, dv))
    want = pt.differential_attention_core(q, k, v, scale, cap, window, lam, diff, eps)
    kp, table = paged(k.transpose(0, 2, 1, 3).reshape(T, 2 * G, dk), page, rng, DT[dtype])
    vp, _ = paged(v, page, rng, DT[dtype], table=table)
    qm = q.transpose(0, 2, 1, 3)                                 # [T, 2, H, dk]
    # the difference of two nearly equal maps, normed to unit size, magnifies the maps' rounding
    tol = 5e-5 if dtype == "float32" else 6e-2
    for lo, hi in ((0, T), (0, 1), (1, 3), (17, 130), (130, 300), (299, 300), (150, 151), (63, 65)):
        got = _two_maps(qm, kp, vp, table, page, lo, hi, H, G, dk, dv, window, scale, cap, lam, diff, eps, dtype)
        err = np.sqrt(((got - want[lo:hi]) ** 2).mean(-1))       # every head's result has unit size
        assert err.max() <= tol, f"portion {lo}..{hi}: {err.max():.3g} at {np.unravel_index(err.argmax(), err.shape)}"
    if cap:
        uncapped = pt.differential_attention_core(q, k, v, scale, 0.0, window, lam, diff, eps)
        if np.abs(uncapped - want).max() > 0.05:                 # the cap bends these scores: leaving it out would show
            got = _two_maps(qm, kp, vp, table, page, 0, T, H, G, dk, dv, window, scale, cap, lam, diff, eps, dtype)
            assert np.abs(got - uncapped).max() > 0.03


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("style,window,page", [("maps", 48, 16), ("maps", 64, 16), ("maps", 17, 8), ("maps", 65, 32), ("maps", 1, 16),
                                               ("maps", 0, 16), ("latent", 0, 16), ("latent", 0, 64), ("latent", 33, 16), ("latent", 32, 8)])
@pytest.mark.parametrize("dk,dv", [(32, 64), (12, 8), (64, 64)])
def test_one_key_that_stands_out_is_seen_exactly_inside_the_window(style, window, page, dtype, dk, dv):
    """Every key is orthogonal to the query but one, whose score stands out by far and whose value is a marker: the
    output shows the marker exactly when that key is visible, in a prompt and for a single decoded token, with the key
    at a page's border, far back, at the sequence's start, and just inside and just outside the window.  ``maps``: the
    call of the two-map attention (twice the heads, capped scores, fewer value heads than key heads); ``latent``: the call
    of the latent attention (one key head whose leading part is the value)."""
    from mimirmind_b200.kernels import attention
    from mimirmind_b200.parts.base import LayerCache
    H, G, T = 6, 2, 400
    rng = np.random.RandomState(window + page + dk)
    for query in (399, 256, 255, 64, 40, 17, 16, 1, 0):
        spots = {query, query - 1, 0, 1, 15, 16, 17, query - window + 1, query - window, query - window - 1, (query // page) * page,
                 (query // page) * page - 1, query - 200, (query // 64) * 64, (query // 64) * 64 - 1}
        for spot in sorted(s for s in spots if 0 <= s <= query):
            inside = window == 0 or query - spot < window
            if style == "maps":
                k = rng.randn(T, 2 * G, dk) * 0.01
                k[:, :, 0] = 0.0
                k[spot, :, 0] = 1.0
                v = rng.randn(T, G, dv) * 0.01
                v[spot] = 5.0
                q = np.zeros((T, 2 * H, dk))
                q[:, :, 0] = 25.0                                   # capped at 20: still far above every other score
                kp, table = paged(k, page, rng, DT[dtype])
                vp, _ = paged(v, page, rng, DT[dtype], table=table)
                cache = LayerCache(arrays={"k": kp, "v": vp}, block_table=table, page_size=page)
                kw = dict(softcap=20.0, value_heads=G)
                heads, kv_heads, key_dim, value_dim = 2 * H, 2 * G, dk, dv
            else:
                wide = dv + dk                                      # the value is the leading part of the key
                row = rng.randn(T, 1, wide) * 0.01
                row[:, :, dv] = 0.0
                row[spot, :, :dv] = 5.0
                row[spot, :, dv] = 1.0
                q = np.zeros((T, H, wide))
                q[:, :, dv] = 25.0
                pool, table = paged(row, page, rng, DT[dtype])
                cache = LayerCache(arrays={"latent": pool}, block_table=table, page_size=page)
                heads, kv_heads, key_dim, value_dim = H, 1, wide, dv
            for lo in (query, max(0, query - 50), max(0, query - 1)):          # decoded alone; the last of a portion; of two tokens
                n = query + 1 - lo
                out = torch.empty((n, heads * value_dim), dtype=DT[dtype], device=DEV)
                if style == "latent":
                    attention.paged_latent_attention(dev(q[lo:query + 1].reshape(n, heads * key_dim), DT[dtype]), pool, cache, out,
                                                     Ctx(lo, query + 1), heads, wide, dv, window, 1.0)
                else:
                    attention.paged_sink_attention(dev(q[lo:query + 1].reshape(n, heads * key_dim), DT[dtype]), cache, out, Ctx(lo, query + 1), heads,
                                                   kv_heads, key_dim, value_dim, window, 1.0, False, **kw)
                last = out[-1].float().cpu().numpy()
                if inside:
                    assert (last > 4.8).all(), f"query {query}, key {spot}, window {window}, from {lo}: the key was not seen"
                elif spot < query:          # the query's own key is always visible, so the weights go to small values
                    assert (np.abs(last) < 0.2).all(), f"query {query}, key {spot}, window {window}, from {lo}: a hidden key was seen"


class BatchCtx:
    """What an attention kernel reads of a step of several requests: request r brings the tokens lo[r]..hi[r]-1."""

    def __init__(self, spans):
        pos, req, self.q_start, self.q_len, self.kv_len = [], [], [], [], []
        for r, (lo, hi) in enumerate(spans):
            self.q_start.append(len(pos))
            self.q_len.append(hi - lo)
            self.kv_len.append(hi)
            pos += list(range(lo, hi))
            req += [r] * (hi - lo)
        self.positions = torch.tensor(pos, dtype=torch.int32, device=DEV)
        self.token_req = torch.tensor(req, dtype=torch.int32, device=DEV)
        self.n_requests, self.max_q_len, self.max_kv_len = len(spans), max(self.q_len), max(self.kv_len)
        self.derived, self.plans = {}, {}


@pytest.mark.parametrize("target_ctas,wide_tiles", [(296, True), (100000, True), (296, False), (100000, False)])
@pytest.mark.parametrize("H,rank,extra,page,window", [(4, 64, 32, 16, 0), (3, 96, 32, 16, 0), (40, 32, 8, 8, 0), (16, 512, 64, 64, 0),
                                                      (1, 48, 16, 32, 0), (5, 128, 24, 16, 45), (2, 256, 64, 16, 0), (33, 16, 8, 16, 100)])
def test_many_heads_over_one_shared_key_head_whose_leading_part_is_the_value(H, rank, extra, page, window, target_ctas, wide_tiles, monkeypatch):
    """The tensor-core kernel of the latent attention against the sum written out in float64: a step of a long portion,
    a portion of two tokens, a portion that starts at position 0 and single tokens of several requests, each with pages
    of its own in one pool; head counts below, at and above a tile's rows; with the key tiles of a row in one CTA and
    shared out over many; with tiles of 64 rows and of 32."""
    from mimirmind_b200.kernels import attention
    from mimirmind_b200.parts.base import LayerCache
    assert attention._latent_lib().mm_attention_latent_supported(rank + extra, rank)
    monkeypatch.setattr(attention, "SINK_TARGET_CTAS", target_ctas)
    monkeypatch.setattr(attention, "USE_LATENT_WIDE_TILES", wide_tiles)
    rng = np.random.RandomState(H * 1000 + rank)
    wide = rank + extra
    spans = [(130, 331), (258, 260), (0, 37), (299, 300), (0, 1), (64, 65), (31, 33)]
    rows = [bf16_round(rng.randn(hi, 1, wide) * 0.7) for _, hi in spans]
    width = max(-(-hi // page) for _, hi in spans)
    n_pages = sum(-(-hi // page) for _, hi in spans) + 3
    order = rng.permutation(n_pages)
    pool = torch.full((n_pages, 1, page, wide), float("nan"), dtype=torch.bfloat16, device=DEV)    # an unwritten row must never be read
    table = np.zeros((len(spans), width), dtype=np.int32)
    at = 0
    for r, (_, hi) in enumerate(spans):
        for p in range(-(-hi // page)):
            table[r, p] = order[at]
            n = min(page, hi - p * page)
            pool[int(order[at]), 0, :n] = dev(rows[r][p * page:p * page + n, 0], torch.bfloat16)
            at += 1
    ctx = BatchCtx(spans)
    n = int(ctx.positions.numel())
    q = bf16_round(rng.randn(n, H, wide))
    scale = 0.9 / np.sqrt(wide)
    want = np.zeros((n, H, rank))
    for r, (lo, hi) in enumerate(spans):
        for t in range(lo, hi):
            first = max(0, t + 1 - window) if window else 0
            keys = rows[r][first:t + 1, 0]
            sc = np.einsum("hw,jw->hj", q[ctx.q_start[r] + t - lo], keys) * scale
            w = np.exp(sc - sc.max(axis=1, keepdims=True))
            want[ctx.q_start[r] + t - lo] = (w / w.sum(axis=1, keepdims=True)) @ keys[:, :rank]
    cache = LayerCache(arrays={"latent": pool}, block_table=torch.from_numpy(table).to(DEV), page_size=page)
    for out_dtype, tol in ((torch.float32, 6e-3), (torch.bfloat16, 1.2e-2)):
        out = torch.full((n, H * rank), float("nan"), dtype=out_dtype, device=DEV)
        attention.paged_latent_attention(dev(q.reshape(n, H * wide), torch.bfloat16), pool, cache, out, ctx, H, wide, rank, window, scale)
        got = out.float().cpu().numpy().reshape(n, H, rank)
        assert np.isfinite(got).all()
        err = np.abs(got - want).max(axis=(1, 2)) / np.abs(want).max()
        assert err.max() < tol, f"token row {int(err.argmax())}: {err.max()}"


@pytest.mark.parametrize("taps,C", [(3, 40), (1, 7), (8, 130), (2, 512)])
def test_short_convolution_without_activation_and_its_state(taps, C):
    """Both forms of the convolution (a walk per channel, a thread per token and channel), cut into portions that leave
    and pick up the last taps - 1 inputs, against the plain convolution over the whole sequence."""
    from mimirmind_b200.kernels import ops
    rng = np.random.RandomState(taps + C)
    T, ld = 90, C + 5
    u = rng.randn(T, ld).astype(np.float32)
    w = rng.randn(C, taps).astype(np.float32)
    want = pt.causal_conv(u[:, :C].astype(np.float64), w.astype(np.float64))
    for form in ("walk", "tokens"):
        tail = torch.full((3, max(1, (taps - 1) * C) + 2), 9.0, device=DEV)            # what the slot's last user left
        got, at = [], 0
        for n in (1, 2, 40, 1, 1, 3, 42):
            rows = dev(u[at:at + n])
            pos = torch.arange(at, at + n, dtype=torch.int32, device=DEV)
            req = torch.zeros(n, dtype=torch.int32, device=DEV)
            meta = torch.tensor([[0, n, at + n, 1]], dtype=torch.int32, device=DEV)
            slots = torch.tensor([1], dtype=torch.int32, device=DEV)
            if form == "walk":
                ops.causal_conv_walk(rows, C, dev(w), tail, meta, slots, pos, 1, silu=False)
                got.append(rows[:, :C].cpu().numpy())
                assert np.array_equal(rows[:, C:].cpu().numpy(), u[at:at + n, C:]), "columns behind the channels were touched"
            else:
                got.append(ops.causal_conv_tokens(rows, C, dev(w), tail, req, meta, slots, pos, 1, silu=False).cpu().numpy())
            at += n
        assert at == T
        assert np.abs(np.concatenate(got) - want).max() <= 2e-6 * max(1.0, np.abs(want).max()), form
        assert (tail[0] == 9.0).all() and (tail[2] == 9.0).all(), "another slot's state was touched"


# ---- whole models -------------------------------------------------------------------------------------------------------
@pytest.fixture(scope="module")
def models(tmp_path_factory):
    cache = {}

    def get(name, cfg=None, overrides=None):
        if name not in cache:
            folder = tu.write_model(str(tmp_path_factory.mktemp(f"tupunex_{name}")), cfg or tu.CONFIGS[name], seed=len(cache) + 21, overrides=overrides)
            cache[name] = (folder,) + pt.load_folder(folder)
        return cache[name]

    return get


def check_rows(trace, outputs, reqs, ref, dtype, what, tol=None):
    got = ru.collect(trace, outputs)
    tol = tol or ROW_TOL[dtype]
    for rid, toks in reqs.items():
        rows = np.stack([got[(rid, p)] for p in range(len(toks))])
        err = rel_rms(rows, ref[rid])
        if dtype == "bfloat16" and err.max() <= 2.5 * tol and (err > tol).sum() <= max(2, 0.02 * len(err)):
            # sharp scores and a difference of maps normed to unit size magnify the rounding of single positions (another
            # position with every change of a rounding); the 32-bit run of the same schedule has to be within its bound everywhere
            continue
        assert err.max() <= tol, (f"{what} {dtype} request {rid}: error {err.max():.3g} at position {int(err.argmax())} of {len(toks)}, "
                                  f"first position above the bound: {int(np.argmax(err > tol))}")
    return got


ONE_LAYER = {
    # each mixer alone in a model of one layer without a feed-forward, so that nothing else shapes the logits
    "maps": tu.config(60, 40, 1e-6, [tu.attention(4, 2, 8, 12, 0.5, 0.4, window=21, softcap=3.0, conv=3)]),
    "maps_wide": tu.config(60, 64, 1e-6, [tu.attention(2, 2, 32, 64, 0.25, 0.7, window=33, softcap=8.0, conv=2)], streams=2),
    "latent": tu.config(60, 40, 1e-6, [tu.latent(3, 8, 6, 10, 16, 0.4, 40.0)]),
    "latent_wide": tu.config(60, 64, 1e-6, [tu.latent(2, 32, 32, 48, 64, 0.2, 10000.0)], streams=2),
}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(ONE_LAYER))
def test_each_mixer_alone_in_a_model_of_one_layer(name, dtype, models):
    folder, cfg, w = models(name, ONE_LAYER[name])
    lo = []
    toks = random_tokens(cfg["vocab"], 120, 3)
    want = pt.forward(cfg, w, toks, lo)
    from mimirmind_b200.engine.loader import load_model
    from mimirmind_b200.engine.runner import ModelRunner, StepEntry
    model, _ = load_model(folder, dtype)
    runner = ModelRunner(model, page_size=16, num_pages=16, max_requests=2)

    class Dump:
        got = {}

        def write(self, block, stage, rows):
            self.got[(block, stage)] = rows.float().cpu().numpy().copy()

    runner.add_request("a")
    runner.stage_dump = Dump()
    logits = runner.step([StepEntry("a", toks, list(range(len(toks))))]).float().cpu().numpy()
    out = runner.stage_dump.got[(0, "l_out")]
    tol = 2e-5 if dtype == "float32" else 3e-2
    assert np.abs(out - lo[0]).max() <= tol * np.abs(lo[0]).max(), "the residual stream behind the layer"
    assert rel_rms(logits, want).max() <= ROW_TOL[dtype]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name,page_size", [("A", 16), ("B", 16), ("C", 8), ("A", 32), ("D", 16), ("B", 64)])
def test_every_way_of_cutting_matches_the_plain_implementation(name, page_size, dtype, models):
    folder, cfg, w = models(name)
    reqs = {f"{name}{i}": random_tokens(cfg["vocab"], n, 100 * i + n) for i, n in enumerate(tu.LENGTHS[name])}
    ref = {rid: pt.forward(cfg, w, t) for rid, t in reqs.items()}
    results = {}
    t = ru.Trace()
    for rid, toks in reqs.items():
        ru.whole(t, rid, toks)
    out, _ = ru.run_in_process(folder, dtype, t, t.max_live_tokens(), page_size)
    results["whole"] = check_rows(t, out, reqs, ref, dtype, "whole")
    t = ru.Trace()
    for rid, toks in reqs.items():
        ru.tail_one_by_one(t, rid, toks, 140)                            # longer than every window: it passes over decoded tokens
    out, _ = ru.run_in_process(folder, dtype, t, t.max_live_tokens(), page_size)
    results["tail"] = check_rows(t, out, reqs, ref, dtype, "tail one by one")
    t = ru.Trace()
    for i, (rid, toks) in enumerate(reqs.items()):
        ru.chunks(t, rid, toks, [[17, 7, 5, 3, 2], [2, 64, 3, 31], [33, 2, 2, 16], [2]][i % 4])
    out, _ = ru.run_in_process(folder, dtype, t, t.max_live_tokens(), page_size)
    results["chunks"] = check_rows(t, out, reqs, ref, dtype, "portions")
    t = ru.Trace()
    twice = dict(reqs)
    twice.update({rid + "x": toks for rid, toks in reqs.items()})
    ru.mixed(t, twice, seed=len(name) + page_size)
    out, runner = ru.run_in_process(folder, dtype, t, t.max_live_tokens(), page_size)
    ref2 = dict(ref)
    ref2.update({rid + "x": ref[rid] for rid in reqs})
    results["mixed"] = check_rows(t, out, twice, ref2, dtype, "mixed")
    assert runner.manager.reuses() > 0, "the pool was large enough that no page was used again"
    for g in runner.manager.groups:
        assert runner.manager.free_pages(g) == runner.manager.total_pages(g)
    if dtype == "float32":
        # the 32-bit kernels sum in an order fixed by position: cutting changes nothing at all
        for mode in ("tail", "chunks", "mixed"):
            for key, row in results["whole"].items():
                assert np.array_equal(results[mode][key], row), f"{mode}: {key} differs from the whole run"


@pytest.mark.parametrize("name,dtype", [("A", "float32"), ("C", "bfloat16"), ("B", "bfloat16")])
def test_decoding_from_the_first_token(name, dtype, models):
    """300 steps of one token each: the convolutions' state, the windows and every cache from an empty start."""
    folder, cfg, w = models(name)
    toks = random_tokens(cfg["vocab"], 300, 5)
    t = ru.Trace()
    ru.chunks(t, "d", toks, [1])
    out, _ = ru.run_in_process(folder, dtype, t, t.max_live_tokens())
    check_rows(t, out, {"d": toks}, {"d": pt.forward(cfg, w, toks)}, dtype, "decode from the first token")


def test_sharp_scores_show_a_window_that_is_one_token_off(models):
    """Large queries, keys and score scales make sharp attention: a key wrongly seen or missed moves the logits by far
    more than the bound.  The plain implementation with every window one token longer or shorter differs."""
    import copy
    cfg = tu.config(80, 48, 1e-6, [tu.attention(2, 1, 16, 16, 0.6, 0.3, window=19, softcap=25.0, conv=2, mlp=tu.dense(32)),
                                   tu.latent(2, 8, 8, 16, 24, 0.9, 100.0, mlp=tu.dense(32)),
                                   tu.attention(4, 4, 8, 8, 0.8, 0.5, window=64, softcap=40.0, conv=3)], streams=2)
    folder, cfg, w = models("sharp", cfg)
    toks = random_tokens(cfg["vocab"], 200, 17)
    ref = pt.forward(cfg, w, toks)
    for delta in (-1, 1):
        off = copy.deepcopy(cfg)
        for layer in off["layers"]:
            if layer["type"] == "attention":
                layer["mixer"]["mask"]["size"] += delta
        assert rel_rms(pt.forward(off, w, toks), ref)[70:].max() > 20 * ROW_TOL["float32"], "the test's weights hide the window"
    for cut in ("whole", "tail", "chunks"):
        t = ru.Trace()
        {"whole": lambda: ru.whole(t, "s", toks), "tail": lambda: ru.tail_one_by_one(t, "s", toks, 150),
         "chunks": lambda: ru.chunks(t, "s", toks, [19, 2, 45, 3])}[cut]()
        out, _ = ru.run_in_process(folder, "float32", t, t.max_live_tokens())
        check_rows(t, out, {"s": toks}, {"s": ref}, "float32", cut)


def test_a_slot_used_again_starts_clean(models):
    """Two state slots, five requests one after the other and in pairs: a request never sees what the slot's last
    user left (the convolutions' last inputs, pages of keys)."""
    from mimirmind_b200.engine.loader import load_model
    from mimirmind_b200.engine.runner import ModelRunner, StepEntry
    folder, cfg, w = models("A")
    model, _ = load_model(folder, "float32")
    runner = ModelRunner(model, page_size=16, num_pages=12, max_requests=2)
    reqs = [random_tokens(cfg["vocab"], n, n) for n in (60, 3, 90, 31, 64)]
    ref = [pt.forward(cfg, w, t) for t in reqs]
    assert runner.add_request(0) and runner.add_request(1) and not runner.add_request(2)
    got0 = runner.step([StepEntry(0, reqs[0][:50], [49]), StepEntry(1, reqs[1], [0, 2])]).cpu().numpy()
    runner.release(1)
    assert runner.add_request(2)
    got1 = runner.step([StepEntry(2, reqs[2][:7], [0, 6]), StepEntry(0, reqs[0][50:], [9])]).cpu().numpy()
    runner.release(0)
    assert runner.add_request(3)
    got2 = runner.step([StepEntry(3, reqs[3], [0, 1, 30]), StepEntry(2, reqs[2][7:], [82])]).cpu().numpy()
    runner.release(2), runner.release(3)
    assert runner.add_request(4)
    got3 = runner.step([StepEntry(4, reqs[4], [0, 1, 63])]).cpu().numpy()
    pairs = ((got0[0], ref[0][49]), (got0[1], ref[1][0]), (got0[2], ref[1][2]), (got1[0], ref[2][0]), (got1[1], ref[2][6]), (got1[2], ref[0][59]),
             (got2[0], ref[3][0]), (got2[1], ref[3][1]), (got2[2], ref[3][30]), (got2[3], ref[2][89]), (got3[0], ref[4][0]), (got3[1], ref[4][1]),
             (got3[2], ref[4][63]))
    for i, (got, want) in enumerate(pairs):
        assert rel_rms(got, want) <= ROW_TOL["float32"], i


@pytest.mark.parametrize("name,dtype", [("A", "float32"), ("B", "bfloat16"), ("D", "float32")])
def test_greedy_generation_through_the_engine(name, dtype, models):
    """Engine.generate (scheduler, prompt portions, captured decode steps) picks the plain implementation's tokens."""
    from mimirmind_b200 import Engine
    folder, cfg, w = models(name)
    prompts = [random_tokens(cfg["vocab"], n, 40 + n) for n in (5, 17, 33, 64)]
    eng = Engine.from_folder(folder, dtype=dtype, page_size=16, cache_tokens=1024, max_context=512, token_budget=48, max_active=4)
    res = eng.generate(prompts, max_new_tokens=24)
    margin = 1e-4 if dtype == "float32" else 0.12
    exact = 0
    for p, r in zip(prompts, res):
        assert r.stats.generated_tokens == 24 and r.stats.finish_reason == "length"
        toks = list(p)
        for i, tok in enumerate(r.tokens):
            row = pt.forward(cfg, w, toks)[-1]
            best = int(np.argmax(row))
            assert row[tok] >= row[best] - margin, f"token {i}: engine chose {tok} ({row[tok]:.4f}), plain {best} ({row[best]:.4f})"
            exact += tok == best
            toks.append(tok)
    assert exact >= (96 if dtype == "float32" else 80)
    assert eng.runner.manager.free_pages() == eng.runner.manager.total_pages()
    # a second run over the same engine (slots and pages used again) gives the same tokens
    again = eng.generate(prompts, max_new_tokens=24)
    if dtype == "float32":
        assert [r.tokens for r in again] == [r.tokens for r in res]


def test_the_replay_program_on_this_design(models, tmp_path):
    folder, cfg, w = models("C")
    reqs = {f"r{i}": random_tokens(cfg["vocab"], n, 11 + i) for i, n in enumerate([3, 90, 41, 150])}
    ref = {rid: pt.forward(cfg, w, t) for rid, t in reqs.items()}
    t = ru.Trace()
    ru.mixed(t, reqs, seed=3)
    t.step([("last", [1, 2, 3], [])], end=["last"])
    out = ru.run_program(folder, "bfloat16", t, t.max_live_tokens(), str(tmp_path / "out"), cfg["vocab"])
    check_rows(t, out, reqs, ref, "bfloat16", "program")


def test_the_command_line_generates_with_this_design(models, tmp_path):
    """bin/mimirmind: random-weights mode writes a Tupunex folder from its config.json, smoke generates from it and from
    a test model; the greedy tokens of the test model are the plain implementation's."""
    import json
    import os
    import subprocess
    import sys
    from conftest import ROOT
    folder, cfg, w = models("D")
    exe = [sys.executable, os.path.join(ROOT, "bin", "mimirmind")]
    conf = {"defaultModel": "m", "models": [{"id": "m", "path": folder}], "runtime": {"dtype": "float32", "maxContextTokens": 256, "cacheTokens": 512}}
    (tmp_path / "config.json").write_text(json.dumps(conf))
    out = subprocess.run(exe + ["smoke", "--config", str(tmp_path / "config.json"), "--prompt", "5 17 3 50", "--max-new", "6"],
                         capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stderr
    lines = out.stdout.strip().splitlines()
    got = [int(t) for t in lines[0].split()]
    assert len(got) == 6 and lines[1] == "generated 6"
    toks = [5, 17, 3, 50]
    for tok in got:
        row = pt.forward(cfg, w, toks)[-1]
        assert row[tok] >= row.max() - 1e-4
        toks.append(tok)
    (tmp_path / "mc.json").write_text(json.dumps(tu.CONFIGS["A"]))
    rw = subprocess.run(exe + ["random-weights", "--model-config", str(tmp_path / "mc.json"), "--seed", "9", "--out", str(tmp_path / "rw"),
                               "--dtype", "bfloat16"], capture_output=True, text=True, timeout=300)
    assert rw.returncode == 0, rw.stderr
    conf["models"][0]["path"] = str(tmp_path / "rw")
    conf["runtime"]["dtype"] = "bfloat16"
    (tmp_path / "config2.json").write_text(json.dumps(conf))
    out = subprocess.run(exe + ["smoke", "--config", str(tmp_path / "config2.json"), "--prompt", "1 2 3", "--max-new", "4"],
                         capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stderr
    assert out.stdout.strip().splitlines()[1] == "generated 4"
