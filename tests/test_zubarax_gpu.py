"""Zubarax on the GPU against the plain implementation (tests/plain_zubarax.py): each mechanism alone, then whole models
under every way of cutting, decoding from the first token, slots and pages used again, generation through the engine's
own entry point, the replay program and the command line."""
import numpy as np
import pytest
import torch

import plain_zubarax as pz
import replay_util as ru
import zubarax_util as zu
from conftest import random_tokens

pytestmark = pytest.mark.gpu

DEV = "cuda"
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}
# relative root-mean-square error of a logits row against float64
ROW_TOL = {"float32": 5e-5, "bfloat16": 5e-2}


def rel_rms(got, want):
    d = np.asarray(got, dtype=np.float64) - want
    return np.sqrt((d * d).mean(axis=-1)) / max(np.sqrt((want * want).mean()), 1e-9)


def dev(a, dtype=torch.float32):
    return torch.from_numpy(np.ascontiguousarray(a)).to(DEV).to(dtype)


def bf16_round(a):
    return torch.from_numpy(np.asarray(a, dtype=np.float32)).to(torch.bfloat16).float().numpy().astype(np.float64)


def i32(a):
    return torch.tensor(a, dtype=torch.int32, device=DEV)


# ---- attention with mixed heads -------------------------------------------------------------------------------------
def _paged(k, v, page_size, rng, dtype):
    """Keys and values of one request scattered over a shuffled pool whose unwritten rows are NaN."""
    T, G, dk = k.shape
    dv = v.shape[2]
    n_pages = (T + page_size - 1) // page_size
    perm = rng.permutation(n_pages + 3)[:n_pages]
    kp = np.full((n_pages + 3, G, page_size, dk), np.nan)
    vp = np.full((n_pages + 3, G, page_size, dv), np.nan)
    for t in range(T):
        kp[perm[t // page_size], :, t % page_size] = k[t]
        vp[perm[t // page_size], :, t % page_size] = v[t]
    return dev(kp, dtype), dev(vp, dtype), i32(perm[None, :].tolist())


class _Ctx:
    pass


def _attend(q, kp, vp, table, page, lo, hi, H, G, dk, dv, scale, dtype, talk, sink, window=0, single=False):
    """Queries lo..hi-1 of one request as one step: a portion, or (``single``) one token per step, as decoding does."""
    from mimirmind_b200.kernels import attention
    from mimirmind_b200.parts.base import LayerCache
    outs = []
    for a, b in ([(p, p + 1) for p in range(lo, hi)] if single else [(lo, hi)]):
        n = b - a
        ctx = _Ctx()
        ctx.positions = torch.arange(a, b, dtype=torch.int32, device=DEV)
        ctx.token_req = torch.zeros(n, dtype=torch.int32, device=DEV)
        ctx.max_q_len, ctx.max_kv_len, ctx.n_requests, ctx.q_start, ctx.q_len, ctx.kv_len = n, b, 1, [0], [n], [b]
        ctx.derived, ctx.plans = {}, {}
        out = torch.empty((n, H * dv), dtype=DT[dtype], device=DEV)
        attention.paged_talking_attention(dev(q[a:b].reshape(n, H * dk), DT[dtype]), LayerCache(arrays={"k": kp, "v": vp}, block_table=table, page_size=page),
                                          out, ctx, H, G, dk, dv, window, scale, dev(talk) if talk is not None else None,
                                          dev(sink) if sink is not None else None)
        outs.append(out.float().cpu().numpy().reshape(n, H, dv))
    return np.concatenate(outs, 0)


@pytest.fixture(params=[True, False], ids=["tensor-cores", "fp32-arithmetic"])
def route(request, monkeypatch):
    """Both kernels of the attention with mixed heads: sizes the tensor-core kernel takes run it, or never."""
    from mimirmind_b200.kernels import attention
    monkeypatch.setattr(attention, "USE_TALKING_MMA", request.param)
    return request.param


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,G,dk,dv,page", [(4, 2, 24, 16, 16), (3, 3, 9, 7, 8), (8, 2, 64, 64, 16), (5, 1, 96, 32, 32), (1, 1, 10, 12, 16), (16, 4, 128, 64, 16),
                                            (6, 6, 96, 96, 16), (32, 8, 128, 128, 16), (20, 4, 64, 128, 8), (3, 1, 32, 64, 64)])
def test_mixed_heads_attention_against_the_plain_one(H, G, dk, dv, page, dtype, route):
    if dtype == "float32" and not route:
        pytest.skip("the 32-bit mode has one route")
    rng = np.random.RandomState(H * 100 + dk)
    T = 300
    q, k, v = rng.randn(T, H, dk), rng.randn(T, G, dk), rng.randn(T, G, dv)
    talk, sink, scale = np.eye(H) + 0.3 * rng.randn(H, H), rng.randn(H), 1.0 / np.sqrt(dk)
    if dtype == "bfloat16":
        q, k, v = bf16_round(q), bf16_round(k), bf16_round(v)
    want = pz.talking_sink_attention_core(q, k, v, talk.astype(np.float32).astype(np.float64), sink.astype(np.float32).astype(np.float64), scale)
    kp, vp, table = _paged(k, v, page, rng, DT[dtype])
    tol = 2e-5 if dtype == "float32" else 2e-2
    for lo, hi, single in ((0, T, False), (0, 1, False), (41, 43, False), (250, T, False), (280, T, True), (0, 3, True)):
        got = _attend(q, kp, vp, table, page, lo, hi, H, G, dk, dv, scale, dtype, talk, sink, single=single)
        assert not np.isnan(got).any()
        assert np.abs(got - want[lo:hi]).max() <= tol * max(1.0, np.abs(want).max()), (lo, hi, single)
    # without mixing and without a sink it is plain softmax attention
    plain = pz.talking_sink_attention_core(q[:50], k[:50], v[:50], np.eye(H), np.full(H, -1e30), scale)
    got = _attend(q, kp, vp, table, page, 0, 50, H, G, dk, dv, scale, dtype, None, None)
    assert np.abs(got - plain).max() <= tol * max(1.0, np.abs(plain).max())


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("dk,dv", [(16, 8), (64, 64), (96, 32)])
def test_one_key_that_stands_out(dk, dv, dtype, route):
    """One key answers one query direction with a score far above the rest: the query's result is that key's value, at the
    sequence's start, on both sides of page borders, hundreds of tokens back, in a portion, in a portion of two tokens and
    for a single token; through another head when the mixing matrix swaps heads; and not at all one token outside a window."""
    H, G, page, T = 4, 2, 16, 700
    rng = np.random.RandomState(dk)
    talk = np.eye(H)[[1, 0, 3, 2]]            # head h's score is its neighbour's
    for spot in (0, 1, 15, 16, 17, 31, 32, 333, 640):
        q, k, v = 0.1 * rng.randn(T, H, dk), 0.1 * rng.randn(T, G, dk), rng.randn(T, G, dv)
        direction = rng.randn(dk)
        direction /= np.linalg.norm(direction)
        k[spot, 0] = 30.0 * direction
        askers = sorted({min(T - 1, spot + d) for d in (0, 1, 2, 40)} | {T - 1})
        for a in askers:
            q[a, 0] = 30.0 * direction         # head 0 asks; after mixing the answer arrives in head 1
        if dtype == "bfloat16":
            q, k, v = bf16_round(q), bf16_round(k), bf16_round(v)
        kp, vp, table = _paged(k, v, page, rng, DT[dtype])
        tol = 1e-4 if dtype == "float32" else 2e-2
        for a in askers:
            for lo, hi, single in ((max(0, a - 20), a + 1, False), (max(0, a - 1), a + 1, False), (a, a + 1, True)):
                got = _attend(q, kp, vp, table, page, lo, hi, H, G, dk, dv, 1.0, dtype, talk, np.zeros(H))
                assert np.abs(got[a - lo, 1] - v[spot, 0]).max() <= tol * 10, (spot, a, lo, hi)
            # a window that ends one token short of the key does not see it; one that reaches it does
            dist = a - spot
            if dist >= 1:
                inside = _attend(q, kp, vp, table, page, a, a + 1, H, G, dk, dv, 1.0, dtype, talk, np.zeros(H), window=dist + 1)
                outside = _attend(q, kp, vp, table, page, a, a + 1, H, G, dk, dv, 1.0, dtype, talk, np.zeros(H), window=dist)
                assert np.abs(inside[0, 1] - v[spot, 0]).max() <= tol * 10
                assert np.abs(outside[0, 1] - v[spot, 0]).max() > 0.1


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_the_learned_sink_takes_its_share(dtype, route):
    H, G, dk, dv, page, T = 3, 3, 32, 32, 16, 90
    rng = np.random.RandomState(3)
    q, k, v = rng.randn(T, H, dk), rng.randn(T, G, dk), rng.randn(T, G, dv)
    if dtype == "bfloat16":
        q, k, v = bf16_round(q), bf16_round(k), bf16_round(v)
    kp, vp, table = _paged(k, v, page, rng, DT[dtype])
    sink = np.array([40.0, -40.0, 0.0])      # drowns head 0, vanishes from head 1, weighs as much as one key of score 0 in head 2
    for single in (False, True):
        got = _attend(q, kp, vp, table, page, 60, T, H, G, dk, dv, 0.2, dtype, None, sink, single=single)
        want = pz.talking_sink_attention_core(q, k, v, np.eye(H), sink, 0.2)[60:]
        plain = pz.talking_sink_attention_core(q, k, v, np.eye(H), np.full(H, -1e30), 0.2)[60:]
        tol = 1e-5 if dtype == "float32" else 2e-2
        assert np.abs(got - want).max() <= tol * 4
        assert np.abs(got[:, 0]).max() < 1e-6 and np.abs(got[:, 1] - plain[:, 1]).max() <= tol * 4
        assert np.abs(got[:, 2] - plain[:, 2]).max() > 1e-3


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,G,dk,dv,rot,normed", [(4, 2, 24, 16, 12, True), (3, 3, 9, 7, 0, True), (2, 1, 64, 64, 64, False), (5, 5, 10, 12, 4, True)])
def test_between_projection_and_attention(H, G, dk, dv, rot, normed, dtype):
    """Norm per head with one weight for all heads, rotation of half-split pairs of the first ``rot`` numbers (positions far
    out as exact as near ones), unit values, and the pages they land in."""
    from mimirmind_b200.kernels import ops
    from mimirmind_b200.parts.latent_attention import split_frequencies
    rng = np.random.RandomState(dk + rot)
    n, page, eps, base = 7, 8, 1e-5, 10000.0
    positions = np.array([0, 1, 7, 8, 100000, 100001, 3])
    rows = rng.randn(n, 5 + (H + G) * dk + G * dv)
    wq, wk = 1.0 + 0.1 * rng.randn(dk), 1.0 + 0.1 * rng.randn(dk)
    x = dev(rows)
    table = None
    if rot:
        f_hi, f_lo = split_frequencies(base, rot, DEV)
        table = ops.rope_half_table(i32(positions.tolist()), f_hi, f_lo)
    q_out = torch.empty((n, H * dk), dtype=DT[dtype], device=DEV)
    kp = torch.zeros((n, G, page, dk), dtype=DT[dtype], device=DEV)
    vp = torch.zeros((n, G, page, dv), dtype=DT[dtype], device=DEV)
    slots = i32([t * page + (t % page) for t in range(n)])          # token t: page t, place t
    ops.talking_prep(x, 5, 5 + H * dk, 5 + (H + G) * dk, dev(wq) if normed else None, dev(wk) if normed else None, eps, table, rot, True, q_out, kp, vp,
                     slots, page, H, G, dk, dv)
    r32 = x.cpu().numpy().astype(np.float64)
    q = r32[:, 5:5 + H * dk].reshape(n, H, dk)
    k = r32[:, 5 + H * dk:5 + (H + G) * dk].reshape(n, G, dk)
    v = r32[:, 5 + (H + G) * dk:].reshape(n, G, dv)
    if normed:
        q, k = pz.rms(q, eps) * wq.astype(np.float32), pz.rms(k, eps) * wk.astype(np.float32)
    if rot:
        q, k = pz.rotate_half(q, positions, rot, base), pz.rotate_half(k, positions, rot, base)
    v = pz.rms(v, eps)
    tol = 3e-6 if dtype == "float32" else 1e-2
    assert np.abs(q_out.float().cpu().numpy().reshape(n, H, dk) - q).max() <= tol * np.abs(q).max()
    for t in range(n):
        assert np.abs(kp[t, :, t % page].float().cpu().numpy() - k[t]).max() <= tol * np.abs(k).max()
        assert np.abs(vp[t, :, t % page].float().cpu().numpy() - v[t]).max() <= tol * np.abs(v).max()
    assert float(kp.float().abs().sum()) > 0 and float(kp[0, :, 1:].float().abs().sum()) == 0.0


# ---- the forget gate per key channel --------------------------------------------------------------------------------------
@pytest.mark.parametrize("H,dk,dv", [(3, 16, 8), (2, 32, 64), (1, 10, 7), (4, 64, 32), (2, 100, 40), (1, 200, 33)])
def test_the_forget_gate_recurrence_against_the_plain_one(H, dk, dv):
    """Three requests of unequal length in one step (one of a single token), then each goes on in a second step from the
    state the first left, in slots somebody left full; a request at position 0 starts from zero whatever its slot holds."""
    from mimirmind_b200.kernels import ops
    rng = np.random.RandomState(dk)
    lens1, lens2 = [37, 1, 5], [1, 50, 2]
    slots = [2, 0, 3]
    ld = 3 + 2 * H * dk + H * dv
    bias, lower = rng.randn(H * dk), 1.0 / (1.0 + np.exp(-rng.randn(H * dk)))
    state = dev(rng.randn(5, H * dv * dk + 11))
    seqs = [rng.randn(a + b, ld) for a, b in zip(lens1, lens2)]
    want = []
    for s in seqs:
        x = s.astype(np.float32).astype(np.float64)
        q = pz.silu(x[:, 3:3 + H * dk]).reshape(-1, H, dk)
        low = lower.astype(np.float32).astype(np.float64)
        f = (low + (1.0 - low) * pz.sigmoid(x[:, 3 + H * dk:3 + 2 * H * dk] + bias.astype(np.float32))).reshape(-1, H, dk)
        want.append(pz.hgrn2_core(q, f, x[:, 3 + 2 * H * dk:].reshape(-1, H, dv)))
    got = [[] for _ in seqs]
    for step, lens in enumerate((lens1, lens2)):
        start = [0, 0, 0] if step == 0 else lens1
        rows = np.concatenate([s[a:a + n] for s, a, n in zip(seqs, start, lens)], 0)
        x = dev(rows)
        q_start = np.concatenate([[0], np.cumsum(lens)[:-1]])
        meta = i32([[int(q_start[r]), lens[r], start[r] + lens[r], slots[r]] for r in range(3)])
        positions = i32(sum([list(range(start[r], start[r] + lens[r])) for r in range(3)], []))
        ops.forget_gate_prep(x, 3, 3 + H * dk, H * dk, dev(bias), dev(lower))
        o = ops.forget_gate_walk(x[:, 3:3 + H * dk], x[:, 3 + H * dk:3 + 2 * H * dk], x[:, 3 + 2 * H * dk:], state, meta, i32(slots), positions, 3, H, dk, dv)
        o = o.cpu().numpy().reshape(-1, H, dv)
        for r in range(3):
            got[r].append(o[q_start[r]:q_start[r] + lens[r]])
    for r in range(3):
        g = np.concatenate(got[r], 0)
        assert np.abs(g - want[r]).max() <= 2e-5 * max(1.0, np.abs(want[r]).max())


@pytest.mark.parametrize("H,dk,dv", [(3, 16, 8), (2, 64, 40), (4, 128, 64), (1, 10, 7)])
def test_chunks_walked_side_by_side_equal_the_walk(H, dk, dv):
    """Long portions are cut into chunks of 64 tokens that are walked side by side; outputs and the states left in the
    slots equal the walk's, for a request from position 0 in a slot somebody left full and one that goes on from a state."""
    from mimirmind_b200.kernels import ops
    rng = np.random.RandomState(dv)
    lens, starts, slots = [300, 130, 64], [0, 77, 5], [1, 3, 0]
    n = sum(lens)
    q, v = dev(rng.randn(n, H * dk)), dev(rng.randn(n, H * dv))
    f = dev(1.0 / (1.0 + np.exp(-2.0 * rng.randn(n, H * dk))))
    state0 = rng.randn(4, H * dv * dk + 3)
    q_start = np.concatenate([[0], np.cumsum(lens)[:-1]])
    meta = i32([[int(q_start[r]), lens[r], starts[r] + lens[r], slots[r]] for r in range(3)])
    positions = i32(sum([list(range(starts[r], starts[r] + lens[r])) for r in range(3)], []))
    chunk_meta, req_chunks = [], []
    for r in range(3):
        first = len(chunk_meta)
        for off in range(0, lens[r], 64):
            chunk_meta.append([int(q_start[r]) + off, min(64, lens[r] - off), r, int(off == 0)])
        req_chunks.append([first, len(chunk_meta) - first])
    s_walk, s_chunk = dev(state0), dev(state0)
    want = ops.forget_gate_walk(q, f, v, s_walk, meta, i32(slots), positions, 3, H, dk, dv).cpu().numpy()
    got = ops.forget_gate_chunked(q, f, v, s_chunk, i32(chunk_meta), i32(req_chunks), i32(slots), positions, H, dk, dv).cpu().numpy()
    assert np.abs(got - want).max() <= 2e-5 * max(1.0, np.abs(want).max())
    assert np.abs(s_chunk.cpu().numpy() - s_walk.cpu().numpy()).max() <= 2e-5 * max(1.0, float(s_walk.abs().max()))
    assert np.array_equal(s_chunk.cpu().numpy()[2], state0.astype(np.float32)[2])          # a slot nobody holds is not touched


# ---- experts ----------------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("E,top", [(6, 2), (5, 5), (8, 1), (64, 6), (3, 1)])
def test_the_sigmoid_routers_choice(E, top):
    from mimirmind_b200.kernels import ops
    rng = np.random.RandomState(E)
    x, w = rng.randn(50, 48), rng.randn(E, 48) * 0.5
    idx, wts = ops.moe_router(dev(x), dev(w), top, 1, 1, scoring="sigmoid")
    want_idx, want_s = pz.router_choice(x.astype(np.float32).astype(np.float64), w.astype(np.float32).astype(np.float64), top)
    assert np.array_equal(idx.cpu().numpy(), want_idx)
    assert np.abs(wts.cpu().numpy() - want_s).max() <= 1e-6


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("n,d,ff,E,top,limit,shared", [(70, 64, 40, 6, 2, 1.5, (24, 0.8)), (1, 54, 33, 5, 5, 0.7, (17, 3.0)), (300, 128, 64, 8, 3, 2.0, None),
                                                        (9, 256, 96, 10, 1, 1.0, (96, 1.0)), (2100, 64, 32, 4, 2, 1.0, (32, 0.5))])
def test_experts_that_weigh_their_input_against_the_plain_ones(n, d, ff, E, top, limit, shared, dtype):
    from mimirmind_b200.config.spec import PartSpec
    from mimirmind_b200.parts.base import Runtime, WeightView
    from mimirmind_b200.parts.moe import RoutedExperts
    rng = np.random.RandomState(n + d)
    w = {"mlp.router": rng.randn(E, d) * 4.0 / np.sqrt(d)}
    for e in range(E):
        w.update({f"mlp.e{e}.gate": rng.randn(ff, d) / np.sqrt(d) * 2, f"mlp.e{e}.up": rng.randn(ff, d) / np.sqrt(d) * 2, f"mlp.e{e}.down": rng.randn(d, ff) / np.sqrt(ff)})
    mlp = {"router": {"top": top}, "expert": {"limit": limit}}
    shared_spec = None
    if shared:
        w.update({"mlp.shared.gate": rng.randn(shared[0], d) / np.sqrt(d) * 2, "mlp.shared.up": rng.randn(shared[0], d) / np.sqrt(d) * 2,
                  "mlp.shared.down": rng.randn(d, shared[0]) / np.sqrt(shared[0])})
        mlp["shared"] = {"limit": shared[1]}
        shared_spec = PartSpec("gated_mlp", {"hidden": d, "intermediate": shared[0], "activation": "clamped", "limit": shared[1],
                                             "gate": "mlp.shared.gate", "up": "mlp.shared.up", "down": "mlp.shared.down"})
    w = {k: bf16_round(v) for k, v in w.items()}
    x = bf16_round(rng.randn(n, d))
    spec = PartSpec("routed_experts", {"hidden": d, "ff": ff, "experts": E, "top": top, "groups": 1, "keep": 1, "router": "mlp.router", "expert": "mlp.e{}",
                                       "scoring": "sigmoid", "weight_on": "input", "activation": "clamped", "limit": limit, "shared": shared_spec})
    rt = Runtime(DT[dtype], torch.device(DEV))
    part = RoutedExperts(spec, WeightView({k: dev(v, torch.bfloat16 if dtype == "bfloat16" else torch.float32) for k, v in w.items()}), rt)
    got = part.forward(dev(x, DT[dtype]), None).float().cpu().numpy()
    want = pz.experts_feed_forward(x, w, "mlp.", mlp)
    branches = part.forward_branches(dev(x, DT[dtype]), None)
    assert len(branches) == (2 if shared else 1) and all(f == 1.0 for _t, f in branches)
    err = np.abs(got - want).max(axis=-1) / np.abs(want).max()
    if dtype == "float32":
        assert err.max() <= 2e-5
    else:
        assert np.median(err) <= 2e-2 and (err > 5e-2).mean() <= 0.02


# ---- the norm after the sum and the small passes ------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("n,d", [(5, 64), (33, 54), (2, 4096), (1, 13000)])
def test_the_norm_after_the_sum(n, d, dtype):
    from mimirmind_b200.kernels import ops
    rng = np.random.RandomState(d)
    x, a, b, w = rng.randn(n, d), rng.randn(n, d), rng.randn(n, d), 1.0 + 0.1 * rng.randn(d)
    if dtype == "bfloat16":
        a, b = bf16_round(a), bf16_round(b)
    x32, w32 = x.astype(np.float32).astype(np.float64), w.astype(np.float32).astype(np.float64)
    for use_a, use_b in ((True, True), (True, False), (False, False)):
        res = dev(x)
        out = torch.empty((n, d), dtype=DT[dtype], device=DEV)
        ops.post_norm(res, dev(a, DT[dtype]) if use_a else None, dev(b, DT[dtype]) if use_b else None, dev(w), 1e-5, 3.0, 0.8, 1.1, out=out)
        y = 3.0 * x32 + (0.8 * a if use_a else 0.0) + (1.1 * b if use_b else 0.0)
        want = pz.rms(y, 1e-5) * w32
        assert np.abs(res.cpu().numpy() - want).max() <= 1e-5 * np.abs(want).max() + 1e-6
        assert np.abs(out.float().cpu().numpy() - want).max() <= (1e-5 if dtype == "float32" else 1e-2) * np.abs(want).max()
    assert np.array_equal(ops.cast_rows(dev(x), DT[dtype]).float().cpu().numpy(), dev(x).to(DT[dtype]).float().cpu().numpy())
    s = ops.scaled_sum2(dev(a, DT[dtype]), dev(b, DT[dtype]), 0.8, 1.1).float().cpu().numpy()
    assert np.abs(s - (0.8 * a + 1.1 * b)).max() <= (1e-6 if dtype == "float32" else 2e-2) * 4


def test_the_clamped_gated_activation():
    from mimirmind_b200.kernels import ops
    rng = np.random.RandomState(2)
    gu = rng.randn(9, 2 * 21) * 3.0
    scale = rng.rand(9) + 0.5
    got = ops.glu_rows(dev(gu), torch.float32, "clamped", 1.25, row_scale=dev(scale)).cpu().numpy()
    g32 = gu.astype(np.float32).astype(np.float64) * scale.astype(np.float32)[:, None]
    g, u = np.minimum(g32[:, :21], 1.25), np.clip(g32[:, 21:], -1.25, 1.25)
    assert np.abs(got - g * pz.sigmoid(1.702 * g) * (u + 1.0)).max() <= 1e-5
    plain = ops.glu_rows(dev(gu), torch.float32, "silu").cpu().numpy()
    x = gu.astype(np.float32).astype(np.float64)
    assert np.abs(plain - pz.silu(x[:, :21]) * x[:, 21:]).max() <= 1e-5


# ---- whole models -------------------------------------------------------------------------------------------------------
@pytest.fixture(scope="module")
def models(tmp_path_factory):
    cache = {}

    def get(name, dtype="float32"):
        """The 16-bit runs get the model with every expert chosen: one expert taken for another on a near tie of rounded
        scores changes a row, and every row after it, by far more than rounding does, which says nothing about the kernels.
        The choice among experts is held to the plain implementation by the 32-bit runs and by the experts' own tests."""
        key = (name, dtype == "bfloat16")
        if key not in cache:
            cfg = zu.every_expert_chosen(zu.CONFIGS[name]) if key[1] else zu.CONFIGS[name]
            folder = zu.write_model(str(tmp_path_factory.mktemp(f"zubarax_{name}")), cfg, seed=len(cache) + 31)
            cache[key] = (folder,) + pz.load_folder(folder)
        return cache[key]

    return get


def check_rows(trace, outputs, reqs, ref, dtype, what):
    """float32: every row within the bound.  bfloat16: a bound on the typical row and on the share of rows beyond the bound;
    what a single position does at an edge is pinned by the 32-bit runs and by the tests of each mechanism alone."""
    got = ru.collect(trace, outputs)
    for rid, toks in reqs.items():
        rows = np.stack([got[(rid, p)] for p in range(len(toks))])
        err = rel_rms(rows, ref[rid])
        over = int((err > ROW_TOL[dtype]).sum())
        allowed = 0 if dtype == "float32" else max(1, int(0.2 * len(toks)))
        assert over <= allowed and not np.isnan(err).any() and (dtype == "float32" or np.median(err) <= 3e-2), (
            f"{what} {dtype} request {rid}: {over} of {len(toks)} rows above the bound, median {np.median(err):.3g}, worst {err.max():.3g} at "
            f"position {int(err.argmax())}, first above: {int(np.argmax(err > ROW_TOL[dtype]))}")
    return got


def test_every_layer_run_against_the_plain_stream(models):
    """The residual stream after every layer run (a layer that runs twice counts twice) of a short prompt, in float32."""
    from mimirmind_b200.engine.loader import load_model
    from mimirmind_b200.engine.runner import ModelRunner, StepEntry

    class Keep:
        def __init__(self):
            self.rows = {}

        def write(self, block, stage, rows):
            if stage == "l_out":
                self.rows[block] = rows.detach().float().cpu().numpy().copy()

    for name in ("A", "C"):
        folder, cfg, w = models(name)
        toks = random_tokens(cfg["vocab"], 29, 3)
        streams = []
        pz.forward(cfg, w, toks, collect=streams)
        model, _ = load_model(folder, "float32")
        runner = ModelRunner(model, page_size=16, num_pages=8, max_requests=2)
        keep = Keep()
        runner.stage_dump = keep
        runner.add_request("s")
        runner.step([StepEntry("s", toks, [28])])
        assert sorted(keep.rows) == list(range(len(cfg["layers"])))
        for i, want in enumerate(streams):
            assert np.abs(keep.rows[i] - want).max() <= 3e-5 * np.abs(want).max(), f"{name}: layer run {i}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name,page_size", [("A", 16), ("B", 16), ("C", 8), ("A", 32), ("D", 16)])
def test_every_way_of_cutting_matches_the_plain_implementation(name, page_size, dtype, models):
    folder, cfg, w = models(name, dtype)
    reqs = {f"{name}{i}": random_tokens(cfg["vocab"], n, 100 * i + n) for i, n in enumerate(zu.LENGTHS[name])}
    ref = {rid: pz.forward(cfg, w, t) for rid, t in reqs.items()}
    results = {}
    t = ru.Trace()
    for rid, toks in reqs.items():
        ru.whole(t, rid, toks)
    out, _ = ru.run_in_process(folder, dtype, t, t.max_live_tokens(), page_size)
    results["whole"] = check_rows(t, out, reqs, ref, dtype, "whole")
    t = ru.Trace()
    for rid, toks in reqs.items():
        ru.tail_one_by_one(t, rid, toks, 80)
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
        # the 32-bit kernels sum in an order fixed by position and walk every state token by token: cutting changes nothing at all
        for mode in ("tail", "chunks", "mixed"):
            for key, row in results["whole"].items():
                assert np.array_equal(results[mode][key], row), f"{mode}: {key} differs from the whole run"


@pytest.mark.parametrize("name,dtype", [("A", "float32"), ("C", "bfloat16")])
def test_decoding_from_the_first_token(name, dtype, models):
    folder, cfg, w = models(name, dtype)
    toks = random_tokens(cfg["vocab"], 260, 5)
    t = ru.Trace()
    ru.chunks(t, "d", toks, [1])
    out, _ = ru.run_in_process(folder, dtype, t, t.max_live_tokens())
    check_rows(t, out, {"d": toks}, {"d": pz.forward(cfg, w, toks)}, dtype, "decode from the first token")


def test_a_slot_used_again_starts_clean(models):
    """Two state slots, five requests one after the other and in pairs: a request never sees what the slot's last user
    left (the matrices, the convolutions' last inputs)."""
    from mimirmind_b200.engine.loader import load_model
    from mimirmind_b200.engine.runner import ModelRunner, StepEntry
    folder, cfg, w = models("A")
    model, _ = load_model(folder, "float32")
    runner = ModelRunner(model, page_size=16, num_pages=12, max_requests=2)
    reqs = [random_tokens(cfg["vocab"], n, n) for n in (60, 3, 90, 31, 64)]
    ref = [pz.forward(cfg, w, t) for t in reqs]
    assert runner.add_request(0) and runner.add_request(1) and not runner.add_request(2)
    got0 = runner.step([StepEntry(0, reqs[0][:50], [49]), StepEntry(1, reqs[1], [2])]).cpu().numpy()
    runner.release(1)
    assert runner.add_request(2)
    got1 = runner.step([StepEntry(2, reqs[2][:7], [6]), StepEntry(0, reqs[0][50:], [9])]).cpu().numpy()
    runner.release(0)
    assert runner.add_request(3)
    got2 = runner.step([StepEntry(3, reqs[3], [30]), StepEntry(2, reqs[2][7:], [82])]).cpu().numpy()
    runner.release(2), runner.release(3)
    assert runner.add_request(4)
    got3 = runner.step([StepEntry(4, reqs[4], [0, 63])]).cpu().numpy()
    for got, want in ((got0[0], ref[0][49]), (got0[1], ref[1][2]), (got1[0], ref[2][6]), (got1[1], ref[0][59]), (got2[0], ref[3][30]),
                      (got2[1], ref[2][89]), (got3[0], ref[4][0]), (got3[1], ref[4][63])):
        assert rel_rms(got, want) <= ROW_TOL["float32"]


@pytest.mark.parametrize("name,dtype", [("A", "float32"), ("B", "bfloat16")])
def test_greedy_generation_through_the_engine(name, dtype, models):
    """Engine.generate (scheduler, prompt portions, captured decode steps) picks the plain implementation's tokens."""
    from mimirmind_b200 import Engine
    folder, cfg, w = models(name, dtype)
    prompts = [random_tokens(cfg["vocab"], n, 40 + n) for n in (5, 17, 33, 64)]
    eng = Engine.from_folder(folder, dtype=dtype, page_size=16, cache_tokens=1024, max_context=512, token_budget=48, max_active=4)
    res = eng.generate(prompts, max_new_tokens=24)
    margin = 1e-4 if dtype == "float32" else 0.15
    exact = 0
    for p, r in zip(prompts, res):
        assert r.stats.generated_tokens == 24 and r.stats.finish_reason == "length"
        toks = list(p)
        for i, tok in enumerate(r.tokens):
            row = pz.forward(cfg, w, toks)[-1]
            best = int(np.argmax(row))
            exact += tok == best
            if dtype == "float32":
                assert row[tok] >= row[best] - margin, f"token {i}: engine chose {tok} ({row[tok]:.4f}), plain {best} ({row[best]:.4f})"
            toks.append(tok)
    assert exact >= (96 if dtype == "float32" else 75)
    assert eng.runner.manager.free_pages() == eng.runner.manager.total_pages()
    again = eng.generate(prompts, max_new_tokens=24)          # slots and pages used again
    if dtype == "float32":
        assert [r.tokens for r in again] == [r.tokens for r in res]


def test_the_replay_program_on_this_design(models, tmp_path):
    folder, cfg, w = models("C")
    reqs = {f"r{i}": random_tokens(cfg["vocab"], n, 11 + i) for i, n in enumerate([3, 90, 41, 150])}
    ref = {rid: pz.forward(cfg, w, t) for rid, t in reqs.items()}
    t = ru.Trace()
    ru.mixed(t, reqs, seed=3)
    t.step([("last", [1, 2, 3], [])], end=["last"])
    out = ru.run_program(folder, "float32", t, t.max_live_tokens(), str(tmp_path / "out"), cfg["vocab"])
    check_rows(t, out, reqs, ref, "float32", "program")


def test_the_command_line_generates_with_this_design(models, tmp_path):
    """bin/mimirmind: smoke generates from a test model (its greedy tokens are the plain implementation's); random-weights
    mode writes a folder of this design from its config.json, and smoke generates from that too."""
    import json
    import os
    import subprocess
    import sys
    from conftest import ROOT
    folder, cfg, w = models("A")
    exe = [sys.executable, os.path.join(ROOT, "bin", "mimirmind")]
    conf = {"defaultModel": "m", "models": [{"id": "m", "path": folder}], "runtime": {"dtype": "float32", "maxContextTokens": 256, "cacheTokens": 512}}
    (tmp_path / "config.json").write_text(json.dumps(conf))
    out = subprocess.run(exe + ["smoke", "--config", str(tmp_path / "config.json"), "--prompt", "5 17 3 99", "--max-new", "6"],
                         capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stderr
    lines = out.stdout.strip().splitlines()
    got = [int(t) for t in lines[0].split()]
    assert len(got) == 6 and lines[1] == "generated 6"
    toks = [5, 17, 3, 99]
    for tok in got:
        row = pz.forward(cfg, w, toks)[-1]
        assert row[tok] >= row.max() - 1e-4
        toks.append(tok)
    (tmp_path / "mc.json").write_text(json.dumps(zu.CONFIGS["B"]))
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
