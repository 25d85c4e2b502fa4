"""Choice of attention kernel for a step.

The 32-bit path and head sizes the tensor-core kernels are not built for run the
position-aligned fp32 kernel; bfloat16 with a supported head size runs the tensor-core
kernels: a tiled prefill kernel for long portions and a split-key kernel for short ones.
The reference dispatches the same way on the query length (decode vs prefill flash,
src/compute/cuda/GpuOps.cpp:2711-2731).
"""
from __future__ import annotations

import torch

from . import ops


def paged_attention(q, cache, out, ctx, num_heads: int, num_kv_heads: int, head_dim: int, window: int,
                    scale: float) -> torch.Tensor:
    if q.dtype == torch.bfloat16:
        from . import attention_bf16
        if attention_bf16.supports(head_dim, num_heads, num_kv_heads):
            return attention_bf16.run(q, cache, out, ctx, num_heads, num_kv_heads, head_dim, window, scale)
    return ops.attention_generic(q, cache.k_pages, cache.v_pages, out, ctx.positions, ctx.token_req,
                                 cache.block_table, cache.page_size, num_heads, num_kv_heads, head_dim, window, scale)


USE_SINK_TMA_DECODE = True   # False: single tokens never take the TMA decode kernel
USE_SINK_TCGEN05 = True    # False: portions never take the tcgen05 prefill kernel (tests compare it with the mma.sync one)
USE_SINK_MMA = True        # False: the sink attention always runs the fp32-arithmetic kernel (tests compare the two)
SINK_PREFILL_MIN = 16      # shorter portions go token by token through the decode kernel
SINK_TILE_ROWS = 64
_sink_declared = False


def _sink_lib():
    global _sink_declared
    from ctypes import c_float, c_int, c_void_p
    from . import lib as _lib
    if not _sink_declared:
        P, I, F = c_void_p, c_int, c_float
        _lib.declare("mm_attention_sink_supported", [I, I])
        _lib.declare("mm_attention_sink_prefill_bf16", [P, P, P, P, P, I, P, I, I, I, I, I, I, I, F, I, P, P, I, F, I, I, P])
        _lib.declare("mm_attention_sink_decode_bf16", [P, P, P, P, P, P, I, P, I, P, P, P, I, I, I, I, I, I, I, F, I, P, P, I, F, I, I, P])
        _lib.declare("mm_attention_decode_tma_bf16_sink", [P, P, P, P, P, I, P, P, P, I, I, I, I, I, I, I, F, I, I, I, P, P])
        _lib.declare("mm_attention_prefill_tcgen05_sink", [P, P, P, P, P, I, P, I, I, I, I, I, I, I, I, F, I, P, P])
        _sink_declared = True
    return _lib.load()


SINK_TARGET_CTAS = 2 * 148     # decode CTAs wanted: the key tiles of a token are shared out until the GPU is full
SINK_MAX_SPLITS = 16


def sink_splits(n_items: int, num_kv_heads: int, window: int, max_kv_len: int) -> int:
    """CTAs per (token, KV head) of the decode kernel: enough to fill the GPU, never more than the token has key tiles."""
    ctas = max(1, n_items * num_kv_heads)
    if ctas >= SINK_TARGET_CTAS // 2:
        return 1
    keys = min(window, max_kv_len) if window > 0 else max_kv_len
    return max(1, min(-(-SINK_TARGET_CTAS // ctas), -(-keys // 64), SINK_MAX_SPLITS))


def sink_plan(ctx, n_tokens: int, tile_rows: int = SINK_TILE_ROWS):
    """The step's tokens sorted once, on the host, into prefill tiles (``tile_rows`` query tokens of one request; portions
    of at least SINK_PREFILL_MIN tokens) and decode items (single tokens); every layer of the step reuses it.  Returns
    (tiles [n, 4] or None, n_tiles, items [m] or None, n_items); items None with n_items > 0 means every token."""
    key = ("sink_attention_plan", tile_rows)
    plan = ctx.plans.get(key)
    if plan is None:
        tiles, items = [], []
        for r in range(ctx.n_requests):
            s, n, kv = ctx.q_start[r], ctx.q_len[r], ctx.kv_len[r]
            if n >= SINK_PREFILL_MIN:
                for off in range(0, n, tile_rows):
                    tiles.append((r, s + off, min(tile_rows, n - off), kv - n + off))
            else:
                items.extend(range(s, s + n))
        tiles.sort(key=lambda tile: tile[3] + tile[2])
        device = ctx.positions.device
        # from pinned memory, without waiting: a copy from pageable memory would hold the host until the device has
        # caught up, and the layers after it would be launched into an empty queue
        staged = []

        def to_device(rows):
            host = torch.tensor(rows, dtype=torch.int32).pin_memory()
            staged.append(host)
            return host.to(device, non_blocking=True)

        d_tiles = to_device(tiles) if tiles else None
        d_items = None if len(items) == n_tokens or not items else to_device(items)
        plan = ctx.plans[key] = (d_tiles, len(tiles), d_items, len(items))
        ctx.plans[key + ("staged",)] = staged                  # the pinned copies live as long as the step's context
    return plan


def paged_sink_attention(q, cache, out, ctx, num_heads: int, num_kv_heads: int, key_dim: int, value_dim: int, window: int,
                         scale: float, sink: bool, sink_logit=None, dist_bias=None, softcap: float = 0.0, value_heads=None,
                         k_pages=None, v_pages=None, value_row=None) -> torch.Tensor:
    """Windowed attention with a softmax sink over pools of keys ``[pages, G, page, key_dim]`` and values
    ``[pages, G, page, value_dim]``.  bfloat16 with key and value sizes the tensor-core kernels are built for: a tiled
    kernel for portions, a kernel that shares keys between the query heads of a KV head for single tokens; anything
    else: the fp32-arithmetic kernel.

    ``softcap`` > 0 bends the scaled score into ``cap * tanh(score / cap)``.  ``value_heads`` (a divisor of the key heads):
    the value pool has that many heads and key head ``g`` reads value head ``g mod value_heads`` (several key heads over one
    set of values).  ``k_pages`` / ``v_pages``: the pools, if they are not the cache's arrays ``k`` and ``v``; ``value_row``:
    how many numbers lie between the values of consecutive tokens (values that are a slice of a wider per-token array).
    ``out`` may be fp32 beside bfloat16 queries: the result is then not rounded (what follows takes a difference of heads)."""
    table = cache.block_table
    k_pages = cache.arrays["k"] if k_pages is None else k_pages
    v_pages = cache.arrays["v"] if v_pages is None else v_pages
    value_heads = num_kv_heads if value_heads is None else int(value_heads)
    value_row = value_dim if value_row is None else int(value_row)
    if (USE_SINK_MMA and value_row == value_dim and q.dtype == torch.bfloat16 and scale > 0 and num_heads // num_kv_heads <= 16
            and _sink_lib().mm_attention_sink_supported(key_dim, value_dim)):
        from .lib import check
        lib = _sink_lib()
        # equal key and value sizes of 64 or 128: the tcgen05 prefill kernel of the plain attention, told of the sink
        from . import attention_bf16
        # a learned sink or a distance bias: the mma.sync kernels take them, the tcgen05 and TMA kernels do not
        out_f32 = int(out.dtype == torch.float32)
        extended = sink_logit is not None or dist_bias is not None or softcap > 0 or value_heads != num_kv_heads or bool(out_f32)
        sink_ptr = sink_logit.data_ptr() if sink_logit is not None else None
        bias_ptr = dist_bias.data_ptr() if dist_bias is not None else None
        dist_max = dist_bias.shape[1] - 1 if dist_bias is not None else 0
        tensor_memory = (USE_SINK_TCGEN05 and not extended and key_dim == value_dim
                         and attention_bf16.tcgen05_prefill_usable(key_dim, cache.page_size))
        tiles, n_tiles, items, n_items = sink_plan(ctx, q.shape[0], attention_bf16.TILE_ROWS_TC if tensor_memory else SINK_TILE_ROWS)
        stream = ops._stream()
        if n_tiles and tensor_memory:
            check(lib.mm_attention_prefill_tcgen05_sink(q.data_ptr(), k_pages.data_ptr(), v_pages.data_ptr(), out.data_ptr(), tiles.data_ptr(),
                                                        n_tiles, table.data_ptr(), table.shape[1], cache.page_size, k_pages.shape[0],
                                                        q.shape[0], num_heads, num_kv_heads, key_dim, int(window), float(scale),
                                                        int(bool(sink)), ops.tcgen05_error_flag(q.device).data_ptr(), stream),
                  "attention_prefill_tcgen05_sink")
        elif n_tiles:
            check(lib.mm_attention_sink_prefill_bf16(q.data_ptr(), k_pages.data_ptr(), v_pages.data_ptr(), out.data_ptr(), tiles.data_ptr(),
                                                     n_tiles, table.data_ptr(), table.shape[1], cache.page_size, num_heads, num_kv_heads,
                                                     key_dim, value_dim, int(window), float(scale), int(bool(sink)), sink_ptr, bias_ptr, dist_max,
                                                     float(softcap), value_heads, out_f32, stream),
                  "attention_sink_prefill_bf16")
        tma = None
        if n_items and USE_SINK_TMA_DECODE and not extended and key_dim == value_dim and key_dim in (64, 128) and cache.page_size in (8, 16, 32, 64):
            # equal key and value sizes of 64 or 128: the TMA decode kernel of the plain attention, in the forms that
            # finish a row inside the kernel (one split, or the splits of a token as one cluster)
            keys = min(window, ctx.max_kv_len) if window > 0 else ctx.max_kv_len
            _len, max_splits, cluster = attention_bf16.choose_split(n_items, num_kv_heads, keys, key_dim, cache.page_size)
            if cluster or max_splits == 1:
                tma = (max_splits, cluster)
        if tma is not None:
            check(lib.mm_attention_decode_tma_bf16_sink(q.data_ptr(), k_pages.data_ptr(), v_pages.data_ptr(), out.data_ptr(),
                                                        items.data_ptr() if items is not None else None, n_items, ctx.positions.data_ptr(),
                                                        ctx.token_req.data_ptr(), table.data_ptr(), table.shape[1], cache.page_size,
                                                        k_pages.shape[0], num_heads, num_kv_heads, key_dim, int(window), float(scale),
                                                        tma[0], int(tma[1]), int(bool(sink)), ops.tcgen05_error_flag(q.device).data_ptr(), stream),
                  "attention_decode_tma_bf16_sink")
        elif n_items:
            splits = sink_splits(n_items, num_kv_heads, window, ctx.max_kv_len)
            part_o = part_ml = None
            if splits > 1:
                skey = ("sink_attention_scratch", n_items, num_heads, splits, value_dim)
                if skey not in ctx.plans:
                    ctx.plans[skey] = (torch.empty((n_items, num_heads, splits, value_dim), dtype=torch.float32, device=q.device),
                                       torch.empty((n_items, num_heads, splits, 2), dtype=torch.float32, device=q.device))
                part_o, part_ml = ctx.plans[skey]
            check(lib.mm_attention_sink_decode_bf16(q.data_ptr(), k_pages.data_ptr(), v_pages.data_ptr(), out.data_ptr(),
                                                    part_o.data_ptr() if part_o is not None else None,
                                                    part_ml.data_ptr() if part_ml is not None else None, splits,
                                                    items.data_ptr() if items is not None else None, n_items, ctx.positions.data_ptr(),
                                                    ctx.token_req.data_ptr(), table.data_ptr(), table.shape[1], cache.page_size, num_heads,
                                                    num_kv_heads, key_dim, value_dim, int(window), float(scale), int(bool(sink)), sink_ptr, bias_ptr,
                                                    dist_max, float(softcap), value_heads, out_f32, stream),
                  "attention_sink_decode_bf16")
        return out
    return ops.attention_sink_generic(q, k_pages, v_pages, out, ctx.positions, ctx.token_req, table, cache.page_size, num_heads,
                                      num_kv_heads, key_dim, value_dim, window, scale, sink, sink_logit=sink_logit, dist_bias=dist_bias,
                                      softcap=softcap, value_heads=value_heads, value_row=value_row)


USE_LATENT_MMA = True      # False: the latent attention always runs the fp32-arithmetic kernel (tests compare the two)
LATENT_TILE_ROWS = 32
USE_LATENT_WIDE_TILES = True    # False: tiles of 32 rows also for portions of prompts (tests run both)
LATENT_KEYS = 32
_latent_declared = False


def _latent_lib():
    global _latent_declared
    from ctypes import c_float, c_int, c_void_p
    from . import lib as _lib
    if not _latent_declared:
        P, I, F = c_void_p, c_int, c_float
        _lib.declare("mm_attention_latent_supported", [I, I])
        _lib.declare("mm_attention_latent_tile_rows", [I])
        _lib.declare("mm_attention_latent_bf16", [P, P, P, P, P, I, P, I, I, I, P, P, I, I, I, I, I, I, F, I, P])
        _latent_declared = True
    return _lib.load()


def latent_plan(ctx, num_heads: int, tile_rows: int = LATENT_TILE_ROWS):
    """The step's (token, head) pairs cut once, on the host, into tiles of at most ``tile_rows`` rows of one request:
    several tokens with all their heads, or one token with a slice of its heads.  A tile names tokens, not positions
    (the kernel reads those from the device), so a captured step replays the same plan.  Returns (tiles [n, 5], n)."""
    key = ("latent_attention_plan", num_heads, tile_rows)
    plan = ctx.plans.get(key)
    if plan is None:
        tiles = []
        per = max(1, tile_rows // num_heads)
        for r in range(ctx.n_requests):
            s, n, kv = ctx.q_start[r], ctx.q_len[r], ctx.kv_len[r]
            for off in range(0, n, per):
                tokens = min(per, n - off)
                for h0 in range(0, num_heads, tile_rows):
                    tiles.append((kv - n + off + tokens, r, s + off, tokens, h0, min(tile_rows, num_heads - h0)))
        tiles.sort(key=lambda t: t[0])           # the kernel starts the last (longest) tiles first
        host = torch.tensor([t[1:] for t in tiles], dtype=torch.int32).reshape(-1, 5).pin_memory()
        plan = ctx.plans[key] = (host.to(ctx.positions.device, non_blocking=True), len(tiles))
        ctx.plans[key + ("staged",)] = host
    return plan


def paged_latent_attention(q, pages, cache, out, ctx, num_heads: int, wide: int, rank: int, window: int, scale: float) -> torch.Tensor:
    """Attention of ``num_heads`` query heads of ``wide`` numbers over one shared key head ``pages`` [pages, 1, page, wide]
    whose leading ``rank`` numbers are the value; ``out`` [n, num_heads * rank].  bfloat16 with a rank the tensor-core
    kernel is built for: that kernel, its key tiles shared out over several CTAs while the step has few query tiles;
    anything else: the fp32-arithmetic kernel."""
    if USE_LATENT_MMA and q.dtype == torch.bfloat16 and scale > 0 and _latent_lib().mm_attention_latent_supported(wide, rank):
        from .lib import check
        lib = _latent_lib()
        # portions of prompts: tiles of 64 rows (two 16-row tiles per warp, half the key traffic per row) where they fit
        tile_rows = 64 if USE_LATENT_WIDE_TILES and ctx.max_q_len * num_heads >= 64 and lib.mm_attention_latent_tile_rows(wide) == 64 else LATENT_TILE_ROWS
        tiles, n_tiles = latent_plan(ctx, num_heads, tile_rows)
        keys = min(window, ctx.max_kv_len) if window > 0 else ctx.max_kv_len
        splits = 1
        if n_tiles < SINK_TARGET_CTAS // 2:
            splits = max(1, min(-(-SINK_TARGET_CTAS // n_tiles), -(-keys // (4 * LATENT_KEYS)), SINK_MAX_SPLITS))
        n_rows = q.shape[0] * num_heads
        part_o = part_ml = None
        if splits > 1:
            skey = ("latent_attention_scratch", n_rows, splits, rank)
            if skey not in ctx.plans:
                ctx.plans[skey] = (torch.empty((n_rows, splits, rank), dtype=torch.float32, device=q.device),
                                   torch.empty((n_rows, splits, 2), dtype=torch.float32, device=q.device))
            part_o, part_ml = ctx.plans[skey]
        check(lib.mm_attention_latent_bf16(q.data_ptr(), pages.data_ptr(), out.data_ptr(),
                                           part_o.data_ptr() if part_o is not None else None,
                                           part_ml.data_ptr() if part_ml is not None else None, splits, tiles.data_ptr(), n_tiles, tile_rows, n_rows,
                                           ctx.positions.data_ptr(), cache.block_table.data_ptr(), cache.block_table.shape[1],
                                           cache.page_size, num_heads, wide, rank, int(window), float(scale),
                                           int(out.dtype == torch.float32), ops._stream()), "attention_latent_bf16")
        return out
    return ops.attention_sink_generic(q, pages, pages, out, ctx.positions, ctx.token_req, cache.block_table, cache.page_size, num_heads,
                                      1, wide, rank, window, scale, False, value_heads=1, value_row=wide)


TALKING_TARGET_CTAS = 2 * 148    # blocks wanted by a step of few tokens: a token's keys are shared out until the GPU is full
TALKING_MAX_SPLITS = 32


def talking_splits(n_tokens: int, window: int, max_kv_len: int, dtype) -> int:
    """Blocks per token of the fp32-arithmetic kernel with mixed heads.  A float32 run never splits: the order of its sums
    then depends on the token's position only, whatever else is in the step."""
    if dtype == torch.float32 or n_tokens >= TALKING_TARGET_CTAS // 2:
        return 1
    keys = min(window, max_kv_len) if window > 0 else max_kv_len
    return max(1, min(-(-TALKING_TARGET_CTAS // n_tokens), -(-keys // 128), TALKING_MAX_SPLITS))


USE_TALKING_MMA = True       # False: the attention with mixed heads always runs the fp32-arithmetic kernel (tests compare the two)
TALKING_TILE_ROWS = 16
_talking_declared = False


def _talking_lib():
    global _talking_declared
    from ctypes import c_float, c_int, c_void_p
    from . import lib as _lib
    if not _talking_declared:
        P, I, F = c_void_p, c_int, c_float
        _lib.declare("mm_attention_talking_mma_supported", [I, I, I, I])
        _lib.declare("mm_attention_talking_mma", [P, P, P, P, P, P, I, P, I, I, P, P, P, I, I, I, I, I, I, I, F, P, P, P])
        _talking_declared = True
    return _lib.load()


def talking_plan(ctx):
    """The step's tokens cut once, on the host, into tiles of at most 16 consecutive tokens of one request; a tile names
    tokens, not positions (the kernel reads those from the device), so a captured step replays the same plan.  Returns
    (tiles [n, 2] on the device, n)."""
    key = ("talking_attention_plan",)
    plan = ctx.plans.get(key)
    if plan is None:
        tiles = []
        for r in range(ctx.n_requests):
            s, n, kv = ctx.q_start[r], ctx.q_len[r], ctx.kv_len[r]
            for off in range(0, n, TALKING_TILE_ROWS):
                rows = min(TALKING_TILE_ROWS, n - off)
                tiles.append((kv - n + off + rows, s + off, rows))
        tiles.sort(key=lambda t: -t[0])           # the tiles with the most keys start first
        host = torch.tensor([t[1:] for t in tiles], dtype=torch.int32).reshape(-1, 2).pin_memory()
        plan = ctx.plans[key] = (host.to(ctx.positions.device, non_blocking=True), len(tiles))
        ctx.plans[key + ("staged",)] = host
    return plan


def paged_talking_attention(q, cache, out, ctx, num_heads: int, num_kv_heads: int, key_dim: int, value_dim: int, window: int,
                            scale: float, talk, sink) -> torch.Tensor:
    """Attention whose scaled scores are mixed between the heads before the softmax (``talk`` [H, H] or None), with a
    learned sink per head (or None), over pools of keys ``[pages, G, page, key_dim]`` and values ``[pages, G, page, value_dim]``.
    bfloat16 with sizes the tensor-core kernel takes: that kernel, for portions and single tokens alike, its key tiles shared
    out over several CTAs while the step has few tiles of tokens; anything else, and the 32-bit mode: the fp32-arithmetic kernel."""
    n = q.shape[0]
    k_pages, v_pages = cache.arrays["k"], cache.arrays["v"]
    if USE_TALKING_MMA and q.dtype == torch.bfloat16 and out.dtype == torch.bfloat16 and \
            _talking_lib().mm_attention_talking_mma_supported(num_heads, num_kv_heads, key_dim, value_dim):
        from .lib import check
        lib = _talking_lib()
        tiles, n_tiles = talking_plan(ctx)
        keys = min(window, ctx.max_kv_len) if window > 0 else ctx.max_kv_len
        splits = 1
        if n_tiles < TALKING_TARGET_CTAS // 2:
            splits = max(1, min(-(-TALKING_TARGET_CTAS // n_tiles), -(-keys // 64), TALKING_MAX_SPLITS))
        part_o = part_ml = None
        if splits > 1:
            skey = ("talking_attention_scratch", n, num_heads, splits, value_dim)
            if skey not in ctx.plans:
                ctx.plans[skey] = (torch.empty((n, num_heads, splits, value_dim), dtype=torch.float32, device=q.device),
                                   torch.empty((n, num_heads, splits, 2), dtype=torch.float32, device=q.device))
            part_o, part_ml = ctx.plans[skey]
        check(lib.mm_attention_talking_mma(q.data_ptr(), k_pages.data_ptr(), v_pages.data_ptr(), out.data_ptr(),
                                           part_o.data_ptr() if part_o is not None else None,
                                           part_ml.data_ptr() if part_ml is not None else None, splits, tiles.data_ptr(), n_tiles, n,
                                           ctx.positions.data_ptr(), ctx.token_req.data_ptr(), cache.block_table.data_ptr(),
                                           cache.block_table.shape[1], cache.page_size, num_heads, num_kv_heads, key_dim, value_dim, int(window),
                                           float(scale), talk.data_ptr() if talk is not None else None,
                                           sink.data_ptr() if sink is not None else None, ops._stream()), "attention_talking_mma")
        return out
    splits = talking_splits(n, window, ctx.max_kv_len, q.dtype)
    scratch = None
    if splits > 1:
        skey = ("talking_attention_scratch", n, num_heads, splits, value_dim)
        if skey not in ctx.plans:
            ctx.plans[skey] = (torch.empty((n, num_heads, splits, value_dim), dtype=torch.float32, device=q.device),
                               torch.empty((n, num_heads, splits, 2), dtype=torch.float32, device=q.device))
        scratch = ctx.plans[skey]
    return ops.attention_talking(q, k_pages, v_pages, out, ctx.positions, ctx.token_req, cache.block_table, cache.page_size,
                                 num_heads, num_kv_heads, key_dim, value_dim, window, scale, talk, sink, splits=splits, scratch=scratch)
