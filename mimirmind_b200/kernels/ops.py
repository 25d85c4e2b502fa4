"""Tensor-level wrappers of the kernel library.

Each function checks devices, dtypes, shapes and contiguity on the host, then launches
on the current CUDA stream.  torch is used for allocation and streams only; every
operation here runs a kernel of this library.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from . import lib as _lib
from .lib import KernelError, check

F32, BF16 = 0, 1


def dtype_code(dt: torch.dtype) -> int:
    if dt == torch.float32:
        return F32
    if dt == torch.bfloat16:
        return BF16
    raise KernelError(f"dtype {dt} is not supported by the kernels (float32 or bfloat16)")


def _stream() -> int:
    """The current stream's handle (of the current device): the raw query, a hundred times cheaper than building a
    torch.cuda.Stream object for every launch."""
    return torch._C._cuda_getCurrentRawStream(torch._C._cuda_getDevice())


def _need(t: torch.Tensor, what: str, dtype: Optional[torch.dtype] = None) -> None:
    if not isinstance(t, torch.Tensor) or not t.is_cuda:
        raise KernelError(f"{what}: expected a CUDA tensor")
    if not t.is_contiguous():
        raise KernelError(f"{what}: tensor must be contiguous")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{what}: expected {dtype}, got {t.dtype}")


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def embedding(ids: torch.Tensor, table: torch.Tensor, out: torch.Tensor, scale: float = 1.0) -> torch.Tensor:
    """out[t,:] = table[ids[t],:] * scale as fp32; ids outside the table give zero rows."""
    _need(ids, "embedding ids", torch.int32)
    _need(table, "embedding table")
    _need(out, "embedding out", torch.float32)
    n, (v, d) = ids.numel(), table.shape
    if out.shape != (n, d):
        raise KernelError(f"embedding: out is {tuple(out.shape)}, expected {(n, d)}")
    check(_lib.load().mm_embedding(ids.data_ptr(), table.data_ptr(), dtype_code(table.dtype), out.data_ptr(), n, v, d,
                                   float(scale), _stream()), "embedding")
    return out


def add_rmsnorm(residual: torch.Tensor, delta: Optional[torch.Tensor], weight: torch.Tensor, eps: float,
                out: torch.Tensor, rows: Optional[torch.Tensor] = None) -> torch.Tensor:
    """residual (fp32) += delta, out = rmsnorm(residual) * weight.  With ``rows`` output row i comes
    from source row rows[i] and the residual is left untouched."""
    _need(residual, "rmsnorm residual", torch.float32)
    _need(weight, "rmsnorm weight")
    _need(out, "rmsnorm out")
    d = residual.shape[-1]
    n_out = out.shape[0]
    if weight.shape != (d,) or out.shape[-1] != d:
        raise KernelError("rmsnorm: width mismatch")
    if delta is not None:
        _need(delta, "rmsnorm delta", out.dtype)
        if delta.shape != residual.shape:
            raise KernelError("rmsnorm: delta and residual differ in shape")
    if rows is not None:
        _need(rows, "rmsnorm rows", torch.int32)
        if rows.numel() != n_out:
            raise KernelError("rmsnorm: rows and out differ in length")
    elif n_out != residual.shape[0]:
        raise KernelError("rmsnorm: out and residual differ in rows")
    check(_lib.load().mm_add_rmsnorm(residual.data_ptr(), _ptr(delta), _ptr(rows), weight.data_ptr(),
                                     dtype_code(weight.dtype), out.data_ptr(), dtype_code(out.dtype), n_out, d,
                                     float(eps), _stream()), "rmsnorm")
    return out


def add_residual(residual: torch.Tensor, delta: torch.Tensor) -> torch.Tensor:
    _need(residual, "add_residual residual", torch.float32)
    _need(delta, "add_residual delta")
    if delta.shape != residual.shape:
        raise KernelError("add_residual: shapes differ")
    check(_lib.load().mm_add_residual(residual.data_ptr(), delta.data_ptr(), dtype_code(delta.dtype), residual.numel(),
                                      _stream()), "add_residual")
    return residual


def silu_mul(gate_up: torch.Tensor, out: torch.Tensor, interleave: int = 0) -> torch.Tensor:
    """out[n,f] = silu(gate) * up.  interleave 0: gate_up[n,f] and gate_up[n,F+f]; interleave 8: gate and
    up alternate in blocks of 8 columns."""
    _need(gate_up, "silu_mul input")
    _need(out, "silu_mul out", gate_up.dtype)
    n, two_f = gate_up.shape
    if two_f % 2 or out.shape != (n, two_f // 2):
        raise KernelError("silu_mul: shapes do not match [n,2F] -> [n,F]")
    check(_lib.load().mm_silu_mul(gate_up.data_ptr(), out.data_ptr(), dtype_code(out.dtype), n, two_f // 2, interleave,
                                  _stream()), "silu_mul")
    return out


def qkv_rope_kvwrite(qkv: torch.Tensor, bias: Optional[torch.Tensor], q_out: torch.Tensor,
                     k_pages: Optional[torch.Tensor], v_pages: Optional[torch.Tensor], positions: torch.Tensor,
                     token_req: torch.Tensor, block_table: torch.Tensor, page_size: int, num_heads: int,
                     num_kv_heads: int, head_dim: int, rotary_dim: int, theta: float, interleave: bool = False) -> None:
    """Adds the bias, rotates q and k by position, writes q to ``q_out`` and k, v into their pages.
    ``interleave``: the q and k columns of ``qkv`` and ``bias`` are in the order of :func:`interleave_halves`."""
    _need(qkv, "qkv")
    n = qkv.shape[0]
    width = (num_heads + 2 * num_kv_heads) * head_dim
    if qkv.shape != (n, width):
        raise KernelError(f"qkv: shape {tuple(qkv.shape)} is not [n, {width}]")
    _need(q_out, "q_out", qkv.dtype)
    if q_out.shape != (n, num_heads * head_dim):
        raise KernelError("q_out: wrong shape")
    if bias is not None:
        _need(bias, "qkv bias")
        if bias.shape != (width,):
            raise KernelError("qkv bias: wrong shape")
    if k_pages is not None:
        for name, pool in (("k_pages", k_pages), ("v_pages", v_pages)):
            _need(pool, name, qkv.dtype)
            if pool.dim() != 4 or pool.shape[1:] != (num_kv_heads, page_size, head_dim):
                raise KernelError(f"{name}: shape {tuple(pool.shape)} is not [pages, {num_kv_heads}, {page_size}, {head_dim}]")
    _need(positions, "positions", torch.int32)
    _need(token_req, "token_req", torch.int32)
    _need(block_table, "block_table", torch.int32)
    if block_table.dim() != 2:
        raise KernelError("block_table: expected [requests, width]")
    check(_lib.load().mm_qkv_rope_kvwrite(
        qkv.data_ptr(), _ptr(bias), dtype_code(bias.dtype) if bias is not None else F32, q_out.data_ptr(),
        _ptr(k_pages), _ptr(v_pages), dtype_code(qkv.dtype), positions.data_ptr(), token_req.data_ptr(),
        block_table.data_ptr(), block_table.shape[1], page_size, n, num_heads, num_kv_heads, head_dim, rotary_dim,
        float(theta), int(interleave), _stream()), "qkv_rope_kvwrite")


def qkv_rope_tables(qkv: torch.Tensor, bias: Optional[torch.Tensor], q_out: torch.Tensor,
                    k_pages: Optional[torch.Tensor], v_pages: Optional[torch.Tensor], table: torch.Tensor,
                    slots: Optional[torch.Tensor], page_size: int, num_heads: int, num_kv_heads: int, head_dim: int,
                    interleave: bool = False) -> None:
    """:func:`qkv_rope_kvwrite` for bfloat16 and a rotation of the whole head, with the step's tables: ``table``
    from :func:`rope_table`, ``slots`` from :func:`slot_mapping` (needed when there are pages to write)."""
    _need(qkv, "qkv", torch.bfloat16)
    n = qkv.shape[0]
    width = (num_heads + 2 * num_kv_heads) * head_dim
    if qkv.shape != (n, width):
        raise KernelError(f"qkv: shape {tuple(qkv.shape)} is not [n, {width}]")
    if head_dim % 16:
        raise KernelError(f"qkv_rope_tables: head size {head_dim} is not a multiple of 16")
    _need(q_out, "q_out", torch.bfloat16)
    if q_out.shape != (n, num_heads * head_dim):
        raise KernelError("q_out: wrong shape")
    if bias is not None:
        _need(bias, "qkv bias")
        if bias.shape != (width,):
            raise KernelError("qkv bias: wrong shape")
    _need(table, "rope table", torch.float32)
    if table.shape != (n, head_dim):
        raise KernelError(f"rope table: shape {tuple(table.shape)} is not [{n}, {head_dim}]")
    if k_pages is not None:
        for name, pool in (("k_pages", k_pages), ("v_pages", v_pages)):
            _need(pool, name, torch.bfloat16)
            if pool.dim() != 4 or pool.shape[1:] != (num_kv_heads, page_size, head_dim):
                raise KernelError(f"{name}: shape {tuple(pool.shape)} is not [pages, {num_kv_heads}, {page_size}, {head_dim}]")
        if slots is None:
            raise KernelError("qkv_rope_tables: pages without slots")
        _need(slots, "slots", torch.int32)
        if slots.shape != (n,):
            raise KernelError("slots: wrong shape")
    check(_lib.load().mm_qkv_rope_tables(
        qkv.data_ptr(), _ptr(bias), dtype_code(bias.dtype) if bias is not None else F32, q_out.data_ptr(),
        _ptr(k_pages), _ptr(v_pages), table.data_ptr(), _ptr(slots), page_size, n, num_heads, num_kv_heads, head_dim,
        int(interleave), _stream()), "qkv_rope_tables")


def gather_rows(src: torch.Tensor, rows: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    _need(src, "gather src")
    _need(rows, "gather rows", torch.int32)
    _need(out, "gather out", src.dtype)
    check(_lib.load().mm_gather_rows(src.data_ptr(), rows.data_ptr(), out.data_ptr(), dtype_code(src.dtype),
                                     rows.numel(), src.shape[-1], _stream()), "gather_rows")
    return out


def attention_generic(q: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor, out: torch.Tensor,
                      positions: torch.Tensor, token_req: torch.Tensor, block_table: torch.Tensor, page_size: int,
                      num_heads: int, num_kv_heads: int, head_dim: int, window: int, scale: float) -> torch.Tensor:
    """Causal attention of every token over its request's pages (fp32 arithmetic, any head size)."""
    _need(q, "attention q")
    n = q.shape[0]
    _need(out, "attention out", q.dtype)
    _need(k_pages, "attention k_pages", q.dtype)
    _need(v_pages, "attention v_pages", q.dtype)
    if q.shape != (n, num_heads * head_dim) or out.shape != q.shape:
        raise KernelError("attention: q/out shape mismatch")
    if k_pages.shape[1:] != (num_kv_heads, page_size, head_dim) or v_pages.shape != k_pages.shape:
        raise KernelError("attention: page pool shape mismatch")
    _need(positions, "positions", torch.int32)
    _need(token_req, "token_req", torch.int32)
    _need(block_table, "block_table", torch.int32)
    check(_lib.load().mm_attention_generic(
        q.data_ptr(), k_pages.data_ptr(), v_pages.data_ptr(), out.data_ptr(), dtype_code(q.dtype), positions.data_ptr(),
        token_req.data_ptr(), block_table.data_ptr(), block_table.shape[1], page_size, n, num_heads, num_kv_heads,
        head_dim, window, float(scale), _stream()), "attention_generic")
    return out


def gemm_simt(a: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor) -> torch.Tensor:
    """out[M,N] = a[M,K] @ w[N,K]^T (+ bias) on the fp32 FMA units, k summed in ascending order."""
    _need(a, "gemm a")
    _need(w, "gemm w")
    _need(out, "gemm out")
    m, k = a.shape
    n = w.shape[0]
    if w.shape != (n, k) or out.shape != (m, n):
        raise KernelError(f"gemm: shapes a{tuple(a.shape)} w{tuple(w.shape)} out{tuple(out.shape)} do not match")
    if bias is not None:
        _need(bias, "gemm bias")
        if bias.shape != (n,):
            raise KernelError("gemm: bias shape mismatch")
    check(_lib.load().mm_gemm_simt(a.data_ptr(), dtype_code(a.dtype), w.data_ptr(), dtype_code(w.dtype), _ptr(bias),
                                   dtype_code(bias.dtype) if bias is not None else F32, out.data_ptr(),
                                   dtype_code(out.dtype), m, n, k, k, n, _stream()), "gemm_simt")
    return out


GEMV_MAX_ROWS = 8      # measured on B200 (7B shapes, 8 layers, whole decode step): from 9 rows on the tcgen05 product is ahead of the register-streaming kernel's two-tile variant (9 rows 1.15 vs 1.25 ms, 12 rows 1.20 vs 1.30 ms)


# Above the streaming kernel's rows and up to here the tcgen05 weight-streaming product (with the fused epilogues) is
# used.  Measured per layer on B200 (7B shapes, sum of the four products against library products + separate norm,
# rotary and activation kernels): 16 rows 94.6 vs 106.9 us, 64 rows 100.6 vs 109.8 us, 128 rows 119 vs 114 us.
SKINNY_MAX_ROWS = 64


def gemv_supported(m: int, n: int, k: int) -> bool:
    return 1 <= m <= GEMV_MAX_ROWS and n % 16 == 0 and k % 32 == 0 and k >= 256


def skinny_supported(m: int, n: int, k: int) -> bool:
    return GEMV_MAX_ROWS < m <= SKINNY_MAX_ROWS and n % 16 == 0 and k % 8 == 0 and k >= 64


def small_batch_supported(m: int, n: int, k: int) -> bool:
    """True if the products of a few rows (and their fused epilogues) take these sizes: the register-streaming
    kernel up to GEMV_MAX_ROWS rows, the tcgen05 one up to SKINNY_MAX_ROWS."""
    return gemv_supported(m, n, k) or skinny_supported(m, n, k)


def _skinny_pad(m: int) -> int:
    return 16 if m <= 16 else (32 if m <= 32 else (64 if m <= 64 else 128))


def _skinny_splits(n: int, k: int) -> int:
    """K splits (= cluster size) of the tcgen05 product: enough CTAs to fill the GPU when the weight has few
    128-row tiles, but no more clusters than are resident at once (256 CTAs in clusters of 8 on 148 SMs), at least
    6 blocks of 64 along K per CTA, and a power of two (other cluster sizes place badly)."""
    tiles, k_blocks = -(-n // 128), -(-k // 64)
    s = 1
    while s < 8 and tiles * s * 2 <= 256 and k_blocks // (s * 2) >= 6:
        s *= 2
    return s


@dataclass
class RowScale:
    """The deferred 1/rms of rows that were written as ``residual * norm_weight``: per 16-column tile of the
    producer, the partial sums of squares of each row ([tiles, 16] fp32).  A consuming matrix product multiplies
    row m of its result by ``1 / sqrt(sum_j ss[j, m] / dim + eps)``."""

    ss: torch.Tensor
    dim: int
    eps: float


def _gemv_layout(n: int, k: int):
    # 8 warps per CTA as row tiles x K splits: as many row tiles per CTA (8, 4, 2, 1) as still leave one and a half
    # CTAs per SM (measured: 1,728 tiles of 5,120 at 8 rows: 4 tiles per CTA 45.9 us, 2: 47.5, 8: 50.8, 1: 51.7;
    # 2,368 tiles of 3,584: 8: 44.6, 2: 49.4; 608 of 896: 2: 6.4, 1: 8.3; 320 tiles and fewer: 1).  The same rule as
    # the library's executor (csrc/exec/core.cu): the order of a sum depends on the split.
    tiles = n // 16
    rt = 8
    while rt > 1 and -(-tiles // rt) < 222:
        rt //= 2
    ks = 8 // rt
    while ks > k // 32:
        ks //= 2
        rt *= 2
    return rt, ks


def _scale_args(scale: Optional["RowScale"], m: int):
    """(pointer, tiles, dim, eps) for the register-streaming kernel: partial sums [tiles, 16]."""
    if scale is None:
        return None, 0, 0, 0.0
    _need(scale.ss, "row scale", torch.float32)
    if scale.ss.dim() != 2 or scale.ss.shape[1] != 16 or m > 16:
        raise KernelError("row scale: expected [tiles, 16] partial sums")
    return scale.ss.data_ptr(), scale.ss.shape[0], int(scale.dim), float(scale.eps)


def _skinny_scale_args(scale: Optional["RowScale"], m: int):
    """(pointer, tiles, dim, row stride, eps) for the tcgen05 product: partial sums [tiles, stride >= m]."""
    if scale is None:
        return None, 0, 0, 0, 0.0
    _need(scale.ss, "row scale", torch.float32)
    if scale.ss.dim() != 2 or scale.ss.shape[1] < m:
        raise KernelError("row scale: expected [tiles, >= rows] partial sums")
    return scale.ss.data_ptr(), scale.ss.shape[0], int(scale.dim), scale.ss.shape[1], float(scale.eps)


def gemv_bf16(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], out_dtype: torch.dtype,
              swiglu: bool = False, scale: Optional[RowScale] = None) -> torch.Tensor:
    """x[M<=16, K] @ w[N, K]^T (+ bias) with the weight-streaming kernel.  ``swiglu``: w interleaves gate and
    up rows in blocks of 8 and the result is silu(gate) * up, [M, N/2].  ``scale``: rows of the product are
    multiplied by the deferred 1/rms before bias and activation."""
    _need(x, "gemv x", torch.bfloat16)
    _need(w, "gemv w", torch.bfloat16)
    m, k = x.shape
    n = w.shape[0]
    if w.shape != (n, k) or not small_batch_supported(m, n, k):
        raise KernelError(f"gemv: shapes x{tuple(x.shape)} w{tuple(w.shape)} are not supported")
    if bias is not None:
        _need(bias, "gemv bias")
    out = torch.empty((m, n // 2 if swiglu else n), dtype=out_dtype, device=x.device)
    if m > GEMV_MAX_ROWS:
        if out.shape[1] % 8:
            raise KernelError("gemv: the tcgen05 product needs output rows of a multiple of 8 columns")
        check(_lib.load().mm_gemm_skinny(w.data_ptr(), x.data_ptr(), _ptr(bias), dtype_code(bias.dtype) if bias is not None else F32,
                                         out.data_ptr(), dtype_code(out_dtype), m, n, k, k, out.shape[1], _skinny_splits(n, k),
                                         int(swiglu), *_skinny_scale_args(scale, m), tcgen05_error_flag(x.device).data_ptr(),
                                         _stream()), "gemm_skinny")
        return out
    rt, ks = _gemv_layout(n, k)
    check(_lib.load().mm_gemv_bf16(w.data_ptr(), x.data_ptr(), _ptr(bias), dtype_code(bias.dtype) if bias is not None else F32,
                                   out.data_ptr(), dtype_code(out_dtype), m, n, k, k, out.shape[1], rt, ks, int(swiglu),
                                   *_scale_args(scale, m), _stream()), "gemv_bf16")
    return out


def gemv_bf16_residual(x: torch.Tensor, w: torch.Tensor, residual: torch.Tensor, norm_weight: Optional[torch.Tensor],
                       eps: float = 0.0, scale: Optional[RowScale] = None):
    """residual[M, N] (fp32, in place) += x @ w^T.  With ``norm_weight`` returns (xw, RowScale): the rows of
    ``residual * norm_weight`` in bfloat16 and the partial sums for their 1/rms; else returns None."""
    _need(x, "gemv x", torch.bfloat16)
    _need(w, "gemv w", torch.bfloat16)
    _need(residual, "gemv residual", torch.float32)
    m, k = x.shape
    n = w.shape[0]
    if w.shape != (n, k) or residual.shape != (m, n) or not small_batch_supported(m, n, k):
        raise KernelError(f"gemv residual: shapes x{tuple(x.shape)} w{tuple(w.shape)} residual{tuple(residual.shape)} are not supported")
    skinny = m > GEMV_MAX_ROWS
    xw = ss = None
    if norm_weight is not None:
        _need(norm_weight, "norm weight")
        if norm_weight.shape != (n,):
            raise KernelError("gemv residual: norm weight has the wrong length")
        xw = torch.empty((m, n), dtype=torch.bfloat16, device=x.device)
        ss = torch.empty((n // 16, _skinny_pad(m) if skinny else 16), dtype=torch.float32, device=x.device)
    if skinny:
        check(_lib.load().mm_gemm_skinny_residual(
            w.data_ptr(), x.data_ptr(), residual.data_ptr(), _ptr(norm_weight),
            dtype_code(norm_weight.dtype) if norm_weight is not None else F32, _ptr(xw), _ptr(ss), ss.shape[1] if ss is not None else 0,
            m, n, k, k, _skinny_splits(n, k), *_skinny_scale_args(scale, m), tcgen05_error_flag(x.device).data_ptr(), _stream()),
            "gemm_skinny_residual")
        return None if norm_weight is None else (xw, RowScale(ss, n, float(eps)))
    rt, ks = _gemv_layout(n, k)
    check(_lib.load().mm_gemv_bf16_residual(w.data_ptr(), x.data_ptr(), residual.data_ptr(), _ptr(norm_weight),
                                            dtype_code(norm_weight.dtype) if norm_weight is not None else F32, _ptr(xw), _ptr(ss),
                                            m, n, k, k, rt, ks, *_scale_args(scale, m), _stream()), "gemv_bf16_residual")
    return None if norm_weight is None else (xw, RowScale(ss, n, float(eps)))


def interleave_halves(t: torch.Tensor, num_rot_heads: int, head_dim: int) -> torch.Tensor:
    """Row order the fused q/k/v product wants: within each of the first ``num_rot_heads`` heads (q and k), rows
    16b..16b+7 are elements 8b.. of the head's first half and rows 16b+8..16b+15 the same elements of the second
    half, so the thread that holds an element holds its rotation partner.  Other rows (v) keep their place."""
    hd, half = head_dim, head_dim // 2
    if hd % 16:
        raise KernelError("interleave_halves: the head size must be a multiple of 16")
    rot = num_rot_heads * hd
    head = t[:rot].reshape(num_rot_heads, 2, half // 8, 8, *t.shape[1:])     # [head, half, block, 8, ...]
    head = head.transpose(1, 2).reshape(rot, *t.shape[1:])                   # [head, block, half, 8, ...]
    return torch.cat([head, t[rot:]], dim=0).contiguous()


def rope_table(positions: torch.Tensor, dim: int, theta: float) -> torch.Tensor:
    """[n, dim] fp32: cos of the dim/2 rotation angles of every token's position, then their sin."""
    _need(positions, "positions", torch.int32)
    out = torch.empty((positions.numel(), dim), dtype=torch.float32, device=positions.device)
    check(_lib.load().mm_rope_table(positions.data_ptr(), out.data_ptr(), positions.numel(), dim, float(theta), _stream()), "rope_table")
    return out


def slot_mapping(positions: torch.Tensor, token_req: torch.Tensor, block_table: torch.Tensor, page_size: int) -> torch.Tensor:
    """[n] int32: where each token's key and value go in a page pool (page * page_size + place in the page), -1: nowhere."""
    _need(positions, "positions", torch.int32)
    _need(token_req, "token_req", torch.int32)
    _need(block_table, "block_table", torch.int32)
    if block_table.dim() != 2:
        raise KernelError("block_table: expected [requests, width]")
    out = torch.empty(positions.numel(), dtype=torch.int32, device=positions.device)
    check(_lib.load().mm_slot_mapping(positions.data_ptr(), token_req.data_ptr(), block_table.data_ptr(), block_table.shape[1],
                                      page_size, positions.numel(), out.data_ptr(), _stream()), "slot_mapping")
    return out


def gemv_bf16_qkv_rope(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], q_out: torch.Tensor,
                       k_pages: Optional[torch.Tensor], v_pages: Optional[torch.Tensor], table: torch.Tensor,
                       slots: Optional[torch.Tensor], page_size: int, num_heads: int, num_kv_heads: int, head_dim: int,
                       scale: Optional[RowScale] = None) -> None:
    """The q/k/v projection of up to 16 tokens with bias, rotary encoding and cache write in its epilogue.
    ``w`` and ``bias`` are in the order of :func:`interleave_halves`; q_out, k and v are in natural order.
    ``table``: :func:`rope_table` of the tokens for this head size; ``slots``: :func:`slot_mapping`."""
    _need(x, "gemv x", torch.bfloat16)
    _need(w, "gemv w", torch.bfloat16)
    m, k = x.shape
    n = (num_heads + 2 * num_kv_heads) * head_dim
    if w.shape != (n, k) or not small_batch_supported(m, n, k) or head_dim % 16:
        raise KernelError(f"gemv qkv: shapes x{tuple(x.shape)} w{tuple(w.shape)} are not supported")
    _need(q_out, "q_out", torch.bfloat16)
    if q_out.shape != (m, num_heads * head_dim):
        raise KernelError("q_out: wrong shape")
    if bias is not None:
        _need(bias, "qkv bias")
        if bias.shape != (n,):
            raise KernelError("qkv bias: wrong shape")
    _need(table, "rope table", torch.float32)
    if table.shape != (m, head_dim):
        raise KernelError("rope table: expected [tokens, head_dim]")
    if k_pages is not None:
        for name, pool in (("k_pages", k_pages), ("v_pages", v_pages)):
            _need(pool, name, torch.bfloat16)
            if pool.dim() != 4 or pool.shape[1:] != (num_kv_heads, page_size, head_dim):
                raise KernelError(f"{name}: shape {tuple(pool.shape)} is not [pages, {num_kv_heads}, {page_size}, {head_dim}]")
        _need(slots, "slots", torch.int32)
        if slots.numel() != m:
            raise KernelError("slots: one per token")
    if m > GEMV_MAX_ROWS:
        check(_lib.load().mm_gemm_skinny_qkv_rope(
            w.data_ptr(), x.data_ptr(), _ptr(bias), dtype_code(bias.dtype) if bias is not None else F32, q_out.data_ptr(),
            _ptr(k_pages), _ptr(v_pages), table.data_ptr(), _ptr(slots) if k_pages is not None else None, page_size,
            num_heads, num_kv_heads, head_dim, m, k, k, _skinny_splits(n, k), *_skinny_scale_args(scale, m),
            tcgen05_error_flag(x.device).data_ptr(), _stream()), "gemm_skinny_qkv_rope")
        return
    rt, ks = _gemv_layout(n, k)
    check(_lib.load().mm_gemv_bf16_qkv_rope(
        w.data_ptr(), x.data_ptr(), _ptr(bias), dtype_code(bias.dtype) if bias is not None else F32, q_out.data_ptr(),
        _ptr(k_pages), _ptr(v_pages), table.data_ptr(), _ptr(slots) if k_pages is not None else None, page_size,
        num_heads, num_kv_heads, head_dim, m, k, k, rt, ks, *_scale_args(scale, m), _stream()), "gemv_bf16_qkv_rope")


_TC_ERR = {}
EPI_BF16, EPI_SWIGLU, EPI_F32 = 0, 1, 2
# Measured on B200 (7B shapes, gate/up product): from 256 rows on the fused product is level with or ahead of the
# library product + activation kernel (65 against 80 us at 256 rows, 197 against 217 at 1,024, 346 against 409 at 2,048);
# below, a 128-row tile leaves the tensor cores short of work and the library's smaller tiles win (58 against 71 us at 96).
TCGEN05_SWIGLU_MIN_ROWS = 256


def tcgen05_error_flag(device) -> torch.Tensor:
    """Device int that the tcgen05 kernels set to 1 when one of their bounded waits ran out."""
    key = str(device)
    if key not in _TC_ERR:
        _TC_ERR[key] = torch.zeros(1, dtype=torch.int32, device=device)
    return _TC_ERR[key]


def check_tcgen05_errors(device) -> None:
    """Raises if a tcgen05 kernel gave up a wait since the last check (synchronises)."""
    flag = _TC_ERR.get(str(device))
    if flag is not None and int(flag.item()) != 0:
        flag.zero_()
        raise KernelError("a tcgen05 kernel gave up waiting on its pipeline; its output is not valid")


def gemm_tcgen05_supported(m: int, n: int, k: int) -> bool:
    return m >= 1 and k % 8 == 0 and n % 8 == 0 and k >= 64


# From this many rows on, the product runs on pairs of CTAs (cta_group::2, 256 x 256 tiles), unless the last pair's
# second CTA would have nothing but padding (384 rows cost as much as 512 there: 126 against 91 us).
TCGEN05_PAIR_MIN_ROWS = 256


def tcgen05_pair_suits(m: int) -> bool:
    return m >= TCGEN05_PAIR_MIN_ROWS and (m - 1) % 256 >= 128


def gemm_tcgen05(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], out_dtype: torch.dtype,
                 swiglu: bool = False, pair: Optional[bool] = None) -> torch.Tensor:
    """x[M, K] @ w[N, K]^T (+ bias) on the tcgen05 tensor cores (TMA operands, TMEM accumulators).
    ``swiglu``: w interleaves gate and up rows in blocks of 8; returns silu(gate) * up, [M, N/2].
    ``pair``: the kernel of CTA pairs or the single-CTA one; None chooses by the number of rows."""
    _need(x, "gemm x", torch.bfloat16)
    _need(w, "gemm w", torch.bfloat16)
    m, k = x.shape
    n = w.shape[0]
    if w.shape != (n, k) or not gemm_tcgen05_supported(m, n, k):
        raise KernelError(f"gemm_tcgen05: shapes x{tuple(x.shape)} w{tuple(w.shape)} are not supported")
    if swiglu:
        if n % 16 or bias is not None or out_dtype != torch.bfloat16:
            raise KernelError("gemm_tcgen05: the SwiGLU epilogue needs N a multiple of 16, no bias, bf16 output")
        out = torch.empty((m, n // 2), dtype=torch.bfloat16, device=x.device)
        epi = EPI_SWIGLU
    else:
        out = torch.empty((m, n), dtype=out_dtype, device=x.device)
        epi = EPI_F32 if out_dtype == torch.float32 else EPI_BF16
    if bias is not None:
        _need(bias, "gemm bias")
    if pair is None:
        pair = tcgen05_pair_suits(m)
    fn = _lib.load().mm_gemm_tcgen05_pair if pair else _lib.load().mm_gemm_tcgen05
    check(fn(x.data_ptr(), w.data_ptr(), _ptr(bias), dtype_code(bias.dtype) if bias is not None else F32,
             out.data_ptr(), epi, m, n, k, k, out.shape[1], tcgen05_error_flag(x.device).data_ptr(), _stream()), "gemm_tcgen05")
    return out


def gemm_tcgen05_act(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], activation: str,
                     pair: Optional[bool] = None) -> torch.Tensor:
    """act(x[M, K] @ w[N, K]^T + bias) as bfloat16 in one launch of the tcgen05 product (the activation on the fp32
    accumulators, in its epilogue); ``activation`` as for :func:`bias_act`."""
    _need(x, "gemm x", torch.bfloat16)
    _need(w, "gemm w", torch.bfloat16)
    m, k = x.shape
    n = w.shape[0]
    if w.shape != (n, k) or not gemm_tcgen05_supported(m, n, k):
        raise KernelError(f"gemm_tcgen05: shapes x{tuple(x.shape)} w{tuple(w.shape)} are not supported")
    if activation not in ACTIVATIONS:
        raise KernelError(f"activation '{activation}' is not one of {', '.join(sorted(ACTIVATIONS))}")
    if bias is not None:
        _need(bias, "gemm bias")
        if bias.shape != (n,):
            raise KernelError("gemm_tcgen05: bias shape mismatch")
    out = torch.empty((m, n), dtype=torch.bfloat16, device=x.device)
    if pair is None:
        pair = tcgen05_pair_suits(m)
    check(_lib.load().mm_gemm_tcgen05_act(x.data_ptr(), w.data_ptr(), _ptr(bias), dtype_code(bias.dtype) if bias is not None else F32,
                                          out.data_ptr(), ACTIVATIONS[activation] + 1, int(pair), m, n, k, k, n,
                                          tcgen05_error_flag(x.device).data_ptr(), _stream()), "gemm_tcgen05_act")
    return out


def argmax_rows(logits: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    _need(logits, "argmax logits", torch.float32)
    r, v = logits.shape
    if out is None:
        out = torch.empty(r, dtype=torch.int32, device=logits.device)
    _need(out, "argmax out", torch.int32)
    if v > 16384:
        # wide rows: several blocks per row, then one to reduce them
        p = min(256, -(-v // 4096))
        part_val = torch.empty((r, p), dtype=torch.float32, device=logits.device)
        part_idx = torch.empty((r, p), dtype=torch.int32, device=logits.device)
        check(_lib.load().mm_argmax_rows_split(logits.data_ptr(), out.data_ptr(), part_val.data_ptr(), part_idx.data_ptr(),
                                               r, v, p, _stream()), "argmax_rows_split")
        return out
    check(_lib.load().mm_argmax_rows(logits.data_ptr(), out.data_ptr(), r, v, _stream()), "argmax_rows")
    return out


def sample_rows(logits: torch.Tensor, temperature: torch.Tensor, top_k: torch.Tensor, top_p: torch.Tensor,
                seeds: torch.Tensor, counters: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    _need(logits, "sample logits", torch.float32)
    r, v = logits.shape
    _need(temperature, "temperature", torch.float32)
    _need(top_k, "top_k", torch.int32)
    _need(top_p, "top_p", torch.float32)
    _need(seeds, "seeds", torch.int64)
    _need(counters, "counters", torch.int64)
    for t in (temperature, top_k, top_p, seeds, counters):
        if t.numel() != r:
            raise KernelError("sample: per-row parameter length mismatch")
    if out is None:
        out = torch.empty(r, dtype=torch.int32, device=logits.device)
    check(_lib.load().mm_sample_rows(logits.data_ptr(), out.data_ptr(), r, v, temperature.data_ptr(), top_k.data_ptr(),
                                     top_p.data_ptr(), seeds.data_ptr(), counters.data_ptr(), _stream()), "sample_rows")
    return out


def apply_penalties(logits: torch.Tensor, recent: Optional[torch.Tensor], repetition: torch.Tensor,
                    frequency: torch.Tensor, presence: torch.Tensor, softcap: Optional[torch.Tensor]) -> torch.Tensor:
    _need(logits, "penalties logits", torch.float32)
    r, v = logits.shape
    w = 0
    if recent is not None:
        _need(recent, "recent tokens", torch.int32)
        w = recent.shape[1]
    for t in (repetition, frequency, presence):
        _need(t, "penalty parameter", torch.float32)
    if softcap is not None:
        _need(softcap, "softcap", torch.float32)
    check(_lib.load().mm_apply_penalties(logits.data_ptr(), r, v, _ptr(recent), w, repetition.data_ptr(),
                                         frequency.data_ptr(), presence.data_ptr(), _ptr(softcap), _stream()),
          "apply_penalties")
    return logits


def window_push(recent: torch.Tensor, widths: torch.Tensor, lengths: torch.Tensor, tokens: torch.Tensor) -> None:
    """recent int32 [R, W]: per row a ring of its last widths[r] tokens; writes tokens[r] at lengths[r] % widths[r]
    and adds one to lengths[r] (int64)."""
    _need(recent, "recent tokens", torch.int32)
    _need(widths, "window widths", torch.int32)
    _need(lengths, "sequence lengths", torch.int64)
    _need(tokens, "tokens", torch.int32)
    r, w = recent.shape
    if widths.numel() != r or lengths.numel() != r or tokens.numel() != r:
        raise KernelError("window_push: one width, length and token per row")
    check(_lib.load().mm_window_push(recent.data_ptr(), r, w, widths.data_ptr(), lengths.data_ptr(), tokens.data_ptr(), _stream()),
          "window_push")


def uniform_from(seed: int, counter: int) -> float:
    """The uniform number in [0,1) the device sampler draws for (seed, counter)."""
    return float(_lib.load().mm_uniform_from(seed & 0xFFFFFFFFFFFFFFFF, counter & 0xFFFFFFFFFFFFFFFF))


# ---- grouped norm, bigram embedding, sink attention, minGRU, bias + activation ------------------------------------------
def group_norm_chain(residual: torch.Tensor, branch: Optional[torch.Tensor], w_post: Optional[torch.Tensor],
                     w_next: Optional[torch.Tensor], groups: int, eps: float, out: Optional[torch.Tensor] = None,
                     rows: Optional[torch.Tensor] = None) -> Optional[torch.Tensor]:
    """RMS norm in ``groups`` equal parts of a row, chained around the residual stream (fp32, in place):
    ``residual += gnorm(branch) * w_post`` (plain add without ``w_post``), then ``out = gnorm(residual) * w_next``.
    Either half may be absent.  With ``rows`` output row i comes from source row rows[i] and nothing is added."""
    _need(residual, "group norm residual", torch.float32)
    d = residual.shape[-1]
    weight = w_post if w_post is not None else w_next
    if weight is None and branch is None:
        raise KernelError("group norm: nothing to do")
    for w in (w_post, w_next):
        if w is not None:
            _need(w, "group norm weight")
            if w.shape != (d,) or w.dtype != weight.dtype:
                raise KernelError("group norm: weight shape or dtype mismatch")
    if branch is not None:
        _need(branch, "group norm branch")
        if branch.shape != residual.shape:
            raise KernelError("group norm: branch and residual differ in shape")
    if w_next is not None:
        _need(out, "group norm out")
        if out.shape[-1] != d or (branch is not None and out.dtype != branch.dtype):
            raise KernelError("group norm: out width or dtype mismatch")
    if rows is not None:
        _need(rows, "group norm rows", torch.int32)
        if out is None or rows.numel() != out.shape[0]:
            raise KernelError("group norm: rows and out differ in length")
    n_out = out.shape[0] if out is not None else residual.shape[0]
    if rows is None and n_out != residual.shape[0]:
        raise KernelError("group norm: out and residual differ in rows")
    act = out.dtype if out is not None else branch.dtype
    check(_lib.load().mm_group_norm_chain(residual.data_ptr(), _ptr(branch), _ptr(w_post), _ptr(w_next),
                                          dtype_code(weight.dtype) if weight is not None else dtype_code(act), _ptr(rows), _ptr(out),
                                          dtype_code(act), n_out, d, int(groups), float(eps), _stream()), "group_norm_chain")
    return out


def group_norm_rows(x: torch.Tensor, weight: torch.Tensor, groups: int, eps: float, out: torch.Tensor) -> torch.Tensor:
    """out = gnorm(x) * weight for rows in the activation dtype."""
    _need(x, "group norm x")
    _need(weight, "group norm weight")
    _need(out, "group norm out", x.dtype)
    n, d = x.shape
    if weight.shape != (d,) or out.shape != x.shape:
        raise KernelError("group norm: shape mismatch")
    check(_lib.load().mm_group_norm_rows(x.data_ptr(), weight.data_ptr(), dtype_code(weight.dtype), out.data_ptr(), dtype_code(x.dtype),
                                         n, d, int(groups), float(eps), _stream()), "group_norm_rows")
    return out


def embedding_bigram(ids: torch.Tensor, positions: torch.Tensor, token_req: torch.Tensor, req_meta: Optional[torch.Tensor],
                     slots: torch.Tensor, state: torch.Tensor, table: torch.Tensor, pairs: torch.Tensor, out: torch.Tensor,
                     buckets: int, mul_prev: int, mul_cur: int) -> torch.Tensor:
    """out[t] = table[id_t] + pairs[(prev_t * mul_prev + id_t * mul_cur) mod buckets] (row ``buckets`` at position 0) as fp32.
    ``state`` [slots] int32 carries every request's last token from step to step; ``req_meta`` [requests, 4] gives each
    request's first token and token count in this step (None: one token per request)."""
    _need(ids, "embedding ids", torch.int32)
    _need(positions, "positions", torch.int32)
    _need(token_req, "token_req", torch.int32)
    _need(slots, "state slots", torch.int32)
    _need(state, "bigram state", torch.int32)
    _need(table, "embedding table")
    _need(pairs, "bigram table", table.dtype)
    _need(out, "embedding out", torch.float32)
    n, (v, d) = ids.numel(), table.shape
    if pairs.shape != (buckets + 1, d) or out.shape != (n, d):
        raise KernelError("bigram embedding: the pair table must be [buckets + 1, width] and out [tokens, width]")
    if req_meta is not None:
        _need(req_meta, "req_meta", torch.int32)
    check(_lib.load().mm_embedding_bigram(ids.data_ptr(), positions.data_ptr(), token_req.data_ptr(), _ptr(req_meta), slots.data_ptr(),
                                          state.data_ptr(), table.data_ptr(), pairs.data_ptr(), dtype_code(table.dtype), out.data_ptr(),
                                          n, v, d, int(buckets), int(mul_prev), int(mul_cur), _stream()), "embedding_bigram")
    return out


def rope_pairs_table(positions: torch.Tensor, inv_freq: torch.Tensor, rot_dims: int) -> torch.Tensor:
    """[n, rot_dims / 2, 2] fp32: (cos, sin) of position * inv_freq[i] for every token and pair of rotated dimensions."""
    _need(positions, "positions", torch.int32)
    _need(inv_freq, "inv_freq", torch.float32)
    half = rot_dims // 2
    if half < 1 or inv_freq.numel() < half:
        raise KernelError("rope pairs table: bad sizes")
    n = positions.numel()
    out = torch.empty((n, half, 2), dtype=torch.float32, device=positions.device)
    check(_lib.load().mm_rope_pairs_table(positions.data_ptr(), inv_freq.data_ptr(), out.data_ptr(), n, half, _stream()), "rope_pairs_table")
    return out


def qkv_pairs_post(qkv: torch.Tensor, q_out: torch.Tensor, k_pages: Optional[torch.Tensor], v_pages: Optional[torch.Tensor],
                   v_first: Optional[torch.Tensor], rot: Optional[torch.Tensor], slots: Optional[torch.Tensor], page_size: int,
                   num_heads: int, num_kv_heads: int, key_dim: int, value_dim: int, rot_dims: int, mix_mode: int, mix: float) -> None:
    """Rotates adjacent pairs of q and k by the angles of ``rot`` (:func:`rope_pairs_table`), mixes the values
    (mode 1: copy them to ``v_first``; 2: v = (1 - mix) v + mix v_first), writes q to ``q_out`` and k and the mixed v
    into their pages ([pages, kv heads, page, key_dim] and [.., value_dim]) at ``slots`` (:func:`slot_mapping`)."""
    _need(qkv, "qkv")
    n = qkv.shape[0]
    H, G, dk, dv = num_heads, num_kv_heads, key_dim, value_dim
    if qkv.shape != (n, (H + G) * dk + G * dv):
        raise KernelError(f"qkv: shape {tuple(qkv.shape)} is not [n, {(H + G) * dk + G * dv}]")
    _need(q_out, "q_out", qkv.dtype)
    if q_out.shape != (n, H * dk):
        raise KernelError("q_out: wrong shape")
    if k_pages is not None:
        _need(k_pages, "k_pages", qkv.dtype)
        _need(v_pages, "v_pages", qkv.dtype)
        if k_pages.shape[1:] != (G, page_size, dk) or v_pages.shape[1:] != (G, page_size, dv) or k_pages.shape[0] != v_pages.shape[0]:
            raise KernelError("qkv post: page pool shape mismatch")
        _need(slots, "slots", torch.int32)
        if slots.shape != (n,):
            raise KernelError("slots: wrong shape")
    if mix_mode:
        _need(v_first, "v_first", qkv.dtype)
        if v_first.shape != (n, G * dv):
            raise KernelError("v_first: wrong shape")
    if rot_dims:
        _need(rot, "rotation table", torch.float32)
        if rot.shape != (n, rot_dims // 2, 2):
            raise KernelError("rotation table: wrong shape")
    check(_lib.load().mm_qkv_pairs_post(qkv.data_ptr(), q_out.data_ptr(), _ptr(k_pages), _ptr(v_pages), _ptr(v_first) if mix_mode else None,
                                        dtype_code(qkv.dtype), _ptr(rot) if rot_dims else None, _ptr(slots) if k_pages is not None else None,
                                        page_size, n, H, G, dk, dv, int(rot_dims), int(mix_mode), float(mix), _stream()), "qkv_pairs_post")


def attention_sink_generic(q: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor, out: torch.Tensor, positions: torch.Tensor,
                           token_req: torch.Tensor, block_table: torch.Tensor, page_size: int, num_heads: int, num_kv_heads: int,
                           key_dim: int, value_dim: int, window: int, scale: float, sink: bool,
                           sink_logit: Optional[torch.Tensor] = None, dist_bias: Optional[torch.Tensor] = None, softcap: float = 0.0,
                           value_heads: Optional[int] = None, value_row: Optional[int] = None) -> torch.Tensor:
    """Windowed causal attention of every token over its request's pages with keys of ``key_dim`` and values of
    ``value_dim``; with ``sink`` the softmax denominator has one added, with ``sink_logit`` (fp32 [heads]) the head's
    ``exp(logit)``; ``dist_bias`` (fp32 [heads, distances]) is added to the scaled score by distance, a head's last entry
    standing for every larger distance (fp32 arithmetic, any sizes).  ``softcap`` > 0: the scaled score becomes
    ``cap * tanh(score / cap)``.  ``value_heads``: heads of the value pool (key head g reads value head g mod value_heads);
    ``value_row``: numbers between the values of consecutive tokens (default ``value_dim``; larger when the values are the
    leading part of a wider per-token array, which may be the key pool itself).  ``out`` has q's type or is fp32."""
    value_heads = num_kv_heads if value_heads is None else int(value_heads)
    value_row = value_dim if value_row is None else int(value_row)
    _need(q, "attention q")
    n = q.shape[0]
    _need(out, "attention out", torch.float32 if out.dtype == torch.float32 else q.dtype)
    _need(k_pages, "attention k_pages", q.dtype)
    _need(v_pages, "attention v_pages", q.dtype)
    if q.shape != (n, num_heads * key_dim) or out.shape != (n, num_heads * value_dim):
        raise KernelError("attention: q/out shape mismatch")
    if k_pages.shape[1:] != (num_kv_heads, page_size, key_dim) or v_pages.shape[1:] != (value_heads, page_size, value_row):
        raise KernelError("attention: page pool shape mismatch")
    _need(positions, "positions", torch.int32)
    _need(token_req, "token_req", torch.int32)
    _need(block_table, "block_table", torch.int32)
    if sink_logit is not None:
        _need(sink_logit, "sink logits", torch.float32)
        if sink_logit.numel() != num_heads:
            raise KernelError("attention: one sink logit per head")
    if dist_bias is not None:
        _need(dist_bias, "distance bias", torch.float32)
        if dist_bias.dim() != 2 or dist_bias.shape[0] != num_heads or dist_bias.shape[1] < 1:
            raise KernelError("attention: the distance bias is [heads, distances]")
    check(_lib.load().mm_attention_sink_generic(
        q.data_ptr(), k_pages.data_ptr(), v_pages.data_ptr(), out.data_ptr(), dtype_code(q.dtype), positions.data_ptr(),
        token_req.data_ptr(), block_table.data_ptr(), block_table.shape[1], page_size, n, num_heads, num_kv_heads, key_dim,
        value_dim, int(window), float(scale), int(bool(sink)), _ptr(sink_logit), _ptr(dist_bias),
        dist_bias.shape[1] - 1 if dist_bias is not None else 0, float(softcap), value_heads, value_row,
        int(out.dtype == torch.float32 and q.dtype != torch.float32), _stream()), "attention_sink_generic")
    return out


def mingru_walk(a: torch.Tensor, y: torch.Tensor, state: torch.Tensor, req_meta: Optional[torch.Tensor], slots: torch.Tensor,
                positions: torch.Tensor, n_requests: int, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """minGRU over each request's tokens in order, one thread per (request, channel): ``a`` [n, 3W] fp32 holds the
    projections for the gate, the candidate and the output gate (``bias`` [2W] fp32: the gate's and the candidate's, added
    here); ``state`` [slots, W] fp32 is read and left updated; ``y`` [n, W] gets state * silu(output gate)."""
    _need(a, "mingru projections", torch.float32)
    _need(y, "mingru out")
    _need(state, "mingru state", torch.float32)
    _need(slots, "state slots", torch.int32)
    _need(positions, "positions", torch.int32)
    n, w3 = a.shape
    W = w3 // 3
    if w3 != 3 * W or y.shape != (n, W) or state.shape[-1] != W:
        raise KernelError("mingru: shape mismatch")
    if req_meta is not None:
        _need(req_meta, "req_meta", torch.int32)
    _check_mingru_bias(bias, W)
    check(_lib.load().mm_mingru_walk(a.data_ptr(), y.data_ptr(), dtype_code(y.dtype), state.data_ptr(), _ptr(req_meta), slots.data_ptr(),
                                     positions.data_ptr(), _ptr(bias), int(n_requests), W, _stream()), "mingru_walk")
    return y


def _check_mingru_bias(bias: Optional[torch.Tensor], W: int) -> None:
    if bias is not None:
        _need(bias, "mingru bias", torch.float32)
        if bias.numel() != 2 * W:
            raise KernelError("mingru: the bias holds the gate's and the candidate's, [2W]")


def mingru_chunked(a: torch.Tensor, y: torch.Tensor, state: torch.Tensor, chunk_meta: torch.Tensor, req_chunks: torch.Tensor,
                   slots: torch.Tensor, positions: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """minGRU as a scan over chunks of tokens (three launches: every chunk from a zero state, the carry along each
    request's chunks, every chunk again from its starting state).  ``chunk_meta`` [chunks, 4] = (first token, tokens,
    request, .), ``req_chunks`` [requests, 2] = (first chunk, chunks)."""
    _need(a, "mingru projections", torch.float32)
    _need(y, "mingru out")
    _need(state, "mingru state", torch.float32)
    _need(chunk_meta, "chunk_meta", torch.int32)
    _need(req_chunks, "req_chunks", torch.int32)
    _need(slots, "state slots", torch.int32)
    _need(positions, "positions", torch.int32)
    n, w3 = a.shape
    W = w3 // 3
    if w3 != 3 * W or y.shape != (n, W) or state.shape[-1] != W:
        raise KernelError("mingru: shape mismatch")
    _check_mingru_bias(bias, W)
    n_chunks, n_req = chunk_meta.shape[0], req_chunks.shape[0]
    scratch = torch.empty((2, max(1, n_chunks), W), dtype=torch.float32, device=a.device)
    check(_lib.load().mm_mingru_chunked(a.data_ptr(), y.data_ptr(), dtype_code(y.dtype), state.data_ptr(), scratch[0].data_ptr(),
                                        scratch[1].data_ptr(), chunk_meta.data_ptr(), req_chunks.data_ptr(), slots.data_ptr(),
                                        positions.data_ptr(), _ptr(bias), n_req, n_chunks, W, _stream()), "mingru_chunked")
    return y


ACTIVATIONS = {"relu2": 0, "gelu_tanh": 1, "silu": 2, "relu": 3}


def gemv_bf16_act(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], activation: str) -> torch.Tensor:
    """act(x[M<=8, K] @ w[N, K]^T + bias) in one launch of the weight-streaming kernel (the activation on the fp32 sums)."""
    _need(x, "gemv x", torch.bfloat16)
    _need(w, "gemv w", torch.bfloat16)
    m, k = x.shape
    n = w.shape[0]
    if w.shape != (n, k) or not gemv_supported(m, n, k):
        raise KernelError(f"gemv: shapes x{tuple(x.shape)} w{tuple(w.shape)} are not supported")
    if bias is not None:
        _need(bias, "gemv bias")
    out = torch.empty((m, n), dtype=torch.bfloat16, device=x.device)
    rt, ks = _gemv_layout(n, k)
    check(_lib.load().mm_gemv_bf16_act(w.data_ptr(), x.data_ptr(), _ptr(bias), dtype_code(bias.dtype) if bias is not None else F32,
                                       out.data_ptr(), BF16, m, n, k, k, n, rt, ks, ACTIVATIONS[activation] + 1, _stream()), "gemv_bf16_act")
    return out


def bias_act(x: torch.Tensor, bias: Optional[torch.Tensor], activation: str, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out = act(x + bias) in fp32 arithmetic; ``activation`` one of relu2 (squared relu), gelu_tanh, silu, relu."""
    _need(x, "bias_act x")
    if activation not in ACTIVATIONS:
        raise KernelError(f"activation '{activation}' is not one of {', '.join(sorted(ACTIVATIONS))}")
    out = torch.empty_like(x) if out is None else out
    _need(out, "bias_act out", x.dtype)
    n, f = x.shape
    if bias is not None:
        _need(bias, "bias_act bias")
        if bias.shape != (f,):
            raise KernelError("bias_act: bias shape mismatch")
    check(_lib.load().mm_bias_act(x.data_ptr(), _ptr(bias), dtype_code(bias.dtype) if bias is not None else F32, out.data_ptr(),
                                  dtype_code(x.dtype), n, f, ACTIVATIONS[activation], _stream()), "bias_act")
    return out


# ---- mixers with a matrix state per head (csrc/linear_state.cu) -------------------------------------------------------
def causal_conv_walk(x: torch.Tensor, channels: int, taps: torch.Tensor, tail: torch.Tensor, req_meta: Optional[torch.Tensor],
                     slots: torch.Tensor, positions: torch.Tensor, n_requests: int, silu: bool = True) -> torch.Tensor:
    """Short causal convolution over time on the first ``channels`` columns of ``x`` [n, ld] fp32, in place, followed by
    silu.  ``taps`` [channels, K] fp32 (last column: the current token); ``tail`` [slots, stride] fp32 holds each request's
    last K-1 inputs at ``[j * channels + c]`` (j = 0 the most recent) and is left updated."""
    _need(x, "conv rows", torch.float32)
    _need(taps, "conv taps", torch.float32)
    _need(slots, "state slots", torch.int32)
    _need(positions, "positions", torch.int32)
    if tail.dtype != torch.float32 or not tail.is_cuda or tail.stride(-1) != 1:
        raise KernelError("conv: the state is fp32 with unit stride in its last axis")
    K = taps.shape[1]
    if taps.shape[0] != channels or x.shape[1] < channels or tail.shape[1] < (K - 1) * channels:
        raise KernelError("conv: shape mismatch")
    check(_lib.load().mm_causal_conv_walk(x.data_ptr(), x.shape[1], channels, taps.data_ptr(), K, tail.data_ptr(), tail.stride(0),
                                          _ptr(req_meta), slots.data_ptr(), positions.data_ptr(), int(n_requests), int(bool(silu)),
                                          _stream()), "causal_conv_walk")
    return x


def causal_conv_tokens(x: torch.Tensor, channels: int, taps: torch.Tensor, tail: torch.Tensor, token_req: torch.Tensor,
                       req_meta: Optional[torch.Tensor], slots: torch.Tensor, positions: torch.Tensor, n_requests: int, silu: bool = True) -> torch.Tensor:
    """The same convolution with one thread per (token, channel), for long portions: returns a new fp32 [n, channels], leaves
    ``x`` as it is, and then leaves every request's last K-1 inputs in ``tail``."""
    _need(x, "conv rows", torch.float32)
    _need(taps, "conv taps", torch.float32)
    _need(token_req, "token_req", torch.int32)
    _need(slots, "state slots", torch.int32)
    _need(positions, "positions", torch.int32)
    if tail.dtype != torch.float32 or not tail.is_cuda or tail.stride(-1) != 1:
        raise KernelError("conv: the state is fp32 with unit stride in its last axis")
    K = taps.shape[1]
    if taps.shape[0] != channels or x.shape[1] < channels or tail.shape[1] < (K - 1) * channels:
        raise KernelError("conv: shape mismatch")
    n = x.shape[0]
    y = torch.empty((n, channels), dtype=torch.float32, device=x.device)
    check(_lib.load().mm_causal_conv_tokens(x.data_ptr(), x.shape[1], channels, taps.data_ptr(), K, tail.data_ptr(), tail.stride(0), y.data_ptr(),
                                            channels, token_req.data_ptr(), _ptr(req_meta), slots.data_ptr(), positions.data_ptr(), n,
                                            int(n_requests), int(bool(silu)), _stream()), "causal_conv_tokens")
    return y


def angle_table(positions: torch.Tensor, freq: torch.Tensor) -> torch.Tensor:
    """(cos, sin) of ``position * freq[i]`` as fp32 [n, len(freq), 2]."""
    _need(positions, "positions", torch.int32)
    _need(freq, "frequencies", torch.float32)
    n, half = positions.numel(), freq.numel()
    out = torch.empty((n, half, 2), dtype=torch.float32, device=positions.device)
    check(_lib.load().mm_angle_table(positions.data_ptr(), freq.data_ptr(), out.data_ptr(), n, half, _stream()), "angle_table")
    return out


def linear_state_prep(x: torch.Tensor, q_off: int, k_off: int, v_off: int, qk_heads: int, dk: int, n_v: int, *, silu: bool = False,
                      rot: Optional[torch.Tensor] = None, rot_dims: int = 0, unit: bool = False, unit_eps: float = 0.0,
                      q_scale: float = 1.0, k_scale: float = 1.0, a_off: int = -1, b_off: int = -1, heads: int = 0,
                      A_log: Optional[torch.Tensor] = None, dt_bias: Optional[torch.Tensor] = None, gate_rows: Optional[torch.Tensor] = None):
    """What stands between the projection and the recurrence, in place on the fp32 rows ``x`` [n, ld]: silu on q, k and v;
    rotation of the half-split pairs of q and k by ``rot`` [n, rot_dims/2, 2]; unit length of every q and k head; the
    two scales.  Returns (gate, beta), each [n, heads] fp32 or None: with ``a_off`` >= 0 the decay per token
    ``exp(-exp(A_log) softplus(a + dt_bias))`` from the row's columns ``a_off..``, with ``b_off`` >= 0 the delta rule's write
    strength ``sigmoid(b)`` from the columns ``b_off..`` (of ``gate_rows`` when given: fp32 rows of their own width)."""
    _need(x, "projection rows", torch.float32)
    n, ld = x.shape
    if gate_rows is not None:
        _need(gate_rows, "gate rows", torch.float32)
        if gate_rows.shape[0] != n or max(a_off, b_off) + heads > gate_rows.shape[1]:
            raise KernelError("linear state prep: gate columns outside their row")
    gate = beta = None
    if a_off >= 0:
        _need(A_log, "A_log", torch.float32)
        _need(dt_bias, "dt_bias", torch.float32)
        gate = torch.empty((n, heads), dtype=torch.float32, device=x.device)
    if b_off >= 0:
        beta = torch.empty((n, heads), dtype=torch.float32, device=x.device)
    if rot_dims:
        _need(rot, "rotation table", torch.float32)
        if rot.shape != (n, rot_dims // 2, 2):
            raise KernelError("rotation table: wrong shape")
    if max(q_off, k_off) + qk_heads * dk > ld or v_off + n_v > ld:
        raise KernelError("linear state prep: columns outside the row")
    check(_lib.load().mm_linear_state_prep(x.data_ptr(), ld, n, q_off, k_off, v_off, qk_heads, dk, n_v, int(bool(silu)),
                                           _ptr(rot) if rot_dims else None, int(rot_dims), int(bool(unit)), float(unit_eps),
                                           float(q_scale), float(k_scale), _ptr(gate_rows), gate_rows.shape[1] if gate_rows is not None else 0,
                                           int(a_off), int(b_off), int(heads), _ptr(A_log), _ptr(dt_bias),
                                           _ptr(gate), _ptr(beta), _stream()), "linear_state_prep")
    return gate, beta


def linear_state_walk(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, state: torch.Tensor, req_meta: Optional[torch.Tensor],
                      slots: torch.Tensor, positions: torch.Tensor, n_requests: int, heads: int, qk_heads: int, dk: int, dv: int,
                      gate: Optional[torch.Tensor] = None, beta: Optional[torch.Tensor] = None,
                      head_decay: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Per head ``S <- g S; u = v`` (or ``beta (v - S^T k)`` when ``beta`` is given); ``S <- S + k u^T; o = S^T q`` over each
    request's tokens in order.  q, k: fp32 column slices [n, qk_heads * dk], v [n, heads * dv] (any row stride);
    ``gate`` [n, heads] or ``head_decay`` [heads]; ``state`` [slots, stride] fp32 holds S as [heads, dv, dk] at its start
    and is left updated.  Returns o fp32 [n, heads * dv]."""
    for t, what in ((q, "q"), (k, "k"), (v, "v")):
        if t.dtype != torch.float32 or not t.is_cuda or t.stride(1) != 1:
            raise KernelError(f"linear state {what}: fp32 rows with unit column stride are needed")
    n = q.shape[0]
    if q.shape[1] != qk_heads * dk or k.shape != q.shape or v.shape != (n, heads * dv):
        raise KernelError("linear state: shape mismatch")
    if state.dtype != torch.float32 or state.stride(-1) != 1 or state.shape[1] < heads * dv * dk:
        raise KernelError("linear state: the state is fp32 [slots, >= heads * dv * dk]")
    for t, what in ((gate, "gate"), (beta, "beta")):
        if t is not None:
            _need(t, what, torch.float32)
            if t.shape != (n, heads):
                raise KernelError(f"linear state {what}: wrong shape")
    if head_decay is not None:
        _need(head_decay, "head decay", torch.float32)
    _need(slots, "state slots", torch.int32)
    _need(positions, "positions", torch.int32)
    out = torch.empty((n, heads * dv), dtype=torch.float32, device=q.device)
    check(_lib.load().mm_linear_state_walk(q.data_ptr(), k.data_ptr(), v.data_ptr(), q.stride(0), k.stride(0), v.stride(0), _ptr(gate),
                                           _ptr(beta), _ptr(head_decay), out.data_ptr(), state.data_ptr(), state.stride(0), _ptr(req_meta),
                                           slots.data_ptr(), positions.data_ptr(), int(n_requests), heads, qk_heads, dk, dv, _stream()),
          "linear_state_walk")
    return out


def linear_state_chunked(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, state: torch.Tensor, chunk_meta: torch.Tensor, req_chunks: torch.Tensor,
                         slots: torch.Tensor, positions: torch.Tensor, heads: int, qk_heads: int, dk: int, dv: int,
                         gate: Optional[torch.Tensor] = None, head_decay: Optional[torch.Tensor] = None) -> torch.Tensor:
    """The same recurrence without the delta rule for long portions, chunk by chunk (three launches: every chunk from a zero
    state, the carry along each request's chunks, every chunk again from its starting state).  ``chunk_meta`` [chunks, 4] =
    (first token, tokens, request, .), ``req_chunks`` [requests, 2] = (first chunk, chunks)."""
    for t, what in ((q, "q"), (k, "k"), (v, "v")):
        if t.dtype != torch.float32 or not t.is_cuda or t.stride(1) != 1:
            raise KernelError(f"linear state {what}: fp32 rows with unit column stride are needed")
    n = q.shape[0]
    if q.shape[1] != qk_heads * dk or k.shape != q.shape or v.shape != (n, heads * dv):
        raise KernelError("linear state: shape mismatch")
    if state.dtype != torch.float32 or state.stride(-1) != 1 or state.shape[1] < heads * dv * dk:
        raise KernelError("linear state: the state is fp32 [slots, >= heads * dv * dk]")
    _need(chunk_meta, "chunk_meta", torch.int32)
    _need(req_chunks, "req_chunks", torch.int32)
    _need(slots, "state slots", torch.int32)
    _need(positions, "positions", torch.int32)
    if gate is not None:
        _need(gate, "gate", torch.float32)
    if head_decay is not None:
        _need(head_decay, "head decay", torch.float32)
    n_chunks, n_req = chunk_meta.shape[0], req_chunks.shape[0]
    out = torch.empty((n, heads * dv), dtype=torch.float32, device=q.device)
    scratch = torch.empty((max(1, n_chunks), heads * dv * dk), dtype=torch.float32, device=q.device)
    gain = torch.empty((max(1, n_chunks), heads), dtype=torch.float32, device=q.device)
    check(_lib.load().mm_linear_state_chunked(q.data_ptr(), k.data_ptr(), v.data_ptr(), q.stride(0), k.stride(0), v.stride(0), _ptr(gate),
                                              _ptr(head_decay), out.data_ptr(), state.data_ptr(), state.stride(0), chunk_meta.data_ptr(),
                                              req_chunks.data_ptr(), slots.data_ptr(), positions.data_ptr(), n_req, n_chunks, heads, qk_heads,
                                              dk, dv, scratch.data_ptr(), gain.data_ptr(), _stream()), "linear_state_chunked")
    return out


GATE_ACTIVATIONS = {"silu": 1, "sigmoid": 2}


def gated_group_norm(x: torch.Tensor, groups: int, group_size: int, out_dtype: torch.dtype, *, eps: float = 0.0, normalize: bool = True,
                     weight: Optional[torch.Tensor] = None, gate: Optional[torch.Tensor] = None, activation: str = "silu") -> torch.Tensor:
    """``x[t, g, :] / rms(x[t, g, :]) * weight * act(gate[t, g, :])`` with each factor optional; ``weight`` fp32 of
    ``group_size`` (one for all groups) or ``groups * group_size``; x and gate may be column slices."""
    n = x.shape[0]
    for t, what in ((x, "x"), (gate, "gate")):
        if t is not None and (not t.is_cuda or t.stride(1) != 1 or t.shape != (n, groups * group_size)):
            raise KernelError(f"gated norm {what}: [n, groups * group_size] with unit column stride is needed")
    w_stride = 0
    if weight is not None:
        _need(weight, "gated norm weight", torch.float32)
        if weight.numel() not in (group_size, groups * group_size):
            raise KernelError("gated norm: the weight has group_size or groups * group_size numbers")
        w_stride = 0 if weight.numel() == group_size and groups > 1 else (group_size if weight.numel() == groups * group_size else 0)
    out = torch.empty((n, groups * group_size), dtype=out_dtype, device=x.device)
    check(_lib.load().mm_gated_group_norm(x.data_ptr(), dtype_code(x.dtype), x.stride(0), _ptr(gate), dtype_code(gate.dtype) if gate is not None else F32,
                                          gate.stride(0) if gate is not None else 0, _ptr(weight), w_stride, out.data_ptr(), dtype_code(out_dtype),
                                          n, groups, group_size, float(eps), int(bool(normalize)), GATE_ACTIVATIONS[activation], _stream()),
          "gated_group_norm")
    return out


def normed_mean2(a: torch.Tensor, b: torch.Tensor, wa: torch.Tensor, wb: torch.Tensor, eps: float, scale: float = 0.5) -> torch.Tensor:
    """``scale * (a / rms(a) * wa + b / rms(b) * wb)`` row by row; the weights fp32."""
    _need(a, "normed mean a")
    _need(b, "normed mean b", a.dtype)
    _need(wa, "normed mean weight", torch.float32)
    _need(wb, "normed mean weight", torch.float32)
    n, d = a.shape
    if b.shape != a.shape or wa.numel() != d or wb.numel() != d:
        raise KernelError("normed mean: shape mismatch")
    out = torch.empty_like(a)
    check(_lib.load().mm_normed_mean2(a.data_ptr(), b.data_ptr(), wa.data_ptr(), wb.data_ptr(), out.data_ptr(), dtype_code(a.dtype), n, d,
                                      float(eps), float(scale), _stream()), "normed_mean2")
    return out


# ---- mixture of experts (csrc/moe.cu) -----------------------------------------------------------------------------------
def moe_route(logits: torch.Tensor, top: int, groups: int, keep: int):
    """The router's choice from fp32 logits [n, E]: (experts int32 [n, top], weights fp32 [n, top])."""
    _need(logits, "router logits", torch.float32)
    n, E = logits.shape
    idx = torch.empty((n, top), dtype=torch.int32, device=logits.device)
    wts = torch.empty((n, top), dtype=torch.float32, device=logits.device)
    check(_lib.load().mm_moe_route(logits.data_ptr(), E, n, E, int(top), int(groups), int(keep), idx.data_ptr(), wts.data_ptr(), _stream()), "moe_route")
    return idx, wts


ROUTER_SCORINGS = {"softmax": 0, "sigmoid": 1}


def moe_router(x: torch.Tensor, w: torch.Tensor, top: int, groups: int, keep: int, scoring: str = "softmax"):
    """The router's product (fp32 sums over ``x`` [n, D] and the fp32 matrix ``w`` [E, D]) and its choice in one launch:
    (experts int32 [n, top], weights fp32 [n, top]).  ``scoring``: ``softmax`` (the chosen scores divided by their sum) or
    ``sigmoid`` (the chosen scores as they are)."""
    _need(x, "router rows")
    _need(w, "router matrix", torch.float32)
    n, D = x.shape
    E = w.shape[0]
    if w.shape[1] != D:
        raise KernelError("moe router: shape mismatch")
    idx = torch.empty((n, top), dtype=torch.int32, device=x.device)
    wts = torch.empty((n, top), dtype=torch.float32, device=x.device)
    check(_lib.load().mm_moe_router_scored(x.data_ptr(), dtype_code(x.dtype), D, w.data_ptr(), n, D, E, int(top), int(groups), int(keep),
                                           ROUTER_SCORINGS[scoring], idx.data_ptr(), wts.data_ptr(), _stream()), "moe_router")
    return idx, wts


MOE_TILE_ROWS = 128       # rows of a tile of the grouped tensor-memory product


@dataclass
class ExpertRows:
    """The step's (token, choice) rows put side by side by expert: ``offsets`` int32 [E + 1]; ``order`` int32 [rows]: the
    row (token * top + choice) at every place; and, when asked for, the row tiles of the grouped tensor-memory product
    (``tiles`` int32 [max_tiles, 3] = first row, end row, expert; ``n_tiles`` int32 [1]), every place's token
    (``row_token``) and every row's place (``place``)."""

    offsets: torch.Tensor
    order: torch.Tensor
    tiles: Optional[torch.Tensor] = None
    n_tiles: Optional[torch.Tensor] = None
    max_tiles: int = 0
    row_token: Optional[torch.Tensor] = None
    place: Optional[torch.Tensor] = None


def moe_sort(idx: torch.Tensor, experts: int, with_tiles: bool = False) -> ExpertRows:
    """Rows (token * top + choice) put side by side by expert, in their order within an expert."""
    _need(idx, "expert choice", torch.int32)
    rows, top = idx.numel(), idx.shape[-1]
    dev = idx.device
    out = ExpertRows(torch.empty((experts + 1,), dtype=torch.int32, device=dev), torch.empty((max(rows, 1),), dtype=torch.int32, device=dev))
    if with_tiles:
        out.max_tiles = -(-rows // MOE_TILE_ROWS) + experts
        out.tiles = torch.empty((out.max_tiles, 3), dtype=torch.int32, device=dev)
        out.n_tiles = torch.empty((1,), dtype=torch.int32, device=dev)
        out.row_token = torch.empty((max(rows, 1),), dtype=torch.int32, device=dev)
        out.place = torch.empty((max(rows, 1),), dtype=torch.int32, device=dev)
    check(_lib.load().mm_moe_sort(idx.data_ptr(), rows, int(experts), out.offsets.data_ptr(), out.order.data_ptr(), int(top), MOE_TILE_ROWS,
                                  _ptr(out.tiles), _ptr(out.n_tiles), _ptr(out.row_token), _ptr(out.place), _stream()), "moe_sort")
    return out


GLU_ACTIVATIONS = {"silu": 0, "clamped": 1}


def moe_gemm(a: torch.Tensor, w: torch.Tensor, rows: ExpertRows, n_rows: int, top: int, gated: bool,
             out_dtype: torch.dtype, tensor_cores: bool = True, interleaved: bool = False, activation: str = "silu", limit: float = 0.0,
             row_scale: Optional[torch.Tensor] = None) -> torch.Tensor:
    """The experts' products over their rows.  ``gated``: ``a`` [tokens, K] are the step's rows, ``w`` [E, 2F, K] the gate's
    rows then the up rows of every expert (``interleaved``: alternating in blocks of 8), result ``silu(gate) * up``
    [n_rows, F] in sorted order.  Otherwise ``a`` [n_rows, K] are sorted rows, ``w`` [E, N, K], and row ``order[i]`` of the
    result [n_rows, N] gets sorted row i's product.  A gated product may take another ``activation`` (``clamped``:
    ``g = min(g, limit)``, ``u = clamp(u, -limit, limit)``, ``g sigmoid(1.702 g) (u + 1)``) and a ``row_scale`` fp32 [tokens, top]
    that multiplies both halves of a (token, choice) row before it (a weight on the expert's input)."""
    _need(a, "moe rows")
    if row_scale is not None:
        _need(row_scale, "moe row scale", torch.float32)
        if row_scale.numel() != n_rows:
            raise KernelError("moe gemm: one scale per (token, choice) row is needed")
    _need(w, "moe weights", a.dtype)
    E, rows_w, K = w.shape
    N = rows_w // 2 if gated else rows_w
    if a.shape[1] != K or (not gated and a.shape[0] != n_rows):
        raise KernelError("moe gemm: shape mismatch")
    out = torch.empty((n_rows, N), dtype=out_dtype, device=a.device)
    check(_lib.load().mm_moe_gemm_act(a.data_ptr(), dtype_code(a.dtype), a.stride(0), w.data_ptr(), dtype_code(w.dtype), out.data_ptr(),
                                      dtype_code(out_dtype), N, rows.offsets.data_ptr(), rows.order.data_ptr(), int(n_rows), E, int(top), N, K,
                                      int(bool(gated)), int(bool(tensor_cores)), int(bool(interleaved)), GLU_ACTIVATIONS[activation],
                                      float(limit), _ptr(row_scale), _stream()), "moe_gemm")
    return out


def moe_gather_scaled(x: torch.Tensor, rows: ExpertRows, wts: Optional[torch.Tensor]) -> torch.Tensor:
    """The step's rows in sorted order, each multiplied by its (token, choice)'s weight (``wts`` fp32 [tokens, top]; None: a
    plain copy) and rounded to their dtype: what the grouped products of experts that weigh their input read."""
    _need(x, "moe rows")
    if rows.row_token is None:
        raise KernelError("moe gather: the rows were sorted without their tile list")
    if wts is not None:
        _need(wts, "moe weights", torch.float32)
    n_rows = rows.row_token.numel()
    out = torch.empty((n_rows, x.shape[1]), dtype=x.dtype, device=x.device)
    check(_lib.load().mm_moe_gather_scaled(x.data_ptr(), dtype_code(x.dtype), rows.row_token.data_ptr(), rows.order.data_ptr(), _ptr(wts),
                                           out.data_ptr(), n_rows, x.shape[1], _stream()), "moe_gather_scaled")
    return out


def moe_gemm_grouped(a: torch.Tensor, w: torch.Tensor, rows: ExpertRows, swiglu: bool, activation: str = "silu", limit: float = 0.0) -> torch.Tensor:
    """The grouped tensor-memory product: ``a`` [n_rows, K] bf16 in sorted order, ``w`` [E, N, K] bf16; every row tile of
    ``rows.tiles`` times its expert's matrix.  ``swiglu``: the matrix interleaves gate and up rows in blocks of 8 and the
    result is ``silu(gate) * up`` [n_rows, N/2]; else [n_rows, N].  bf16, in sorted order."""
    _need(a, "moe rows", torch.bfloat16)
    _need(w, "moe weights", torch.bfloat16)
    if rows.tiles is None:
        raise KernelError("moe gemm: the rows were sorted without their tile list")
    n_rows, K = a.shape
    E, N, _ = w.shape
    out = torch.empty((n_rows, N // 2 if swiglu else N), dtype=torch.bfloat16, device=a.device)
    check(_lib.load().mm_gemm_tcgen05_grouped_act(a.data_ptr(), w.data_ptr(), out.data_ptr(), 1 if swiglu else 0, n_rows, E, N, K, K, out.shape[1],
                                                  rows.tiles.data_ptr(), rows.n_tiles.data_ptr(), rows.max_tiles,
                                                  GLU_ACTIVATIONS[activation] if swiglu else 0, float(limit),
                                                  tcgen05_error_flag(a.device).data_ptr(), _stream()), "gemm_tcgen05_grouped")
    return out


def moe_combine(y: torch.Tensor, wts: Optional[torch.Tensor], out_dtype: torch.dtype, place: Optional[torch.Tensor] = None,
                top: Optional[int] = None) -> torch.Tensor:
    """``out[t] = sum_c wts[t, c] * y[row(t, c)]`` in the order of the choice; ``row(t, c) = t * top + c``, or
    ``place[t * top + c]`` when ``y`` stands in sorted order.  ``wts`` None (then ``top`` says how many rows a token has):
    the plain sum."""
    _need(y, "moe outputs")
    if wts is not None:
        _need(wts, "moe weights", torch.float32)
        n, top = wts.shape
    else:
        top = int(top)
        n = y.shape[0] // top
    d = y.shape[1]
    if y.shape[0] != n * top:
        raise KernelError("moe combine: shape mismatch")
    out = torch.empty((n, d), dtype=out_dtype, device=y.device)
    check(_lib.load().mm_moe_combine(y.data_ptr(), dtype_code(y.dtype), _ptr(wts), _ptr(place), out.data_ptr(), dtype_code(out_dtype), n, top, d,
                                     _stream()), "moe_combine")
    return out


# ---- residual connections over several streams (csrc/hyper_connections.cu) ---------------------------------------------
def stream_copies(x: torch.Tensor, streams: int) -> torch.Tensor:
    """fp32 [n, D] -> fp32 [n, streams * D]: every stream starts as a copy of the row."""
    _need(x, "stream copies", torch.float32)
    n, d = x.shape
    out = torch.empty((n, streams * d), dtype=torch.float32, device=x.device)
    check(_lib.load().mm_stream_copies(x.data_ptr(), out.data_ptr(), n, int(streams), d, _stream()), "stream_copies")
    return out


def hc_read(x: torch.Tensor, streams: int, a: torch.Tensor, norm_weight: Optional[torch.Tensor], eps: float, out_dtype: torch.dtype,
            rows: Optional[torch.Tensor] = None, n_rows: Optional[int] = None) -> torch.Tensor:
    """``u = sum_s a[s] x_s`` over the streams of ``x`` (fp32 [n, streams * D]) and, with ``norm_weight``, its RMS norm
    ``u w / sqrt(mean(u^2) + eps)``; with ``rows`` output row i is made from source row rows[i]."""
    _need(x, "streams", torch.float32)
    _need(a, "stream weights", torch.float32)
    n, d = x.shape[0], x.shape[1] // streams
    if x.shape[1] != streams * d or a.numel() != streams:
        raise KernelError("stream read: shape mismatch")
    if norm_weight is not None:
        _need(norm_weight, "norm weight")
        if norm_weight.numel() != d:
            raise KernelError("stream read: the norm weight has another width")
    if rows is not None:
        _need(rows, "rows", torch.int32)
        n = int(n_rows) if n_rows is not None else rows.numel()
    out = torch.empty((n, d), dtype=out_dtype, device=x.device)
    check(_lib.load().mm_hc_read(x.data_ptr(), _ptr(rows), a.data_ptr(), _ptr(norm_weight),
                                 dtype_code(norm_weight.dtype) if norm_weight is not None else F32, float(eps), out.data_ptr(),
                                 dtype_code(out_dtype), n, int(streams), d, _stream()), "hc_read")
    return out


def hc_write(x: torch.Tensor, streams: int, y: torch.Tensor, scale: Optional[torch.Tensor], mix: torch.Tensor, b: torch.Tensor,
             a_next: Optional[torch.Tensor] = None, norm_weight: Optional[torch.Tensor] = None, eps: float = 0.0,
             out_dtype: Optional[torch.dtype] = None) -> Optional[torch.Tensor]:
    """All streams at once from the old ones, in place: ``x_t <- sum_s mix[s, t] x_s + b[t] (scale . y)``.  With ``a_next``
    the next sublayer's input ``sum_t a_next[t] x_t`` (RMS-normed with ``norm_weight`` if given) comes out of the same pass."""
    _need(x, "streams", torch.float32)
    _need(y, "branch")
    _need(mix, "stream mix", torch.float32)
    _need(b, "stream out", torch.float32)
    n, d = x.shape[0], x.shape[1] // streams
    if x.shape[1] != streams * d or y.shape != (n, d) or mix.numel() != streams * streams or b.numel() != streams:
        raise KernelError("stream write: shape mismatch")
    if scale is not None:
        _need(scale, "layer scale", torch.float32)
        if scale.numel() != d:
            raise KernelError("stream write: the layer scale has another width")
    out = None
    if a_next is not None:
        _need(a_next, "stream weights", torch.float32)
        if a_next.numel() != streams:
            raise KernelError("stream write: shape mismatch")
        if norm_weight is not None:
            _need(norm_weight, "norm weight")
        out = torch.empty((n, d), dtype=out_dtype or y.dtype, device=x.device)
    check(_lib.load().mm_hc_write(x.data_ptr(), y.data_ptr(), dtype_code(y.dtype), _ptr(scale), mix.data_ptr(), b.data_ptr(), _ptr(a_next),
                                  _ptr(norm_weight) if a_next is not None else None,
                                  dtype_code(norm_weight.dtype) if norm_weight is not None else F32, float(eps), _ptr(out),
                                  dtype_code(out.dtype) if out is not None else F32, n, int(streams), d, _stream()), "hc_write")
    return out


# ---- steps around an attention kernel (csrc/attention_parts.cu) --------------------------------------------------------
def rope_half_table(positions: torch.Tensor, f_hi: torch.Tensor, f_lo: torch.Tensor) -> torch.Tensor:
    """(cos, sin) of ``position * (f_hi[i] + f_lo[i])`` as fp32 [n, len(f_hi), 2]; the two words of each frequency come from
    its float64 value, and the rounding of the product is carried, so the angle is good to the last bit of an fp32."""
    _need(positions, "positions", torch.int32)
    _need(f_hi, "frequencies", torch.float32)
    _need(f_lo, "frequencies", torch.float32)
    n, half = positions.numel(), f_hi.numel()
    if f_lo.numel() != half or half < 1:
        raise KernelError("rotation table: bad sizes")
    out = torch.empty((n, half, 2), dtype=torch.float32, device=positions.device)
    check(_lib.load().mm_rope_half_table(positions.data_ptr(), f_hi.data_ptr(), f_lo.data_ptr(), out.data_ptr(), n, half, _stream()), "rope_half_table")
    return out


def qkv_split_post(rows: torch.Tensor, q_off: int, k_off: int, v_off: int, q_out: torch.Tensor, k_pages: Optional[torch.Tensor],
                   v_pages: Optional[torch.Tensor], slots: Optional[torch.Tensor], page_size: int, q_heads: int, k_heads: int, key_dim: int,
                   v_heads: int, value_dim: int) -> None:
    """Cuts fp32 rows [n, ld] into queries (``q_heads * key_dim`` numbers at ``q_off``, written to ``q_out``), keys
    (``k_heads * key_dim`` at ``k_off``) and values (``v_heads * value_dim`` at ``v_off``), the last two written into
    their pages ``[pages, heads, page_size, size]`` at ``slots``."""
    if rows.dtype != torch.float32 or not rows.is_cuda or rows.stride(1) != 1:
        raise KernelError("qkv split: fp32 rows with unit column stride are needed")
    n = rows.shape[0]
    _need(q_out, "q_out")
    if q_out.shape != (n, q_heads * key_dim):
        raise KernelError("qkv split: q_out has another shape")
    if k_pages is not None:
        _need(k_pages, "k_pages", q_out.dtype)
        _need(v_pages, "v_pages", q_out.dtype)
        _need(slots, "slots", torch.int32)
        if k_pages.shape[1:] != (k_heads, page_size, key_dim) or v_pages.shape[1:] != (v_heads, page_size, value_dim):
            raise KernelError("qkv split: page pool shape mismatch")
    check(_lib.load().mm_qkv_split_post(rows.data_ptr(), rows.stride(0), int(q_off), int(k_off), int(v_off), q_out.data_ptr(), _ptr(k_pages),
                                        _ptr(v_pages), dtype_code(q_out.dtype), _ptr(slots) if k_pages is not None else None, int(page_size), n,
                                        int(q_heads), int(k_heads), int(key_dim), int(v_heads), int(value_dim), _stream()), "qkv_split_post")


def latent_prep(rows: torch.Tensor, q_off: int, c_off: int, norm_weight: torch.Tensor, eps: float, rot: Optional[torch.Tensor], rot_dims: int,
                q_plain: torch.Tensor, q_full: torch.Tensor, pages: Optional[torch.Tensor], slots: Optional[torch.Tensor], page_size: int,
                heads: int, dim: int, rot_dim: int, rank: int) -> None:
    """Between the projections of a latent attention and its kernel: from fp32 rows [n, ld] (every head's ``dim`` plain and
    ``rot_dim`` rotated query numbers at ``q_off``; the latent's ``rank`` numbers and the shared key part's ``rot_dim`` at
    ``c_off``) the plain query parts go to ``q_plain`` [n, heads * dim], the turned ones into ``q_full``
    [n, heads, rank + rot_dim] behind each head's first ``rank`` places, and (normed latent, turned key part) into the
    pages [pages, 1, page_size, rank + rot_dim] at ``slots``."""
    if rows.dtype != torch.float32 or not rows.is_cuda or rows.stride(1) != 1:
        raise KernelError("latent prep: fp32 rows with unit column stride are needed")
    n = rows.shape[0]
    _need(q_plain, "q_plain")
    _need(q_full, "q_full", q_plain.dtype)
    _need(norm_weight, "latent norm weight")
    if q_plain.shape != (n, heads * dim) or q_full.shape != (n, heads * (rank + rot_dim)) or norm_weight.numel() != rank:
        raise KernelError("latent prep: shape mismatch")
    if rot_dims:
        _need(rot, "rotation table", torch.float32)
        if rot.shape != (n, rot_dims // 2, 2):
            raise KernelError("latent prep: rotation table of another shape")
    if pages is not None:
        _need(pages, "latent pages", q_plain.dtype)
        _need(slots, "slots", torch.int32)
        if pages.shape[1:] != (1, page_size, rank + rot_dim):
            raise KernelError("latent prep: page pool shape mismatch")
    check(_lib.load().mm_latent_prep(rows.data_ptr(), rows.stride(0), int(q_off), int(c_off), norm_weight.data_ptr(), dtype_code(norm_weight.dtype),
                                     float(eps), _ptr(rot) if rot_dims else None, int(rot_dims), q_plain.data_ptr(), q_full.data_ptr(), _ptr(pages),
                                     dtype_code(q_plain.dtype), _ptr(slots) if pages is not None else None, int(page_size), n, int(heads), int(dim),
                                     int(rot_dim), int(rank), _stream()), "latent_prep")


HEAD_MATMUL_LIBRARY_FROM = 64      # rows from which the per-head products of bfloat16 rows are one batched library product


def head_matmul(x: torch.Tensor, matrices: torch.Tensor, out: torch.Tensor, heads: int) -> torch.Tensor:
    """``out[t, h, :] = x[t, h, :] . matrices[h]`` with ``matrices`` [heads, K, N]; ``x`` is [n, heads * K] and ``out``
    [n, heads * N'] with N' >= N (each head's result goes to the first N places of its N' wide part); both may be column
    slices of wider rows."""
    H, K, N = matrices.shape
    n = x.shape[0]
    if H != heads or x.shape[1] != H * K or out.shape[0] != n or out.shape[1] % H or out.shape[1] // H < N:
        raise KernelError("head product: shape mismatch")
    if x.dtype != matrices.dtype or out.dtype != x.dtype or not matrices.is_contiguous() or x.stride(1) != 1 or out.stride(1) != 1:
        raise KernelError("head product: one dtype and unit column strides are needed")
    if x.dtype == torch.bfloat16 and n >= HEAD_MATMUL_LIBRARY_FROM and x.is_contiguous() and out.is_contiguous():
        # a portion of a prompt: one batched product of the vendor library over the heads, operands and result in place
        wide = out.shape[1] // H
        torch.bmm(x.view(n, H, K).transpose(0, 1), matrices, out=out.view(n, H, wide)[:, :, :N].transpose(0, 1))
        return out
    check(_lib.load().mm_head_matmul(x.data_ptr(), x.stride(0), K, matrices.data_ptr(), out.data_ptr(), out.stride(0), out.shape[1] // H,
                                     dtype_code(x.dtype), n, H, K, N, _stream()), "head_matmul")
    return out


def head_finish(att: torch.Tensor, heads: int, value_dim: int, *, pair: bool = False, lam: float = 0.0, eps: Optional[float] = None,
                post: float = 1.0, gate: Optional[torch.Tensor] = None, out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """Per (token, head) of an attention output ``att`` [n, heads_in * value_dim] (``pair``: heads_in = 2 * heads and head h's
    second map is head ``heads + h``): ``o = a1 - lam * a2``; with ``eps`` ``o / sqrt(mean(o^2) + eps)``; times ``post`` and
    ``sigmoid(gate[t, h])`` (``gate`` fp32 [n, >= heads], may be a column slice).  Returns [n, heads * value_dim] of
    ``out_dtype`` (default: that of ``att``; an fp32 ``att`` may be given out as bfloat16)."""
    _need(att, "attention output")
    n = att.shape[0]
    heads_in = 2 * heads if pair else heads
    if att.shape != (n, heads_in * value_dim):
        raise KernelError("head finish: shape mismatch")
    if gate is not None and (gate.dtype != torch.float32 or not gate.is_cuda or gate.stride(1) != 1 or gate.shape[0] != n or gate.shape[1] < heads):
        raise KernelError("head finish: the gate is fp32 [n, heads] with unit column stride")
    out_dtype = out_dtype or att.dtype
    if out_dtype != att.dtype and att.dtype != torch.float32:
        raise KernelError("head finish: only an fp32 input can be given out in another type")
    out = torch.empty((n, heads * value_dim), dtype=out_dtype, device=att.device)
    check(_lib.load().mm_head_finish(att.data_ptr(), heads_in, heads if pair else 0, float(lam), int(eps is not None), float(eps or 0.0), float(post),
                                     _ptr(gate), gate.stride(0) if gate is not None else 0, out.data_ptr(), dtype_code(att.dtype),
                                     dtype_code(out_dtype), n, int(heads),
                                     int(value_dim), _stream()), "head_finish")
    return out


# ---- attention with mixed heads (csrc/attention_talking.cu) -----------------------------------------------------------------
def talking_prep(rows: torch.Tensor, q_off: int, k_off: int, v_off: int, q_norm: Optional[torch.Tensor], k_norm: Optional[torch.Tensor],
                 eps: float, rot: Optional[torch.Tensor], rot_dims: int, v_unit: bool, q_out: torch.Tensor, k_pages: Optional[torch.Tensor],
                 v_pages: Optional[torch.Tensor], slots: Optional[torch.Tensor], page_size: int, heads: int, kv_heads: int, key_dim: int,
                 value_dim: int) -> None:
    """Between the projections (and convolutions) of an attention and its kernel: from fp32 rows [n, ld] every q head
    (``heads * key_dim`` numbers at ``q_off``) and k head (``kv_heads * key_dim`` at ``k_off``) is RMS-normed over its
    ``key_dim`` numbers with the fp32 weight ``q_norm`` / ``k_norm`` (None: not normed) and its first ``rot_dims`` numbers
    are turned by ``rot`` [n, rot_dims/2, 2] (number i pairs with i + rot_dims/2); every v head (``kv_heads * value_dim``
    at ``v_off``) is divided by its root mean square when ``v_unit``.  q goes to ``q_out`` [n, heads * key_dim], k and v
    into their pages ``[pages, kv_heads, page_size, size]`` at ``slots``."""
    if rows.dtype != torch.float32 or not rows.is_cuda or rows.stride(1) != 1:
        raise KernelError("attention prep: fp32 rows with unit column stride are needed")
    n = rows.shape[0]
    _need(q_out, "q_out")
    if q_out.shape != (n, heads * key_dim):
        raise KernelError("attention prep: q_out has another shape")
    for w, what in ((q_norm, "q norm"), (k_norm, "k norm")):
        if w is not None:
            _need(w, what, torch.float32)
            if w.numel() != key_dim:
                raise KernelError(f"attention prep: the {what} weight has one number per key channel")
    if rot_dims:
        _need(rot, "rotation table", torch.float32)
        if rot.shape != (n, rot_dims // 2, 2):
            raise KernelError("attention prep: rotation table of another shape")
    if max(q_off + heads * key_dim, k_off + kv_heads * key_dim, v_off + kv_heads * value_dim) > rows.shape[1]:
        raise KernelError("attention prep: columns outside the row")
    if k_pages is not None:
        _need(k_pages, "k_pages", q_out.dtype)
        _need(v_pages, "v_pages", q_out.dtype)
        _need(slots, "slots", torch.int32)
        if k_pages.shape[1:] != (kv_heads, page_size, key_dim) or v_pages.shape[1:] != (kv_heads, page_size, value_dim):
            raise KernelError("attention prep: page pool shape mismatch")
    check(_lib.load().mm_talking_prep(rows.data_ptr(), rows.stride(0), int(q_off), int(k_off), int(v_off), _ptr(q_norm), _ptr(k_norm), float(eps),
                                      _ptr(rot) if rot_dims else None, int(rot_dims), int(bool(v_unit)), q_out.data_ptr(), _ptr(k_pages),
                                      _ptr(v_pages), dtype_code(q_out.dtype), _ptr(slots) if k_pages is not None else None, int(page_size), n,
                                      int(heads), int(kv_heads), int(key_dim), int(value_dim), _stream()), "talking_prep")


def attention_talking(q: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor, out: torch.Tensor, positions: torch.Tensor,
                      token_req: torch.Tensor, block_table: torch.Tensor, page_size: int, num_heads: int, num_kv_heads: int, key_dim: int,
                      value_dim: int, window: int, scale: float, talk: Optional[torch.Tensor], sink: Optional[torch.Tensor],
                      splits: int = 1, scratch=None) -> torch.Tensor:
    """Causal (or windowed) attention whose scaled scores are mixed between the heads before the softmax,
    ``s_h = sum_g talk[h, g] r_g`` (``talk`` fp32 [H, H]; None: not mixed), with ``exp(sink_h)`` in head h's denominator
    (``sink`` fp32 [H]; None: plain softmax); fp32 arithmetic, any sizes.  ``splits`` > 1 shares a token's keys out over
    that many blocks (``scratch``: fp32 [n, H, splits, dv] and [n, H, splits, 2]) and merges them in a second launch."""
    _need(q, "q")
    _need(k_pages, "k_pages", q.dtype)
    _need(v_pages, "v_pages", q.dtype)
    _need(out, "attention out", q.dtype)
    _need(positions, "positions", torch.int32)
    _need(token_req, "token_req", torch.int32)
    _need(block_table, "block_table", torch.int32)
    n = q.shape[0]
    if q.shape != (n, num_heads * key_dim) or out.shape != (n, num_heads * value_dim):
        raise KernelError("attention: q or out has another shape")
    if k_pages.shape[1:] != (num_kv_heads, page_size, key_dim) or v_pages.shape[1:] != (num_kv_heads, page_size, value_dim):
        raise KernelError("attention: page pool shape mismatch")
    for t, what, count in ((talk, "head mixing matrix", num_heads * num_heads), (sink, "sink logits", num_heads)):
        if t is not None:
            _need(t, what, torch.float32)
            if t.numel() != count:
                raise KernelError(f"attention: the {what} has another size")
    part_o = part_ml = None
    if splits > 1:
        part_o, part_ml = scratch if scratch is not None else (
            torch.empty((n, num_heads, splits, value_dim), dtype=torch.float32, device=q.device),
            torch.empty((n, num_heads, splits, 2), dtype=torch.float32, device=q.device))
    check(_lib.load().mm_attention_talking(q.data_ptr(), k_pages.data_ptr(), v_pages.data_ptr(), out.data_ptr(), dtype_code(q.dtype), _ptr(part_o),
                                           _ptr(part_ml), int(splits), positions.data_ptr(), token_req.data_ptr(), block_table.data_ptr(),
                                           block_table.shape[1], int(page_size), n, int(num_heads), int(num_kv_heads), int(key_dim), int(value_dim),
                                           int(window), float(scale), _ptr(talk), _ptr(sink), _stream()), "attention_talking")
    return out


# ---- a forget gate per key channel (csrc/linear_state.cu) -----------------------------------------------------------------------
def forget_gate_prep(x: torch.Tensor, q_off: int, f_off: int, n_qf: int, bias: Optional[torch.Tensor], lower: Optional[torch.Tensor],
                     silu_q: bool = True) -> None:
    """In place on the fp32 rows ``x`` [n, ld]: silu on the ``n_qf`` numbers at ``q_off``; the ``n_qf`` numbers ``z`` at
    ``f_off`` become the forget gate ``l + (1 - l) sigmoid(z + bias)`` with the lower bound ``l`` per channel (both fp32
    [n_qf] or None)."""
    _need(x, "projection rows", torch.float32)
    for t, what in ((bias, "forget bias"), (lower, "lower bound")):
        if t is not None:
            _need(t, what, torch.float32)
            if t.numel() != n_qf:
                raise KernelError(f"forget gate: the {what} has one number per channel")
    check(_lib.load().mm_forget_gate_prep(x.data_ptr(), x.shape[1], x.shape[0], int(q_off), int(f_off), int(n_qf), int(bool(silu_q)), _ptr(bias),
                                          _ptr(lower), _stream()), "forget_gate_prep")


def forget_gate_walk(q: torch.Tensor, f: torch.Tensor, v: torch.Tensor, state: torch.Tensor, req_meta: Optional[torch.Tensor],
                     slots: torch.Tensor, positions: torch.Tensor, n_requests: int, heads: int, dk: int, dv: int) -> torch.Tensor:
    """Per head ``S <- diag(f) S + (1 - f) v^T; o = S^T q`` over each request's tokens in order.  q, f: fp32 column slices
    [n, heads * dk], v [n, heads * dv] (any row stride); ``state`` [slots, stride] fp32 holds S as [heads, dv, dk] at its
    start and is left updated.  Returns o fp32 [n, heads * dv]."""
    for t, what in ((q, "q"), (f, "f"), (v, "v")):
        if t.dtype != torch.float32 or not t.is_cuda or t.stride(1) != 1:
            raise KernelError(f"forget gate walk {what}: fp32 rows with unit column stride are needed")
    n = q.shape[0]
    if q.shape[1] != heads * dk or f.shape != q.shape or v.shape != (n, heads * dv):
        raise KernelError("forget gate walk: shape mismatch")
    if state.dtype != torch.float32 or state.stride(-1) != 1 or state.shape[1] < heads * dv * dk:
        raise KernelError("forget gate walk: the state is fp32 [slots, >= heads * dv * dk]")
    _need(slots, "state slots", torch.int32)
    _need(positions, "positions", torch.int32)
    out = torch.empty((n, heads * dv), dtype=torch.float32, device=q.device)
    check(_lib.load().mm_forget_gate_walk(q.data_ptr(), f.data_ptr(), v.data_ptr(), q.stride(0), f.stride(0), v.stride(0), out.data_ptr(),
                                          state.data_ptr(), state.stride(0), _ptr(req_meta), slots.data_ptr(), positions.data_ptr(),
                                          int(n_requests), int(heads), int(dk), int(dv), _stream()), "forget_gate_walk")
    return out


def forget_gate_chunked(q: torch.Tensor, f: torch.Tensor, v: torch.Tensor, state: torch.Tensor, chunk_meta: torch.Tensor, req_chunks: torch.Tensor,
                        slots: torch.Tensor, positions: torch.Tensor, heads: int, dk: int, dv: int) -> torch.Tensor:
    """The same recurrence for long portions, chunk by chunk (three launches: every chunk from a zero state, the carry along
    each request's chunks, every chunk again from its starting state).  ``chunk_meta`` [chunks, 4] = (first token, tokens,
    request, .), ``req_chunks`` [requests, 2] = (first chunk, chunks)."""
    for t, what in ((q, "q"), (f, "f"), (v, "v")):
        if t.dtype != torch.float32 or not t.is_cuda or t.stride(1) != 1:
            raise KernelError(f"forget gate walk {what}: fp32 rows with unit column stride are needed")
    n = q.shape[0]
    if q.shape[1] != heads * dk or f.shape != q.shape or v.shape != (n, heads * dv):
        raise KernelError("forget gate walk: shape mismatch")
    if state.dtype != torch.float32 or state.stride(-1) != 1 or state.shape[1] < heads * dv * dk:
        raise KernelError("forget gate walk: the state is fp32 [slots, >= heads * dv * dk]")
    _need(chunk_meta, "chunk_meta", torch.int32)
    _need(req_chunks, "req_chunks", torch.int32)
    _need(slots, "state slots", torch.int32)
    _need(positions, "positions", torch.int32)
    n_chunks, n_req = chunk_meta.shape[0], req_chunks.shape[0]
    out = torch.empty((n, heads * dv), dtype=torch.float32, device=q.device)
    scratch = torch.empty((max(1, n_chunks), heads * dv * dk), dtype=torch.float32, device=q.device)
    gain = torch.empty((max(1, n_chunks), heads * dk), dtype=torch.float32, device=q.device)
    check(_lib.load().mm_forget_gate_chunked(q.data_ptr(), f.data_ptr(), v.data_ptr(), q.stride(0), f.stride(0), v.stride(0), out.data_ptr(),
                                             state.data_ptr(), state.stride(0), chunk_meta.data_ptr(), req_chunks.data_ptr(), slots.data_ptr(),
                                             positions.data_ptr(), n_req, n_chunks, int(heads), int(dk), int(dv), scratch.data_ptr(), gain.data_ptr(),
                                             _stream()), "forget_gate_chunked")
    return out


# ---- the norm after the sum, gated activations as a pass of their own (csrc/post_norm.cu) ------------------------------------------
def post_norm(residual: torch.Tensor, a: Optional[torch.Tensor], b: Optional[torch.Tensor], weight: torch.Tensor, eps: float, alpha: float,
              ca: float = 1.0, cb: float = 1.0, out: Optional[torch.Tensor] = None) -> Optional[torch.Tensor]:
    """``y = alpha x + ca a + cb b``, ``x <- y / sqrt(mean(y^2) + eps) * weight`` on the fp32 residual ``x`` [n, D] in place;
    a, b: branch outputs [n, D] of one dtype (either may be None); ``out`` also gets the new rows in its own dtype."""
    _need(residual, "residual", torch.float32)
    _need(weight, "norm weight", torch.float32)
    n, D = residual.shape
    dt = None
    for t in (a, b):
        if t is not None:
            _need(t, "branch", dt)
            dt = t.dtype
            if t.shape != (n, D):
                raise KernelError("post norm: a branch has another shape")
    if out is not None:
        _need(out, "post norm out")
        if out.shape != (n, D):
            raise KernelError("post norm: out has another shape")
    if a is None and b is not None:
        a, ca, b = b, cb, None
    b_dtype = dtype_code(dt) if dt is not None else F32                  # no branch: the kernel reads none
    out_dtype = dtype_code(out.dtype) if out is not None else b_dtype    # no out: the kernel writes none
    check(_lib.load().mm_post_norm(residual.data_ptr(), _ptr(a), _ptr(b), b_dtype, weight.data_ptr(), _ptr(out), out_dtype, n, D, float(alpha),
                                   float(ca), float(cb), float(eps), _stream()), "post_norm")
    return out


def glu_rows(gate_up: torch.Tensor, out_dtype: torch.dtype, activation: str = "silu", limit: float = 0.0,
             row_scale: Optional[torch.Tensor] = None) -> torch.Tensor:
    """The gated activation of rows [n, 2F] whose first F columns are the gate's and the rest the up projection's
    (``GLU_ACTIVATIONS``), each row multiplied by ``row_scale`` [n] first when given: [n, F] of ``out_dtype``."""
    if not gate_up.is_cuda or gate_up.stride(1) != 1 or gate_up.shape[1] % 2:
        raise KernelError("gated activation: rows of an even width with unit column stride are needed")
    n, F2 = gate_up.shape
    if row_scale is not None:
        _need(row_scale, "row scale", torch.float32)
    out = torch.empty((n, F2 // 2), dtype=out_dtype, device=gate_up.device)
    check(_lib.load().mm_glu_rows(gate_up.data_ptr(), dtype_code(gate_up.dtype), gate_up.stride(0), out.data_ptr(), dtype_code(out_dtype), n, F2 // 2,
                                  GLU_ACTIVATIONS[activation], float(limit), _ptr(row_scale), _stream()), "glu_rows")
    return out


def cast_rows(x: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
    """fp32 rows in ``out_dtype``."""
    _need(x, "rows", torch.float32)
    out = torch.empty(x.shape, dtype=out_dtype, device=x.device)
    check(_lib.load().mm_cast_rows(x.data_ptr(), out.data_ptr(), dtype_code(out_dtype), x.numel(), _stream()), "cast_rows")
    return out


def scaled_sum2(a: torch.Tensor, b: torch.Tensor, ca: float, cb: float) -> torch.Tensor:
    """``ca * a + cb * b`` element by element."""
    _need(a, "scaled sum a")
    _need(b, "scaled sum b", a.dtype)
    if a.shape != b.shape:
        raise KernelError("scaled sum: shape mismatch")
    out = torch.empty_like(a)
    check(_lib.load().mm_scaled_sum2(a.data_ptr(), b.data_ptr(), out.data_ptr(), dtype_code(a.dtype), a.numel(), float(ca), float(cb), _stream()),
          "scaled_sum2")
    return out
