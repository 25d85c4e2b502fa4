"""ctypes binding of the CUDA kernel library.

The library exports plain C entry points (``mm_*``) that take device pointers, sizes
and a stream and return an error code; this module loads it, declares the prototypes
and turns a non-zero code into :class:`KernelError` carrying the library's message.
There is no fallback: if the library cannot be built or loaded, the error surfaces.
"""
from __future__ import annotations

import ctypes
import threading
from ctypes import c_float, c_int, c_longlong, c_ulonglong, c_void_p
from typing import Optional

from .build import library_path


class KernelError(RuntimeError):
    pass


_lock = threading.Lock()
_lib: Optional[ctypes.CDLL] = None

P = c_void_p
I = c_int
F = c_float

_PROTOTYPES = {
    "mm_embedding": [P, P, I, P, I, I, I, F, P],
    "mm_add_rmsnorm": [P, P, P, P, I, P, I, I, I, F, P],
    "mm_add_residual": [P, P, I, c_longlong, P],
    "mm_silu_mul": [P, P, I, I, I, I, P],
    "mm_gemm_tcgen05": [P, P, P, I, P, I, I, I, I, I, I, P, P],
    "mm_gemm_tcgen05_act": [P, P, P, I, P, I, I, I, I, I, I, I, P, P],
    "mm_gemm_tcgen05_pair": [P, P, P, I, P, I, I, I, I, I, I, P, P],
    "mm_gemv_bf16": [P, P, P, I, P, I, I, I, I, I, I, I, I, I, P, I, I, F, P],
    "mm_blas_gemm_nt": [P, P, P, P, I, I, I, I, P],
    "mm_gemv_bf16_act": [P, P, P, I, P, I, I, I, I, I, I, I, I, I, P],
    "mm_gemv_bf16_residual": [P, P, P, P, I, P, P, I, I, I, I, I, I, P, I, I, F, P],
    "mm_gemv_bf16_qkv_rope": [P, P, P, I, P, P, P, P, P, I, I, I, I, I, I, I, I, I, P, I, I, F, P],
    "mm_gemm_skinny": [P, P, P, I, P, I, I, I, I, I, I, I, I, P, I, I, I, F, P, P],
    "mm_gemm_skinny_residual": [P, P, P, P, I, P, P, I, I, I, I, I, I, P, I, I, I, F, P, P],
    "mm_gemm_skinny_qkv_rope": [P, P, P, I, P, P, P, P, P, I, I, I, I, I, I, I, I, P, I, I, I, F, P, P],
    "mm_rope_table": [P, P, I, I, F, P],
    "mm_slot_mapping": [P, P, P, I, I, I, P, P],
    "mm_qkv_rope_kvwrite": [P, P, I, P, P, P, I, P, P, P, I, I, I, I, I, I, I, F, I, P],
    "mm_qkv_rope_tables": [P, P, I, P, P, P, P, P, I, I, I, I, I, I, P],
    "mm_gather_rows": [P, P, P, I, I, I, P],
    "mm_attention_generic": [P, P, P, P, I, P, P, P, I, I, I, I, I, I, I, F, P],
    "mm_gemm_simt": [P, I, P, I, P, I, P, I, I, I, I, I, I, P],
    "mm_argmax_rows": [P, P, I, I, P],
    "mm_argmax_rows_split": [P, P, P, P, I, I, I, P],
    "mm_sample_rows": [P, P, I, I, P, P, P, P, P, P],
    "mm_apply_penalties": [P, I, I, P, I, P, P, P, P, P],
    "mm_window_push": [P, I, I, P, P, P, P],
    "mm_group_norm_chain": [P, P, P, P, I, P, P, I, I, I, I, F, P],
    "mm_group_norm_rows": [P, P, I, P, I, I, I, I, F, P],
    "mm_embedding_bigram": [P, P, P, P, P, P, P, P, I, P, I, I, I, I, c_longlong, c_longlong, P],
    "mm_qkv_pairs_post": [P, P, P, P, P, I, P, P, I, I, I, I, I, I, I, I, F, P],
    "mm_rope_pairs_table": [P, P, P, I, I, P],
    "mm_attention_sink_generic": [P, P, P, P, I, P, P, P, I, I, I, I, I, I, I, I, F, I, P, P, I, F, I, I, I, P],
    "mm_mingru_walk": [P, P, I, P, P, P, P, P, I, I, P],
    "mm_mingru_chunked": [P, P, I, P, P, P, P, P, P, P, P, I, I, I, P],
    "mm_bias_act": [P, P, I, P, I, I, I, I, P],
    "mm_causal_conv_walk": [P, I, I, P, I, P, c_longlong, P, P, P, I, I, P],
    "mm_linear_state_prep": [P, I, I, I, I, I, I, I, I, I, P, I, I, F, F, F, P, I, I, I, I, P, P, P, P, P],
    "mm_causal_conv_tokens": [P, I, I, P, I, P, c_longlong, P, I, P, P, P, P, I, I, I, P],
    "mm_moe_router": [P, I, I, P, I, I, I, I, I, I, P, P, P],
    "mm_angle_table": [P, P, P, I, I, P],
    "mm_linear_state_walk": [P, P, P, I, I, I, P, P, P, P, P, c_longlong, P, P, P, I, I, I, I, I, P],
    "mm_linear_state_chunked": [P, P, P, I, I, I, P, P, P, P, c_longlong, P, P, P, P, I, I, I, I, I, I, P, P, P],
    "mm_gated_group_norm": [P, I, I, P, I, I, P, I, P, I, I, I, I, F, I, I, P],
    "mm_normed_mean2": [P, P, P, P, P, I, I, I, F, F, P],
    "mm_moe_route": [P, I, I, I, I, I, I, P, P, P],
    "mm_moe_sort": [P, I, I, P, P, I, I, P, P, P, P, P],
    "mm_moe_gemm": [P, I, I, P, I, P, I, I, P, P, I, I, I, I, I, I, I, I, P],
    "mm_moe_combine": [P, I, P, P, P, I, I, I, I, P],
    "mm_stream_copies": [P, P, I, I, I, P],
    "mm_hc_read": [P, P, P, P, I, F, P, I, I, I, I, P],
    "mm_hc_write": [P, P, I, P, P, P, P, P, I, F, P, I, I, I, I, P],
    "mm_rope_half_table": [P, P, P, P, I, I, P],
    "mm_qkv_split_post": [P, I, I, I, I, P, P, P, I, P, I, I, I, I, I, I, I, P],
    "mm_latent_prep": [P, I, I, I, P, I, F, P, I, P, P, P, I, P, I, I, I, I, I, I, P],
    "mm_head_matmul": [P, c_longlong, I, P, P, c_longlong, I, I, I, I, I, I, P],
    "mm_head_finish": [P, I, I, F, I, F, F, P, I, P, I, I, I, I, I, P],
    "mm_moe_router_scored": [P, I, I, P, I, I, I, I, I, I, I, P, P, P],
    "mm_moe_gemm_act": [P, I, I, P, I, P, I, I, P, P, I, I, I, I, I, I, I, I, I, F, P, P],
    "mm_gemm_tcgen05_grouped_act": [P, P, P, I, I, I, I, I, I, I, P, P, I, I, F, P, P],
    "mm_moe_gather_scaled": [P, I, P, P, P, P, I, I, P],
    "mm_talking_prep": [P, I, I, I, I, P, P, F, P, I, I, P, P, P, I, P, I, I, I, I, I, I, P],
    "mm_attention_talking": [P, P, P, P, I, P, P, I, P, P, P, I, I, I, I, I, I, I, I, F, P, P, P],
    "mm_forget_gate_prep": [P, I, I, I, I, I, I, P, P, P],
    "mm_forget_gate_walk": [P, P, P, I, I, I, P, P, c_longlong, P, P, P, I, I, I, I, P],
    "mm_forget_gate_chunked": [P, P, P, I, I, I, P, P, c_longlong, P, P, P, P, I, I, I, I, I, P, P, P],
    "mm_post_norm": [P, P, P, I, P, P, I, I, I, F, F, F, F, P],
    "mm_glu_rows": [P, I, c_longlong, P, I, I, I, I, F, P, P],
    "mm_cast_rows": [P, P, I, c_longlong, P],
    "mm_scaled_sum2": [P, P, P, I, c_longlong, F, F, P],
    "mm_gemm_tcgen05_grouped": [P, P, P, I, I, I, I, I, I, I, P, P, I, P, P],
}


def load(verbose: bool = True) -> ctypes.CDLL:
    global _lib
    if _lib is not None:          # the usual case, without the lock: every launch comes through here
        return _lib
    with _lock:
        if _lib is not None:
            return _lib
        path = library_path(build_if_needed=True, verbose=verbose)
        lib = ctypes.CDLL(path)
        lib.mm_last_error.restype = ctypes.c_char_p
        lib.mm_last_error.argtypes = []
        lib.mm_set_pdl.argtypes = [c_int]
        lib.mm_set_pdl.restype = None
        lib.mm_get_pdl.argtypes = []
        lib.mm_get_pdl.restype = c_int
        lib.mm_set_gemv_blocks.argtypes = [c_int]
        lib.mm_set_gemv_blocks.restype = c_int
        lib.mm_launch_count.argtypes = []
        lib.mm_launch_count.restype = c_longlong
        lib.mm_uniform_from.restype = c_float
        lib.mm_uniform_from.argtypes = [c_ulonglong, c_ulonglong]
        for name, args in _PROTOTYPES.items():
            fn = getattr(lib, name, None)
            if fn is None:
                continue  # optional kernels are declared by the module that binds them
            fn.restype = c_int
            fn.argtypes = args
        _lib = lib
        return lib


def declare(name: str, argtypes, restype=c_int):
    """Declare the prototype of an entry point that is not in the core table."""
    lib = load()
    fn = getattr(lib, name)
    fn.argtypes = argtypes
    fn.restype = restype
    return fn


def launch_count() -> int:
    """Kernels of this library launched (or recorded into a graph under capture) so far."""
    return int(load().mm_launch_count())


def check(code: int, what: str) -> None:
    if code != 0:
        msg = load().mm_last_error().decode("utf-8", "replace")
        raise KernelError(f"{what} failed (code {code}): {msg}")
