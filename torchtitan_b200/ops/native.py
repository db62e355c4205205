"""Loader for the in-tree native library (``torchtitan_b200/_lib/libtt_b200.so``).

The library is plain C ABI (built by ``__graft_entry__.build()`` with nvcc for sm_100a) and is
called through ctypes with raw device pointers and the current CUDA stream. On a machine with
a GPU, using any CUDA op of this framework without the library raises immediately: there is no
silent fallback to library kernels.
"""

from __future__ import annotations

import ctypes
import os
from ctypes import c_float, c_int, c_longlong, c_void_p

_LIB = None
_LIB_PATH = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "_lib", "libtt_b200.so")


def lib_path() -> str:
    return _LIB_PATH


def available() -> bool:
    return os.path.exists(_LIB_PATH)


def _sig(fn, argtypes, restype=c_int):
    fn.argtypes = argtypes
    fn.restype = restype


def lib():
    global _LIB
    if _LIB is not None:
        return _LIB
    if not os.path.exists(_LIB_PATH):
        raise RuntimeError(
            f"native library {_LIB_PATH} is missing: run `python -c 'import __graft_entry__ as g; g.build()'` "
            "from the repository root (needs nvcc)"
        )
    L = ctypes.CDLL(_LIB_PATH)
    P, I, LL, F = c_void_p, c_int, c_longlong, c_float
    _sig(L.tt_gemm_bf16, [P, P, P, I, I, I, I, LL, I, LL, LL, I, I, P, I, I, P])
    _sig(L.tt_gemm_error, [])
    _sig(L.tt_gemm_set_pair, [I])
    _sig(L.tt_rmsnorm_fwd, [P, P, P, P, LL, I, F, I, P])
    _sig(L.tt_rmsnorm_bwd_blocks, [LL, I])
    _sig(L.tt_rmsnorm_bwd, [P, P, P, P, P, P, P, LL, I, I, P])
    _sig(L.tt_rope, [P, P, P, P, I, I, I, I, I, I, I, I, P])
    _sig(L.tt_swiglu_fwd, [P, P, P, LL, I, P])
    _sig(L.tt_swiglu_bwd, [P, P, P, P, P, LL, I, P])
    _sig(L.tt_ce_fwd, [P, P, P, P, P, P, LL, I, LL, I, I, P])
    _sig(L.tt_ce_bwd, [P, P, P, P, P, P, LL, I, LL, I, I, I, P])
    _sig(L.tt_adamw, [P, P, P, P, P, LL, F, F, F, F, F, I, I, P, P])
    _sig(L.tt_sumsq, [P, P, P, LL, I, I, P])
    _sig(L.tt_attn_supported, [I, I, I, I, I])
    _sig(L.tt_attn_fwd, [P, P, P, P, P, I, I, I, I, I, I, I, F, P])
    _sig(L.tt_attn_bwd, [P, P, P, P, P, P, P, P, P, P, I, I, I, I, I, I, I, F, P])
    _sig(L.tt_attn_error, [])
    _sig(L.tt_attn_fwd_range, [P, P, P, P, P, P, I, I, I, I, I, I, I, F, P])
    _sig(L.tt_attn_bwd_range, [P, P, P, P, P, P, P, P, P, P, P, P, I, I, I, I, I, I, I, F, P])
    _sig(L.tt_grouped_gemm, [P, P, P, P, LL, I, I, I, I, LL, LL, P])
    _sig(L.tt_grouped_gemm_wgrad, [P, P, P, P, LL, I, I, I, LL, LL, I, P])
    _sig(L.tt_grouped_gemm_error, [])
    if hasattr(L, "tt_grouped_gemm_set_pair"):
        _sig(L.tt_grouped_gemm_set_pair, [I], None)
    _sig(L.tt_kv_write, [P, P, P, P, P, LL, I, I, P])
    _sig(L.tt_paged_decode, [P, P, P, P, P, P, F, I, I, I, I, I, I, P])
    _sig(L.tt_sample, [P, P, P, P, I, I, LL, F, I, P])
    _sig(L.tt_moe_route_fwd, [P, P, P, P, P, I, I, I, I, I, F, P])
    _sig(L.tt_moe_route_bwd, [P, P, P, P, I, I, I, I, I, F, P])
    _sig(L.tt_moe_sort, [P, P, P, P, LL, I, P])
    _sig(L.tt_moe_gather, [P, P, P, P, LL, I, P])
    _sig(L.tt_moe_combine, [P, P, P, P, LL, I, I, P])
    _sig(L.tt_moe_rowdot, [P, P, P, P, LL, I, I, P])
    _sig(L.tt_gemm_fp8, [P, P, P, I, I, I, LL, LL, LL, I, I, I, P, P, I, P])
    _sig(L.tt_gemm_allgather_a, [P, P, I, I, I, P, P, I, I, I, I, LL, LL, I, P, I, I, P])
    if hasattr(L, "tt_ep_push"):
        _sig(L.tt_ep_publish_counts, [P, P, P, I, I, I, I, P])
        _sig(L.tt_ep_build_maps, [P, P, I, I, I, I, I, I, I, P, P, P, P, P, P, P, I, P])
        if hasattr(L, "tt_ep_build_maps_opt"):
            _sig(L.tt_ep_build_maps_opt, [P, P, I, I, I, I, I, I, I, P, P, P, P, P, P, P, I, I, P])
        _sig(L.tt_ep_push, [P, P, I, P, P, P, P, I, I, I, P])
        _sig(L.tt_ep_wait, [P, I, P])
        _sig(L.tt_ep_error, [P])
        L.tt_ep_set_wait_ns.argtypes = [ctypes.c_ulonglong]
        L.tt_ep_set_wait_ns.restype = None
        _sig(L.tt_ep_push_ctas, [])
    if hasattr(L, "tt_gemm_bf16_res"):
        _sig(L.tt_gemm_bf16_res, [P, P, P, P, I, I, I, I, LL, I, LL, LL, LL, P])
    if hasattr(L, "tt_grouped_gemm_mxfp8"):
        _sig(L.tt_grouped_gemm_mxfp8, [P, P, P, P, P, P, I, I, I, I, I, LL, LL, LL, LL, I, I, LL, I, P])
    if hasattr(L, "tt_gemm_mxfp8"):
        _sig(L.tt_gemm_mxfp8, [P, P, P, P, P, I, I, I, LL, LL, LL, I, P])
        _sig(L.tt_mx_swizzle_scales, [P, I, I, I, P, P])
        if hasattr(L, "tt_gemm_mx_set_pair"):
            _sig(L.tt_gemm_mx_set_pair, [I], None)
        L.tt_mx_scales_bytes.argtypes = [I, I, I]
        L.tt_mx_scales_bytes.restype = LL
    if hasattr(L, "tt_mxfp8_quant_rows"):
        _sig(L.tt_mxfp8_quant_rows, [P, LL, I, I, P, P, P])
        _sig(L.tt_mxfp8_quant_cols, [P, LL, I, I, P, P, P])
    if hasattr(L, "tt_mxfp8_quant_rows_swz"):
        _sig(L.tt_mxfp8_quant_rows_swz, [P, LL, I, I, P, P, P])
        _sig(L.tt_mxfp8_quant_cols_swz, [P, LL, I, I, P, P, P])
    if hasattr(L, "tt_sample_top_p"):
        _sig(L.tt_sample_top_p, [P, P, P, P, I, I, LL, F, F, I, P])
    if hasattr(L, "tt_fp8_quant_rows"):
        _sig(L.tt_fp8_quant_rows, [P, LL, I, I, P, P, I, I, P])
        _sig(L.tt_fp8_quant_cols, [P, LL, I, I, P, P, I, I, P])
        _sig(L.tt_fp8_quant_tensor, [P, LL, I, I, P, P, I, I, P])
    if hasattr(L, "tt_attn_fwd_sinks"):
        _sig(L.tt_attn_fwd_sinks, [P, P, P, P, P, P, P, I, I, I, I, I, I, I, F, P])
    if hasattr(L, "tt_attn_fwd_dims"):
        _sig(L.tt_attn_fwd_dims, [P, P, P, P, P, P, P, I, I, I, I, I, I, I, I, F, P])
        _sig(L.tt_attn_supported_dims, [I, I, I, I, I, I])
    if hasattr(L, "tt_attn_bwd_dims"):
        _sig(L.tt_attn_bwd_dims, [P, P, P, P, P, P, P, P, P, P, P, P, I, I, I, I, I, I, I, I, F, P])
    if hasattr(L, "tt_attn_bwd_fused"):
        _sig(L.tt_attn_bwd_fused, [P, P, P, P, P, P, P, P, P, P, P, P, P, I, I, I, I, I, I, I, F, P])
        _sig(L.tt_attn_set_dq_mode, [I], None)
        if os.environ.get("TT_ATTN_BWD_MODE"):      # measurement aid: see tt_attn_set_dq_mode in csrc/attention.cu
            L.tt_attn_set_dq_mode(int(os.environ["TT_ATTN_BWD_MODE"]))
    if hasattr(L, "tt_gemm_rs_set_interleave"):
        L.tt_gemm_rs_set_interleave.argtypes = [I]
        L.tt_gemm_rs_set_interleave.restype = None
    if hasattr(L, "tt_gemm_reduce_scatter"):
        _sig(L.tt_gemm_reduce_scatter, [P, P, P, P, P, I, I, I, I, I, LL, I, LL, I, I, P])
    if hasattr(L, "tt_push_cast"):
        _sig(L.tt_push_cast, [P, I, P, I, P])
        _sig(L.tt_wait_flags, [P, I, I, P])
    for name, sig in _OPTIONAL.items():
        if hasattr(L, name):
            _sig(getattr(L, name), sig)
    _LIB = L
    return L


# symbols that newer builds of the library add (bound when present)
_OPTIONAL: dict = {}


def register_optional(name: str, argtypes) -> None:
    _OPTIONAL[name] = argtypes
    if _LIB is not None and hasattr(_LIB, name):
        _sig(getattr(_LIB, name), argtypes)


def has(name: str) -> bool:
    """True when the built library exports ``name`` (optional kernels of newer builds)."""
    return available() and hasattr(lib(), name)


CALLS = 0  # number of native launch calls made by this process (bench reporting)


def check(rc: int, what: str) -> None:
    global CALLS
    CALLS += 1
    if rc != 0:
        raise RuntimeError(f"{what} failed with code {rc}")


def kernel_errors() -> dict:
    """Error words set by kernels whose bounded waits expired (reading clears them)."""
    L = lib()
    out = {"gemm": L.tt_gemm_error(), "attention": L.tt_attn_error(), "grouped_gemm": L.tt_grouped_gemm_error()}
    if hasattr(L, "tt_gemm_mx_error"):
        out["gemm_mx"] = L.tt_gemm_mx_error()
    if hasattr(L, "tt_ep_error"):
        e4 = (ctypes.c_int * 4)()
        if L.tt_ep_error(e4) == 1:
            out["ep"] = tuple(e4)
    if hasattr(L, "tt_comm_error"):                      # peer-memory collectives of the FSDP / weight-sync transports
        c4 = (ctypes.c_int * 4)()
        if L.tt_comm_error(c4) != 0:
            out["comm"] = tuple(c4)                          # (code, peer, expected version, version seen)
    return {k: v for k, v in out.items() if v}
