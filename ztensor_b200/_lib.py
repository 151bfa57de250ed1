"""Loader of libztq_sm100a.so, the C-ABI kernel library (include/ztq.h).

There is no fallback: if the library has not been built, or a call returns a
CUDA error, an exception is raised.  The error text follows the reference's
binding layer (internal/cuda/kernels/elementwise_purego.go:11-16)."""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libztq_sm100a.so")

_vp, _i, _ll = C.c_void_p, C.c_int, C.c_longlong

# name -> argument types; every entry point returns an int (cudaError_t or a probe value)
SIGNATURES = {
    "gemm_q4_f32": [_vp, _vp, _vp, _i, _i, _i, _i, _vp],
    "gemm_q8_f32": [_vp, _vp, _vp, _i, _i, _i, _vp],
    "ternary_gemv_f32": [_vp, _vp, _vp, _i, _i, _vp],
    "ztq_gemv_q4_0": [_vp, _i, _vp, _vp, _i, _i, _i, _i, _vp],
    "ztq_gemv_iq4nl": [_vp, _i, _vp, _vp, _i, _i, _i, _i, _vp],
    "ztq_gemv_q8_0": [_vp, _vp, _vp, _i, _i, _i, _i, _vp],
    "ztq_gemv_w4g": [_vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _vp],
    "ztq_gemm_w4g_tc_workspace_bytes": [_i, _i, _i],
    "ztq_gemm_w4g_tc": [_vp, _vp, _vp, _vp, _i, _i, _i, _i, _vp, C.c_size_t, _i, _vp],
    "ztq_gemm_w4g_tc_allreduce": [_vp, _vp, _vp, _vp, _i, _i, _i, _i, _vp, C.c_size_t, _i, _vp, _vp],
    "ztq_gemm_q4_0_tc_workspace_bytes": [_i, _i, _i],
    "ztq_gemm_q4_0_tc": [_vp, _i, _vp, _vp, _i, _i, _i, _vp, C.c_size_t, _i, _vp],
    "ztq_gemm_q8_0_tc_workspace_bytes": [_i, _i, _i],
    "ztq_gemm_q8_0_tc": [_vp, _vp, _vp, _i, _i, _i, _vp, C.c_size_t, _i, _vp],
    "ztq_gemv_q4k": [_vp, _ll, _vp, _vp, _i, _i, _i, _i, _vp],
    "ztq_repack_blocks144": [_vp, _vp, _ll, _vp],
    "ztq_gemv_q5k": [_vp, _ll, _vp, _vp, _i, _i, _i, _i, _vp],
    "ztq_repack_blocks176": [_vp, _vp, _ll, _vp],
    "ztq_gemv_q6k": [_vp, _ll, _vp, _vp, _i, _i, _i, _i, _vp],
    "ztq_repack_blocks210": [_vp, _vp, _ll, _vp],
    "ztq_gemv_w4g_fused": [_vp, _vp, _vp, _vp, _i, _i, _i, _i, _vp, _vp],
    "ztq_interleave_rows": [_vp, _vp, _vp, _ll, _i, _vp],
    "ztq_gemv_ternary": [_vp, _vp, _vp, _vp, _i, _i, _i, _i, _vp],
    "ztq_gemv_w4g_allreduce": [_vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _vp, _vp],
    "ztq_gemv_q4_0_allreduce": [_vp, _i, _vp, _vp, _i, _i, _i, _i, _vp, _vp],
    "ztq_splitk_workspace_bytes": [_i, _i],
    "ztq_gemv_w4g_splitk": [_vp, _vp, _vp, _vp, _i, _i, _i, _i, _vp, C.c_size_t, _i, _vp],
    "ztq_gemv_q4_0_splitk": [_vp, _i, _vp, _vp, _i, _i, _i, _vp, C.c_size_t, _i, _vp],
    "ztq_gemv_w4g_splitk_static": [_vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _vp],
    "ztq_symm_alloc": [C.POINTER(C.c_void_p), C.c_size_t],
    "ztq_symm_free": [_vp],
    "ztq_symm_zero": [_vp, C.c_size_t],
    "ztq_ipc_export": [_vp, _vp],
    "ztq_ipc_open": [_vp, C.POINTER(C.c_void_p)],
    "ztq_ipc_close": [_vp],
    "ztq_repack_blocks18": [_vp, _vp, _ll, _vp],
    "ztq_pack_w4g_meta": [_vp, _vp, _vp, _ll, _vp],
    "ztq_repack_ternary_rows": [_vp, _vp, _i, _i, _vp],
    "ztq_quantize_q4_0": [_vp, _vp, _ll, _vp],
    "ztq_quantize_q8_0": [_vp, _vp, _ll, _vp],
    "ztq_quantize_w4g": [_vp, _vp, _vp, _ll, _i, _i, _vp],
    "ztq_dequantize": [_i, _vp, _vp, _vp, _ll, _i, _vp],
    "ztq_matmul_wkn_f32": [_vp, _vp, _vp, _i, _i, _i, _i, _vp],
    "ztq_describe_plan": [_i, _i, _i, _i, _i, _i, C.POINTER(C.c_int)],
    "ztq_probe_launch": [_i, _i, _i, _i, _vp],
    "ztq_check_sm100": [],
    "ztq_abi_version": [],
    "ztq_device_error": [],
}

_lib = None


class KernelLibraryMissing(RuntimeError):
    pass


def lib() -> C.CDLL:
    """dlopen the kernel library once; raise if it is not there."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise KernelLibraryMissing(
                f"{LIB_PATH} not found: build it with `make -C ztensor_b200/csrc` "
                "(or __graft_entry__.build()); there is no CPU fallback")
        handle = C.CDLL(LIB_PATH, mode=C.RTLD_GLOBAL)
        for name, args in SIGNATURES.items():
            fn = getattr(handle, name)        # AttributeError if a declared symbol is missing
            fn.argtypes = args
            fn.restype = C.c_size_t if name.endswith("_workspace_bytes") else C.c_int
        _lib = handle
    return _lib


def check(ret: int, name: str) -> None:
    if ret != 0:
        raise RuntimeError(f"{name} kernel failed (cuda error {ret})")
