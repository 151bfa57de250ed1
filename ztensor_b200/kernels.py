"""Python bindings of the C-ABI launchers, one function per kernel.

Same shape as the reference's per-kernel Go wrappers
(internal/cuda/kernels/gemm_q4_purego.go:14, gemm_q8_purego.go,
ternary_gemv_purego.go:19): raw device pointers and ints in, an error out.
Arguments are torch CUDA tensors only so that `.data_ptr()` yields a device
pointer; torch does none of the arithmetic.
"""
from __future__ import annotations

import ctypes as C

import torch

from . import _lib

X_F32, Y_F32, X_KB, Y_NB, NO_PDL, PLAIN, FP32_DECODE = 1, 2, 4, 8, 16, 32, 64
FMT_Q4_0, FMT_IQ4NL, FMT_W4G, FMT_Q8_0, FMT_TERNARY = 0, 1, 2, 3, 4


def _ptr(t):
    if t is None:
        return None
    if not t.is_cuda:
        raise ValueError("kernel arguments must be CUDA tensors (device pointers)")
    return t.data_ptr()


def _stream(stream):
    if stream is None:
        return torch.cuda.current_stream().cuda_stream
    return stream.cuda_stream if hasattr(stream, "cuda_stream") else int(stream)


def q4_gpu_data_offset(total_blocks: int) -> int:
    """tensor.Q4GPUDataOffset (tensor/quantized.go:196-199)."""
    return (total_blocks * 2 + 15) & ~15


def gemm_q4_f32(a_q4, b, c, m, k, n, data_offset, stream=None):
    """kernels.GemmQ4F32 (gemm_q4_purego.go:14-29)."""
    _lib.check(_lib.lib().gemm_q4_f32(_ptr(a_q4), _ptr(b), _ptr(c), m, k, n, data_offset, _stream(stream)), "gemm_q4_f32")


def gemm_q8_f32(a_q8, b, c, m, k, n, stream=None):
    """kernels.GemmQ8F32 (gemm_q8_purego.go)."""
    _lib.check(_lib.lib().gemm_q8_f32(_ptr(a_q8), _ptr(b), _ptr(c), m, k, n, _stream(stream)), "gemm_q8_f32")


def ternary_gemv_f32(w, x, y, m, k, stream=None):
    """kernels.TernaryGemvF32 (ternary_gemv_purego.go:19-37)."""
    _lib.check(_lib.lib().ternary_gemv_f32(_ptr(w), _ptr(x), _ptr(y), m, k, _stream(stream)), "ternary_gemv_f32")


def gemv_q4_0(w_sep, data_offset, x, y, n, k, batch, flags=0, stream=None):
    _lib.check(_lib.lib().ztq_gemv_q4_0(_ptr(w_sep), data_offset, _ptr(x), _ptr(y), n, k, batch, flags, _stream(stream)), "ztq_gemv_q4_0")


def gemv_iq4nl(w_sep, data_offset, x, y, n, k, batch, flags=0, stream=None):
    _lib.check(_lib.lib().ztq_gemv_iq4nl(_ptr(w_sep), data_offset, _ptr(x), _ptr(y), n, k, batch, flags, _stream(stream)), "ztq_gemv_iq4nl")


def gemv_q8_0(w, x, y, n, k, batch, flags=0, stream=None):
    _lib.check(_lib.lib().ztq_gemv_q8_0(_ptr(w), _ptr(x), _ptr(y), n, k, batch, flags, _stream(stream)), "ztq_gemv_q8_0")


def gemv_w4g(qdata, meta, x, y, n, k, group, batch, flags=0, stream=None):
    _lib.check(_lib.lib().ztq_gemv_w4g(_ptr(qdata), _ptr(meta), _ptr(x), _ptr(y), n, k, group, batch, flags, _stream(stream)), "ztq_gemv_w4g")


def gemv_ternary(w_rows, row_scale, x, y, n, k, batch, flags=0, stream=None):
    _lib.check(_lib.lib().ztq_gemv_ternary(_ptr(w_rows), _ptr(row_scale), _ptr(x), _ptr(y), n, k, batch, flags, _stream(stream)), "ztq_gemv_ternary")


def repack_blocks18(aos, sep, n_blocks, stream=None):
    _lib.check(_lib.lib().ztq_repack_blocks18(_ptr(aos), _ptr(sep), n_blocks, _stream(stream)), "ztq_repack_blocks18")


def pack_w4g_meta(scales, zeros, meta, n_groups, stream=None):
    _lib.check(_lib.lib().ztq_pack_w4g_meta(_ptr(scales), _ptr(zeros), _ptr(meta), n_groups, _stream(stream)), "ztq_pack_w4g_meta")


def repack_ternary_rows(flat, rows, m, k, stream=None):
    _lib.check(_lib.lib().ztq_repack_ternary_rows(_ptr(flat), _ptr(rows), m, k, _stream(stream)), "ztq_repack_ternary_rows")


def quantize_q4_0(src, sep, n, stream=None):
    _lib.check(_lib.lib().ztq_quantize_q4_0(_ptr(src), _ptr(sep), n, _stream(stream)), "ztq_quantize_q4_0")


def quantize_q8_0(src, blocks, n, stream=None):
    _lib.check(_lib.lib().ztq_quantize_q8_0(_ptr(src), _ptr(blocks), n, _stream(stream)), "ztq_quantize_q8_0")


def quantize_w4g(src, qdata, meta, n, group=128, awq=False, stream=None):
    _lib.check(_lib.lib().ztq_quantize_w4g(_ptr(src), _ptr(qdata), _ptr(meta), n, group, 1 if awq else 0, _stream(stream)), "ztq_quantize_w4g")


def dequantize(fmt, w, meta, dst, n, aux, stream=None):
    _lib.check(_lib.lib().ztq_dequantize(fmt, _ptr(w), _ptr(meta), _ptr(dst), n, aux, _stream(stream)), "ztq_dequantize")


def probe_launch(grid, threads, smem_bytes, flags=0, stream=None):
    """An empty kernel with a GEMV's launch shape (the floor of a dependent launch)."""
    _lib.check(_lib.lib().ztq_probe_launch(grid, threads, smem_bytes, flags, _stream(stream)), "ztq_probe_launch")


def check_sm100() -> bool:
    return _lib.lib().ztq_check_sm100() == 1


def device_error() -> int:
    return _lib.lib().ztq_device_error()


def gemv_w4g_allreduce(qdata, meta, x, y, n, k, group, batch, ar, flags=0, stream=None):
    """Row-parallel shard: GEMV + all-reduce of y in one kernel (ar: collective.FusedAllReduce)."""
    _lib.check(_lib.lib().ztq_gemv_w4g_allreduce(_ptr(qdata), _ptr(meta), _ptr(x), _ptr(y), n, k, group, batch, flags,
                                                 ar.ptr(), _stream(stream)), "ztq_gemv_w4g_allreduce")


def splitk_workspace_bytes(n, splits) -> int:
    return int(_lib.lib().ztq_splitk_workspace_bytes(n, splits))


def gemv_w4g_splitk(qdata, meta, x, y, n, k, group, splits, workspace, flags=0, stream=None):
    _lib.check(_lib.lib().ztq_gemv_w4g_splitk(_ptr(qdata), _ptr(meta), _ptr(x), _ptr(y), n, k, group, splits, _ptr(workspace),
                                              workspace.numel() * workspace.element_size(), flags, _stream(stream)),
               "ztq_gemv_w4g_splitk")


def gemv_q4_0_splitk(w_sep, data_offset, x, y, n, k, splits, workspace, flags=0, stream=None):
    _lib.check(_lib.lib().ztq_gemv_q4_0_splitk(_ptr(w_sep), data_offset, _ptr(x), _ptr(y), n, k, splits, _ptr(workspace),
                                               workspace.numel() * workspace.element_size(), flags, _stream(stream)),
               "ztq_gemv_q4_0_splitk")


STATIC_SCRATCH_BYTES = 1 << 20


def gemv_w4g_splitk_static(qdata, meta, x, y, n, k, group, splits, flags=0, stream=None):
    """Split-K GEMV whose partial sums live in the library's built-in scratch array (no workspace argument,
    no allocation; n * splits * 4 <= STATIC_SCRATCH_BYTES; calls must not overlap on the GPU)."""
    _lib.check(_lib.lib().ztq_gemv_w4g_splitk_static(_ptr(qdata), _ptr(meta), _ptr(x), _ptr(y), n, k, group, splits, flags,
                                                     _stream(stream)), "ztq_gemv_w4g_splitk_static")


def gemm_w4g_tc_workspace_bytes(n, k, batch) -> int:
    return int(_lib.lib().ztq_gemm_w4g_tc_workspace_bytes(n, k, batch))


def gemm_w4g_tc(qdata, meta, x, y, n, k, group, batch, workspace, flags=0, stream=None):
    """W4A16 skinny GEMM on tcgen05 / TMEM (the batch >= 16 path); workspace: uint8 CUDA tensor."""
    _lib.check(_lib.lib().ztq_gemm_w4g_tc(_ptr(qdata), _ptr(meta), _ptr(x), _ptr(y), n, k, group, batch, _ptr(workspace),
                                          workspace.numel() * workspace.element_size(), flags, _stream(stream)),
               "ztq_gemm_w4g_tc")


def gemm_w4g_tc_allreduce(qdata, meta, x, y, n, k, group, batch, workspace, ar, flags=0, stream=None):
    """Row-parallel shard with 3 or more activation rows: the tensor-core GEMM with the all-reduce of y in its epilogue
    (ar: collective.FusedAllReduce sized for min(batch, 16) * n cells)."""
    _lib.check(_lib.lib().ztq_gemm_w4g_tc_allreduce(_ptr(qdata), _ptr(meta), _ptr(x), _ptr(y), n, k, group, batch, _ptr(workspace),
                                                    workspace.numel() * workspace.element_size(), flags, ar.ptr(), _stream(stream)),
               "ztq_gemm_w4g_tc_allreduce")


def gemm_q4_0_tc_workspace_bytes(n, k, batch) -> int:
    return int(_lib.lib().ztq_gemm_q4_0_tc_workspace_bytes(n, k, batch))


def gemm_q4_0_tc(w_sep, data_offset, x, y, n, k, batch, workspace, flags=0, stream=None):
    """Q4_0 skinny GEMM on tcgen05 / TMEM (three or more activation rows); workspace: uint8 CUDA tensor."""
    _lib.check(_lib.lib().ztq_gemm_q4_0_tc(_ptr(w_sep), data_offset, _ptr(x), _ptr(y), n, k, batch, _ptr(workspace),
                                           workspace.numel() * workspace.element_size(), flags, _stream(stream)),
               "ztq_gemm_q4_0_tc")


def gemm_q8_0_tc_workspace_bytes(n, k, batch) -> int:
    return int(_lib.lib().ztq_gemm_q8_0_tc_workspace_bytes(n, k, batch))


def gemm_q8_0_tc(blocks36, x, y, n, k, batch, workspace, flags=0, stream=None):
    """Q8_0 skinny GEMM on tcgen05 / TMEM (three or more activation rows) on the raw 36-byte blocks."""
    _lib.check(_lib.lib().ztq_gemm_q8_0_tc(_ptr(blocks36), _ptr(x), _ptr(y), n, k, batch, _ptr(workspace),
                                           workspace.numel() * workspace.element_size(), flags, _stream(stream)),
               "ztq_gemm_q8_0_tc")


class ZtqGemvFusion(C.Structure):
    _fields_ = [("residual", C.c_void_p), ("norm_weight", C.c_void_p), ("sum_out", C.c_void_p),
                ("eps_bits", C.c_uint), ("swiglu", C.c_int)]


def gemv_w4g_fused(qdata, meta, x, y, n, k, group=128, flags=0, norm_weight=None, eps=1e-5, residual=None, sum_out=None,
                   swiglu=False, stream=None):
    """Batch-1 W4A16 GEMV with RMSNorm folded into the activation load and / or SwiGLU into the output store."""
    import struct
    fz = ZtqGemvFusion(_ptr(residual), _ptr(norm_weight), _ptr(sum_out),
                       struct.unpack("<I", struct.pack("<f", float(eps)))[0], 1 if swiglu else 0)
    _lib.check(_lib.lib().ztq_gemv_w4g_fused(_ptr(qdata), _ptr(meta), _ptr(x), _ptr(y), n, k, group, flags, C.byref(fz),
                                             _stream(stream)), "ztq_gemv_w4g_fused")


def interleave_rows(a, b, out, rows, row_bytes, stream=None):
    _lib.check(_lib.lib().ztq_interleave_rows(_ptr(a), _ptr(b), _ptr(out), rows, row_bytes, _stream(stream)),
               "ztq_interleave_rows")


def gemv_q4k(w_sep, data_offset, x, y, n, k, batch=1, flags=0, stream=None):
    """Q4_K GEMV on the separated layout of repack_blocks144 (data_offset = 16 * number of super-blocks)."""
    _lib.check(_lib.lib().ztq_gemv_q4k(_ptr(w_sep), data_offset, _ptr(x), _ptr(y), n, k, batch, flags, _stream(stream)),
               "ztq_gemv_q4k")


def repack_blocks144(aos, sep, nblocks, stream=None):
    _lib.check(_lib.lib().ztq_repack_blocks144(_ptr(aos), _ptr(sep), nblocks, _stream(stream)), "ztq_repack_blocks144")


def gemv_q5k(w_sep, data_offset, x, y, n, k, batch=1, flags=0, stream=None):
    """Q5_K GEMV on the separated layout of repack_blocks176 (data_offset = 48 * number of super-blocks)."""
    _lib.check(_lib.lib().ztq_gemv_q5k(_ptr(w_sep), data_offset, _ptr(x), _ptr(y), n, k, batch, flags, _stream(stream)),
               "ztq_gemv_q5k")


def repack_blocks176(aos, sep, nblocks, stream=None):
    _lib.check(_lib.lib().ztq_repack_blocks176(_ptr(aos), _ptr(sep), nblocks, _stream(stream)), "ztq_repack_blocks176")


def gemv_q6k(w_sep, data_offset, x, y, n, k, batch=1, flags=0, stream=None):
    """Q6_K GEMV on the separated layout of repack_blocks210 (data_offset = 96 * number of super-blocks)."""
    _lib.check(_lib.lib().ztq_gemv_q6k(_ptr(w_sep), data_offset, _ptr(x), _ptr(y), n, k, batch, flags, _stream(stream)),
               "ztq_gemv_q6k")


def repack_blocks210(aos, sep, nblocks, stream=None):
    _lib.check(_lib.lib().ztq_repack_blocks210(_ptr(aos), _ptr(sep), nblocks, _stream(stream)), "ztq_repack_blocks210")


PLAN_FMT = {"q4_0": 0, "iq4nl": 1, "w4g": 2, "q8_0": 3, "ternary": 4, "q4_k": 5, "q5_k": 6, "q6_k": 7, "w4g_tc": 8}


def describe_plan(fmt: str, n: int, k: int, batch: int = 1, group: int = 128, sms: int = 148) -> dict:
    """The launch plan of the first launch of such a call on a device of `sms` SMs (ztq_describe_plan): host
    arithmetic only, so it also answers without a GPU."""
    out = (C.c_int * 12)()
    if _lib.lib().ztq_describe_plan(PLAN_FMT[fmt], n, k, group, batch, sms, out) != 0:
        raise ValueError(f"no plan for {fmt} {n}x{k} batch {batch}")
    v = list(out)
    if v[0] == 3:
        return dict(kernel="tensor", columns=v[1], k_slices=v[2], groups_per_slice=v[3], row_tiles=v[4], items=v[5],
                    grid=v[6], items_per_cta=v[7])
    return dict(kernel=("plain", "stream", "pair")[v[0]], rows_per_launch=v[1], rt=v[2], rows_per_stage=v[3], stages=v[4],
                overlay_stages=v[5], rows_per_pass=v[6], grid=v[7], tiles_per_cta=v[8], passes_per_cta=v[9],
                warps_per_team=v[10], teams=v[11])
