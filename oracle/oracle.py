"""ctypes front end of the CPU oracle (libztq_oracle.so).

TEST INFRASTRUCTURE ONLY: imported by tests/, by the smoke check and by the
bench's CPU-baseline legs.  The GPU product path never imports this module.

The classes mirror the reference's CPU storages just far enough to replay its
engine dispatch (compute/cpu_engine.go:1124-1240, 2277-2434) on numpy arrays:
the arithmetic itself lives in ztq_oracle.c.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from dataclasses import dataclass

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libztq_oracle.so")


def build(force: bool = False) -> str:
    """Compile the C restatement with the recipe in oracle/Makefile."""
    src = os.path.join(_HERE, "ztq_oracle.c")
    if force or not os.path.exists(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE, "-B" if force else "-s", "libztq_oracle.so"])
    return _LIB_PATH


def _load():
    build()
    lib = C.CDLL(_LIB_PATH)
    vp, i64, i32, f32, u16 = C.c_void_p, C.c_int64, C.c_int, C.c_float, C.c_uint16
    sig = {
        "zo_f32_to_f16": (u16, [f32]),
        "zo_f16_to_f32": (f32, [u16]),
        "zo_xblas_f16_bits_to_f32": (f32, [u16]),
        "zo_f16_from_f32": (None, [vp, i64, vp]),
        "zo_f16_slice": (None, [vp, i64, vp]),
        "zo_q4_num_blocks": (i64, [i64]),
        "zo_quantize_q4": (None, [vp, i64, vp]),
        "zo_dequantize_q4": (None, [vp, i64, vp]),
        "zo_q4_gpu_data_offset": (i64, [i64]),
        "zo_q4_raw_bytes_gpu": (None, [vp, i64, vp]),
        "zo_quantize_q8": (None, [vp, i64, vp]),
        "zo_dequantize_q8": (None, [vp, i64, vp]),
        "zo_iq4nl_table": (None, [vp]),
        "zo_dequantize_iq4nl": (None, [vp, i64, vp]),
        "zo_ternary_pack": (None, [vp, i64, vp]),
        "zo_ternary_get": (C.c_int8, [vp, i64]),
        "zo_ternary_gemv": (None, [vp, vp, i32, i32, vp]),
        "zo_gptq4_data_bytes": (i64, [i64, i32]),
        "zo_awq_data_bytes": (i64, [i64, i32]),
        "zo_quantize_gptq4": (None, [vp, i64, i32, vp, vp, vp]),
        "zo_dequantize_gptq4": (None, [vp, vp, vp, i64, i32, vp]),
        "zo_quantize_awq": (None, [vp, i64, i32, vp, vp, vp]),
        "zo_dequantize_awq": (None, [vp, vp, vp, i64, i32, vp]),
        "zo_sgemm_simd": (None, [i32, i32, i32, vp, vp, vp]),
        "zo_gemm_q4_f32_fused": (None, [i32, i32, i32, vp, vp, vp]),
        "zo_gemm_f32_q4_nt": (None, [i32, i32, i32, vp, vp, vp, i32]),
        "zo_gemm_q8_f32": (None, [i32, i32, i32, vp, vp, vp]),
        "zo_gemm_f32_q8_nt": (None, [i32, i32, i32, vp, vp, vp, i32]),
        "zo_nt_threads": (i32, [i32, i32, i32]),
        "zo_num_cpu": (i32, []),
        "zo_quantize_q4k": (None, [vp, i64, vp]),
        "zo_dequantize_q4k": (None, [vp, i64, vp]),
        "zo_q4k_scales_mins": (None, [vp, vp, vp]),
        "zo_gemm_q4k_f32": (None, [i32, i32, i32, vp, vp, vp]),
        "zo_gemm_f32_q4k_nt": (None, [i32, i32, i32, vp, vp, vp, i32]),
        "zo_dequantize_q5k": (None, [vp, i64, vp]),
        "zo_make_q5k_blocks": (None, [vp, i64, vp]),
        "zo_gemm_f32_q5k_nt": (None, [i32, i32, i32, vp, vp, vp, i32]),
        "zo_dequantize_q6k": (None, [vp, i64, vp]),
        "zo_make_q6k_blocks": (None, [vp, i64, vp]),
        "zo_gemm_f32_q6k_nt": (None, [i32, i32, i32, vp, vp, vp, i32]),
        "zo_fused_add_rmsnorm": (None, [vp, vp, vp, vp, vp, C.c_float, i32]),
        "zo_fused_swiglu": (None, [vp, vp, vp, i32]),
    }
    for name, (res, args) in sig.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    return lib


LIB = _load()


def _p(a: np.ndarray):
    return a.ctypes.data_as(C.c_void_p)


def _f32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float32)


# --------------------------------------------------------------------------
# binary16
# --------------------------------------------------------------------------

def f32_to_f16_bits(a) -> np.ndarray:
    a = _f32(a).ravel()
    out = np.empty(a.size, np.uint16)
    LIB.zo_f16_from_f32(_p(a), a.size, _p(out))
    return out


def f16_bits_to_f32(bits) -> np.ndarray:
    bits = np.ascontiguousarray(bits, dtype=np.uint16).ravel()
    out = np.empty(bits.size, np.float32)
    LIB.zo_f16_slice(_p(bits), bits.size, _p(out))
    return out


# --------------------------------------------------------------------------
# storages (same names as tensor/*.go)
# --------------------------------------------------------------------------

@dataclass
class Q4Storage:
    """tensor/quantized.go:23-34; blocks = AoS bytes as RawBytes() returns them (:148-156)."""
    blocks: np.ndarray
    len: int

    def num_blocks(self) -> int:
        return (self.len + 31) // 32

    def raw_bytes(self) -> np.ndarray:
        return self.blocks

    def raw_bytes_gpu(self) -> np.ndarray:
        nb = self.num_blocks()
        out = np.empty(int(LIB.zo_q4_gpu_data_offset(nb)) + nb * 16, np.uint8)
        LIB.zo_q4_raw_bytes_gpu(_p(self.blocks), nb, _p(out))
        return out

    def slice(self) -> np.ndarray:
        out = np.empty(self.len, np.float32)
        LIB.zo_dequantize_q4(_p(self.blocks), self.len, _p(out))
        return out

    def scales_bits(self) -> np.ndarray:
        return self.blocks.reshape(-1, 18)[:, :2].copy().view(np.uint16).ravel()

    def codes(self) -> np.ndarray:
        """Unsigned nibble of every element (value + 8), element order."""
        d = self.blocks.reshape(-1, 18)[:, 2:]
        return np.concatenate([d & 0xF, d >> 4], axis=1).ravel()[: self.len]


def quantize_q4(src) -> Q4Storage:
    src = _f32(src).ravel()
    nb = (src.size + 31) // 32
    blocks = np.empty(nb * 18, np.uint8)
    LIB.zo_quantize_q4(_p(src), src.size, _p(blocks))
    return Q4Storage(blocks, src.size)


def q4_gpu_data_offset(total_blocks: int) -> int:
    return int(LIB.zo_q4_gpu_data_offset(total_blocks))


@dataclass
class Q8Storage:
    """tensor/quantized.go:283-298; blocks = 36-byte AoS as RawBytes() (:427-438)."""
    blocks: np.ndarray
    len: int

    def num_blocks(self) -> int:
        return (self.len + 31) // 32

    def raw_bytes(self) -> np.ndarray:
        return self.blocks

    def slice(self) -> np.ndarray:
        out = np.empty(self.len, np.float32)
        LIB.zo_dequantize_q8(_p(self.blocks), self.len, _p(out))
        return out

    def scales(self) -> np.ndarray:
        return self.blocks.reshape(-1, 36)[:, :4].copy().view(np.float32).ravel()

    def codes(self) -> np.ndarray:
        return self.blocks.reshape(-1, 36)[:, 4:].copy().view(np.int8).ravel()[: self.len]


def quantize_q8(src) -> Q8Storage:
    src = _f32(src).ravel()
    nb = (src.size + 31) // 32
    blocks = np.empty(nb * 36, np.uint8)
    LIB.zo_quantize_q8(_p(src), src.size, _p(blocks))
    return Q8Storage(blocks, src.size)


def iq4nl_table() -> np.ndarray:
    t = np.empty(16, np.float32)
    LIB.zo_iq4nl_table(_p(t))
    return t


@dataclass
class IQ4NLStorage:
    """tensor/iq4_storage.go:49-72: raw 18-byte blocks; the reference has no quantizer."""
    raw: np.ndarray
    len: int

    def num_blocks(self) -> int:
        return (self.len + 31) // 32

    def raw_bytes(self) -> np.ndarray:
        return self.raw

    def slice(self) -> np.ndarray:
        out = np.empty(self.len, np.float32)
        LIB.zo_dequantize_iq4nl(_p(self.raw), self.len, _p(out))
        return out


def new_iq4nl_from_raw(raw, num_elements: int) -> IQ4NLStorage:
    """NewIQ4NLStorageFromRaw, tensor/iq4_storage.go:61-72 (same error cases)."""
    if num_elements <= 0:
        raise ValueError(f"numElements must be positive, got {num_elements}")
    nb = (num_elements + 31) // 32
    raw = np.ascontiguousarray(raw, dtype=np.uint8).ravel()
    if raw.size < nb * 18:
        raise ValueError(f"IQ4_NL raw data too short: need {nb*18} bytes for {nb} blocks, got {raw.size}")
    return IQ4NLStorage(raw[: nb * 18].copy(), num_elements)


def make_iq4nl_blocks(src) -> IQ4NLStorage:
    """Harness-side IQ4_NL block generator (NOT a reference function).

    d = fp16(absmax / 1.3312578); nibble = index of the table entry nearest to
    w/d; byte i = nibble[2i] | nibble[2i+1] << 4 as DequantizeIQ4NL reads them.
    Parity is defined on the resulting bytes.
    """
    src = _f32(src).ravel()
    assert src.size % 32 == 0
    w = src.reshape(-1, 32)
    tab = iq4nl_table()
    absmax = np.abs(w).max(axis=1)
    d16 = f32_to_f16_bits(absmax / np.float32(1.3312578))
    d = f16_bits_to_f32(d16)
    inv = np.where(d > 0, 1.0 / np.where(d > 0, d, 1), 0).astype(np.float32)
    idx = np.abs((w * inv[:, None])[:, :, None] - tab[None, None, :]).argmin(axis=2).astype(np.uint8)
    blocks = np.empty((w.shape[0], 18), np.uint8)
    blocks[:, :2] = d16.view(np.uint8).reshape(-1, 2)
    blocks[:, 2:] = idx[:, 0::2] | (idx[:, 1::2] << 4)
    return IQ4NLStorage(blocks.ravel(), src.size)


@dataclass
class TernaryStorage:
    """tensor/ternary_storage.go:5-10: 2 bits per value, flat (rows are not padded)."""
    data: np.ndarray
    len: int

    def raw_bytes(self) -> np.ndarray:
        return self.data

    def get(self, i: int) -> int:
        if i < 0 or i >= self.len:
            raise IndexError("tensor: TernaryStorage index out of range")
        return int(LIB.zo_ternary_get(_p(self.data), i))

    def slice(self) -> np.ndarray:
        sh = (np.arange(self.len) % 4) * 2
        return (((self.data[np.arange(self.len) // 4] >> sh) & 3).astype(np.int8) - 1).astype(np.float32)


def new_ternary_from(values) -> TernaryStorage:
    """NewTernaryStorageFrom, tensor/ternary_storage.go:27-35 (panics -> ValueError)."""
    v = np.ascontiguousarray(values, dtype=np.int8).ravel()
    if v.size and (v.min() < -1 or v.max() > 1):
        raise ValueError("tensor: TernaryStorage value must be -1, 0, or 1")
    data = np.zeros((v.size + 3) // 4, np.uint8)
    LIB.zo_ternary_pack(_p(v), v.size, _p(data))
    return TernaryStorage(data, v.size)


@dataclass
class GroupQuantStorage:
    """GPTQStorage (bits=4) / AWQStorage: tensor/quantized_gptq.go:31-41, quantized_awq.go:32-40."""
    kind: str                 # "gptq" | "awq"
    data: np.ndarray          # packed bytes, groups concatenated
    scales: np.ndarray        # uint16 fp16 bits per group
    zeros: np.ndarray         # uint16 fp16 bits per group
    len: int
    group_size: int

    def num_groups(self) -> int:
        return (self.len + self.group_size - 1) // self.group_size

    def bits(self) -> int:
        return 4

    def slice(self) -> np.ndarray:
        out = np.empty(self.len, np.float32)
        fn = LIB.zo_dequantize_gptq4 if self.kind == "gptq" else LIB.zo_dequantize_awq
        fn(_p(self.data), _p(self.scales), _p(self.zeros), self.len, self.group_size, _p(out))
        return out

    def codes(self) -> np.ndarray:
        assert self.len % self.group_size == 0 and self.group_size % 8 == 0
        return np.stack([self.data & 0xF, self.data >> 4], axis=1).ravel()[: self.len]


def _quantize_group(kind: str, src, group: int) -> GroupQuantStorage:
    src = _f32(src).ravel()
    ng = (src.size + group - 1) // group
    nbytes = int((LIB.zo_gptq4_data_bytes if kind == "gptq" else LIB.zo_awq_data_bytes)(src.size, group))
    data = np.empty(nbytes, np.uint8)
    scales = np.empty(ng, np.uint16)
    zeros = np.empty(ng, np.uint16)
    fn = LIB.zo_quantize_gptq4 if kind == "gptq" else LIB.zo_quantize_awq
    fn(_p(src), src.size, group, _p(data), _p(scales), _p(zeros))
    return GroupQuantStorage(kind, data, scales, zeros, src.size, group)


def quantize_gptq(src, group_size: int = 128, bits: int = 4) -> GroupQuantStorage:
    if bits != 4:
        raise ValueError("oracle restates the 4-bit GPTQ path only")
    return _quantize_group("gptq", src, group_size)


def quantize_awq(src, group_size: int = 128) -> GroupQuantStorage:
    return _quantize_group("awq", src, group_size)


@dataclass
class Float16Storage:
    """tensor/fp16_storage.go:14-22."""
    bits: np.ndarray
    len: int

    def slice(self) -> np.ndarray:
        return f16_bits_to_f32(self.bits)


def new_float16_from_f32(src) -> Float16Storage:
    b = f32_to_f16_bits(src)
    return Float16Storage(b, b.size)


# --------------------------------------------------------------------------
# xblas
# --------------------------------------------------------------------------

def sgemm_simd(m, n, k, a, b, c=None) -> np.ndarray:
    a, b = _f32(a).ravel(), _f32(b).ravel()
    if c is None:
        c = np.zeros(m * n, np.float32)
    LIB.zo_sgemm_simd(m, n, k, _p(a), _p(b), _p(c))
    return c


def gemm_q4_f32(m, n, k, a: Q4Storage, b) -> np.ndarray:
    b = _f32(b).ravel()
    c = np.empty(m * n, np.float32)
    LIB.zo_gemm_q4_f32_fused(m, n, k, _p(a.blocks), _p(b), _p(c))
    return c


def gemm_f32_q4_nt(m, n, k, a, b: Q4Storage, ncpu: int = 0) -> np.ndarray:
    a = _f32(a).ravel()
    c = np.empty(m * n, np.float32)
    LIB.zo_gemm_f32_q4_nt(m, n, k, _p(a), _p(b.blocks), _p(c), ncpu)
    return c


def gemm_q8_f32(m, n, k, a: Q8Storage, b) -> np.ndarray:
    b = _f32(b).ravel()
    c = np.zeros(m * n, np.float32)
    LIB.zo_gemm_q8_f32(m, n, k, _p(a.blocks), _p(b), _p(c))
    return c


def gemm_f32_q8_nt(m, n, k, a, b: Q8Storage, ncpu: int = 0) -> np.ndarray:
    a = _f32(a).ravel()
    c = np.empty(m * n, np.float32)
    LIB.zo_gemm_f32_q8_nt(m, n, k, _p(a), _p(b.blocks), _p(c), ncpu)
    return c


def nt_threads(n: int, k: int, ncpu: int = 0) -> int:
    return int(LIB.zo_nt_threads(n, k, ncpu))


def num_cpu() -> int:
    return int(LIB.zo_num_cpu())


# --------------------------------------------------------------------------
# engine level (2-D operands only: what the GEMV path uses)
# --------------------------------------------------------------------------

def cpu_engine_matmul(a, a_shape, b, b_shape) -> np.ndarray:
    """CPUEngine.MatMul for 2-D float32 tensors, compute/cpu_engine.go:1124-1240.

    `a` / `b` are float32 arrays or one of the storages above.  Dispatch order
    is tryQuantizedMatMul's (:2277-2434): Q4/Q8 on A, then Q4/Q8 on B (B is then
    the physical [N,K] weight behind a logical [K,N] shape); every other storage
    is dequantized with Slice() and multiplied by SgemmSimd.
    """
    m, k = a_shape
    k2, n = b_shape
    if k != k2:
        raise ValueError(f"invalid shapes for matrix multiplication: a.Shape()={list(a_shape)}, b.Shape()={list(b_shape)}")
    if isinstance(a, Q4Storage):
        return gemm_q4_f32(m, n, k, a, _dense(b)).reshape(m, n)
    if isinstance(a, Q8Storage):
        return gemm_q8_f32(m, n, k, a, _dense(b)).reshape(m, n)
    if isinstance(b, Q4Storage):
        return gemm_f32_q4_nt(m, n, k, _dense(a), b).reshape(m, n)
    if isinstance(b, Q8Storage):
        return gemm_f32_q8_nt(m, n, k, _dense(a), b).reshape(m, n)
    return sgemm_simd(m, n, k, _dense(a), _dense(b)).reshape(m, n)


def _dense(t) -> np.ndarray:
    return t.slice() if hasattr(t, "slice") else _f32(t).ravel()


def matmul_w4a16(a, a_shape, b, b_shape) -> np.ndarray:
    """compute.MatMulW4A16, compute/w4a16.go:71-119: dequantize the 4-bit operand
    and decode the fp16 operand to float32, then the engine's float32 MatMul."""
    w4 = (Q4Storage, GroupQuantStorage)
    if isinstance(a, w4) and isinstance(b, Float16Storage):
        pass
    elif isinstance(b, w4) and isinstance(a, Float16Storage):
        pass
    else:
        raise ValueError("MatMulW4A16: inputs are not W4A16 — need 4-bit weights and FP16 activations")
    return cpu_engine_matmul(a.slice(), a_shape, b.slice(), b_shape)


def ternary_gemv(weights: TernaryStorage, x, rows: int, cols: int) -> np.ndarray:
    """compute.TernaryGEMV, compute/ternary_gemv.go:12-60."""
    x = _f32(x).ravel()
    y = np.empty(rows, np.float32)
    LIB.zo_ternary_gemv(_p(weights.data), _p(x), rows, cols, _p(y))
    return y


def ternary_gemv_scaled(weights: TernaryStorage, x_bits, row_scale_bits, rows: int, cols: int) -> np.ndarray:
    """TernaryGEMV on fp16-decoded x, then y[n] *= f32(scale16[n]) in float32.

    The per-row scale is not in the reference (it has none); this is the
    benchmark configuration's epilogue, defined here once for both sides."""
    y = ternary_gemv(weights, f16_bits_to_f32(x_bits), rows, cols)
    return (y * f16_bits_to_f32(row_scale_bits)).astype(np.float32)


def fused_add_rmsnorm(x, residual, weight, eps: float):
    """fused_add_rmsnorm.cu of the reference, one row: returns (normed, x + residual); residual may be None."""
    x = _f32(x)
    w = _f32(weight)
    res = _f32(residual) if residual is not None else None
    normed = np.empty_like(x)
    summed = np.empty_like(x)
    LIB.zo_fused_add_rmsnorm(_p(x), _p(res) if res is not None else None, _p(w), _p(normed), _p(summed), float(eps), x.size)
    return normed, summed


def fused_swiglu(w1, w3) -> np.ndarray:
    """fused_swiglu.cu of the reference: w1 * sigmoid(w1) * w3."""
    a, b = _f32(w1), _f32(w3)
    out = np.empty_like(a)
    LIB.zo_fused_swiglu(_p(a), _p(b), _p(out), a.size)
    return out


# ---- Q4_K (tensor/quantized_kquant.go) -----------------------------------------------------------
@dataclass
class Q4KStorage:
    """tensor.Q4KStorage: super-blocks of 256 weights in 144 bytes (fp16 d, fp16 dmin, 12 bytes of 6-bit scales
    and mins, 128 bytes of nibbles)."""
    raw: np.ndarray
    len: int

    def num_blocks(self) -> int:
        return (self.len + 255) // 256

    def slice(self) -> np.ndarray:
        dst = np.empty(self.len, dtype=np.float32)
        LIB.zo_dequantize_q4k(_p(self.raw), self.len, _p(dst))
        return dst

    def scales_mins(self, block: int):
        sc = np.zeros(8, dtype=np.uint8)
        mn = np.zeros(8, dtype=np.uint8)
        LIB.zo_q4k_scales_mins(_p(self.raw[block * 144:]), _p(sc), _p(mn))
        return sc, mn

    def raw_bytes_gpu(self) -> np.ndarray:
        """Device layout of this build: the 16 header bytes of every super-block first, then (16-byte aligned)
        the 128 nibble bytes of every super-block -- the split tensor.Q4Storage.RawBytesGPU makes for Q4_0."""
        nb = self.num_blocks()
        blocks = self.raw.reshape(nb, 144)
        return np.concatenate([blocks[:, :16].reshape(-1), blocks[:, 16:].reshape(-1)])


def quantize_q4k(src) -> Q4KStorage:
    src = _f32(src)
    nb = (src.size + 255) // 256
    raw = np.zeros(nb * 144, dtype=np.uint8)
    LIB.zo_quantize_q4k(_p(src), src.size, _p(raw))
    return Q4KStorage(raw, src.size)


def new_q4k_from_raw(raw, num_elements: int) -> Q4KStorage:
    """NewQ4KStorageFromRaw (quantized_kquant.go:248-260)."""
    raw = np.ascontiguousarray(raw, dtype=np.uint8)
    if num_elements <= 0:
        raise ValueError("numElements must be positive")
    need = (num_elements + 255) // 256 * 144
    if raw.size < need:
        raise ValueError(f"raw data too short: need {need} bytes, got {raw.size}")
    return Q4KStorage(raw[:need].copy(), num_elements)


def gemm_q4k_f32(m, n, k, a: Q4KStorage, b) -> np.ndarray:
    c = np.zeros(m * n, dtype=np.float32)
    LIB.zo_gemm_q4k_f32(m, n, k, _p(a.raw), _p(_f32(b)), _p(c))
    return c


def gemm_f32_q4k_nt(m, n, k, a, b: Q4KStorage, ncpu: int = 0) -> np.ndarray:
    c = np.zeros(m * n, dtype=np.float32)
    LIB.zo_gemm_f32_q4k_nt(m, n, k, _p(_f32(a)), _p(b.raw), _p(c), ncpu)
    return c


# ---- Q5_K (tensor/quantized_kquant.go:489-621) ---------------------------------------------------
@dataclass
class Q5KStorage:
    """tensor.Q5KStorage: 176-byte super-blocks {fp16 d, fp16 dmin, 12 scale bytes, 128 bytes ql, 32 bytes qh}."""
    raw: np.ndarray
    len: int

    def num_blocks(self) -> int:
        return (self.len + 255) // 256

    def slice(self) -> np.ndarray:
        dst = np.empty(self.len, dtype=np.float32)
        LIB.zo_dequantize_q5k(_p(self.raw), self.len, _p(dst))
        return dst

    def raw_bytes_gpu(self) -> np.ndarray:
        """Device layout of this build: per super-block 48 bytes {16 header bytes, 32 bytes qh} first, then the
        128 low-nibble bytes of every super-block."""
        nb = self.num_blocks()
        blocks = self.raw.reshape(nb, 176)
        side = np.concatenate([blocks[:, :16], blocks[:, 144:176]], axis=1)
        return np.concatenate([side.reshape(-1), blocks[:, 16:144].reshape(-1)])


def make_q5k_blocks(src) -> Q5KStorage:
    """Test-data generator (the reference has no Q5_K quantizer): Q4_K's recipe with 31 levels."""
    src = _f32(src)
    nb = (src.size + 255) // 256
    raw = np.zeros(nb * 176, dtype=np.uint8)
    LIB.zo_make_q5k_blocks(_p(src), src.size, _p(raw))
    return Q5KStorage(raw, src.size)


def new_q5k_from_raw(raw, num_elements: int) -> Q5KStorage:
    """NewQ5KStorageFromRaw (quantized_kquant.go:564-577)."""
    raw = np.ascontiguousarray(raw, dtype=np.uint8)
    if num_elements <= 0:
        raise ValueError("numElements must be positive")
    need = (num_elements + 255) // 256 * 176
    if raw.size < need:
        raise ValueError(f"raw data too short: need {need} bytes, got {raw.size}")
    return Q5KStorage(raw[:need].copy(), num_elements)


def gemm_f32_q5k_nt(m, n, k, a, b: Q5KStorage, ncpu: int = 0) -> np.ndarray:
    c = np.zeros(m * n, dtype=np.float32)
    LIB.zo_gemm_f32_q5k_nt(m, n, k, _p(_f32(a)), _p(b.raw), _p(c), ncpu)
    return c


# ---- Q6_K (tensor/quantized_kquant.go:335-483) ---------------------------------------------------
@dataclass
class Q6KStorage:
    """tensor.Q6KStorage: 210-byte super-blocks {128 bytes ql, 64 bytes qh, 16 int8 scales, fp16 d}."""
    raw: np.ndarray
    len: int

    def num_blocks(self) -> int:
        return (self.len + 255) // 256

    def slice(self) -> np.ndarray:
        dst = np.empty(self.len, dtype=np.float32)
        LIB.zo_dequantize_q6k(_p(self.raw), self.len, _p(dst))
        return dst

    def raw_bytes_gpu(self) -> np.ndarray:
        """Device layout of this build: per super-block 96 side bytes {64 bytes qh, 16 scales, fp16 d, 14 zero
        bytes} first, then the 128 ql bytes of every super-block."""
        nb = self.num_blocks()
        blocks = self.raw.reshape(nb, 210)
        side = np.zeros((nb, 96), dtype=np.uint8)
        side[:, :64] = blocks[:, 128:192]
        side[:, 64:80] = blocks[:, 192:208]
        side[:, 80:82] = blocks[:, 208:210]
        return np.concatenate([side.reshape(-1), blocks[:, :128].reshape(-1)])


def make_q6k_blocks(src) -> Q6KStorage:
    """Test-data generator (the reference has no Q6_K quantizer): the recipe of its test builder."""
    src = _f32(src)
    nb = (src.size + 255) // 256
    raw = np.zeros(nb * 210, dtype=np.uint8)
    LIB.zo_make_q6k_blocks(_p(src), src.size, _p(raw))
    return Q6KStorage(raw, src.size)


def new_q6k_from_raw(raw, num_elements: int) -> Q6KStorage:
    """NewQ6KStorageFromRaw (quantized_kquant.go:397-409)."""
    raw = np.ascontiguousarray(raw, dtype=np.uint8)
    if num_elements <= 0:
        raise ValueError("numElements must be positive")
    need = (num_elements + 255) // 256 * 210
    if raw.size < need:
        raise ValueError(f"raw data too short: need {need} bytes, got {raw.size}")
    return Q6KStorage(raw[:need].copy(), num_elements)


def gemm_f32_q6k_nt(m, n, k, a, b: Q6KStorage, ncpu: int = 0) -> np.ndarray:
    c = np.zeros(m * n, dtype=np.float32)
    LIB.zo_gemm_f32_q6k_nt(m, n, k, _p(_f32(a)), _p(b.raw), _p(c), ncpu)
    return c
