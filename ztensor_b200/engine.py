"""ctypes front end of libztq_host.so, the C++ mirror of the reference's engine API
(ztensor_b200/host/ztq_engine.h).  Used by the parity tests and as the binding
example for foreign callers; the arithmetic is in the CUDA library."""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

from . import _lib

_HERE = os.path.dirname(os.path.abspath(__file__))
HOST_LIB_PATH = os.path.join(_HERE, "libztq_host.so")
KIND = {"cpu": 0, "gpu": 1, "f16": 2, "q4": 3, "q8": 4, "iq4nl": 5, "gptq": 6, "awq": 7, "ternary": 8, "q4k": 9, "q5k": 10, "q6k": 11}
_h = None


def host():
    global _h
    if _h is None:
        _lib.lib()                                           # kernel library first (RTLD_GLOBAL)
        if not os.path.exists(HOST_LIB_PATH):
            raise _lib.KernelLibraryMissing(f"{HOST_LIB_PATH} not found: build it with `make -C ztensor_b200/host`")
        h = C.CDLL(HOST_LIB_PATH)
        for name in ("zt_engine_new", "zt_tensor_cpu", "zt_tensor_f16_raw", "zt_tensor_f16_from_f32", "zt_tensor_q4_raw",
                     "zt_tensor_q8_blocks", "zt_tensor_iq4nl_raw", "zt_tensor_q4k_raw", "zt_tensor_q5k_raw", "zt_tensor_q6k_raw", "zt_tensor_gptq_raw", "zt_tensor_awq_raw",
                     "zt_tensor_ternary", "zt_quantize", "zt_device_tensor", "zt_tensor_w4g_device", "zt_matmul_async",
                     "zt_end_capture", "zt_tensor_view", "zt_engine_stream"):
            getattr(h, name).restype = C.c_void_p
        h.zt_engine_launches.restype = C.c_longlong
        h.zt_tensor_bytes.restype = C.c_longlong
        h.zt_pool_driver_allocs.restype = C.c_longlong
        h.zt_pool_epoch.restype = C.c_longlong
        h.zt_tensor_device_ptr.restype = C.c_ulonglong
        h.zt_copy_from_host.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_longlong, C.c_char_p, C.c_int]
        h.zt_copy_to_host.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_longlong, C.c_char_p, C.c_int]
        h.zt_tensor_w4g_device.argtypes = [C.c_void_p, C.c_longlong, C.c_longlong, C.c_longlong, C.c_int, C.c_int, C.c_int,
                                           C.POINTER(C.c_int), C.c_int, C.c_char_p, C.c_int]
        h.zt_tensor_view.argtypes = [C.c_void_p, C.c_longlong, C.c_longlong, C.POINTER(C.c_int), C.c_int, C.c_char_p, C.c_int]
        _h = h
    return _h


def _p(a):
    return a.ctypes.data_as(C.c_void_p) if a is not None else None


def _shape(shape):
    return (C.c_int * len(shape))(*shape), len(shape)


class EngineError(RuntimeError):
    pass


class Tensor:
    def __init__(self, handle):
        if not handle:
            raise EngineError("null tensor handle")
        self.h = C.c_void_p(handle)

    def __del__(self):
        if getattr(self, "h", None) and _h is not None:
            _h.zt_tensor_free(self.h)
            self.h = None

    @property
    def shape(self):
        buf = (C.c_int * 8)()
        r = host().zt_tensor_shape(self.h, buf, 8)
        return tuple(buf[i] for i in range(r))

    @property
    def device_ptr(self) -> int:
        return int(host().zt_tensor_device_ptr(self.h))

    def view(self, offset_elems: int, length: int, shape) -> "Tensor":
        s, r = _shape(shape)
        e = _err()
        return Tensor(_chk(host().zt_tensor_view(self.h, offset_elems, length, s, r, e, 512), e))

    @property
    def refcount(self) -> int:
        return int(host().zt_tensor_refcount(self.h))

    def free_storage(self):
        host().zt_tensor_free_storage(self.h)

    @property
    def resident(self) -> bool:
        return bool(host().zt_tensor_resident(self.h))

    def bytes(self, which=0) -> np.ndarray:
        n = host().zt_tensor_bytes(self.h, which, None, 0)
        out = np.empty(max(n, 0), np.uint8)
        host().zt_tensor_bytes(self.h, which, _p(out), n)
        return out


def _err():
    return C.create_string_buffer(512)


def _chk(handle_or_rc, err, is_handle=True):
    if (is_handle and not handle_or_rc) or (not is_handle and handle_or_rc != 0):
        raise EngineError(err.value.decode())
    return handle_or_rc


def cpu_tensor(data, shape) -> Tensor:
    d = np.ascontiguousarray(data, np.float32)
    s, r = _shape(shape)
    return Tensor(host().zt_tensor_cpu(_p(d), s, r))


def f16_tensor_from_bits(bits, shape) -> Tensor:
    b = np.ascontiguousarray(bits, np.uint16)
    s, r = _shape(shape)
    return Tensor(host().zt_tensor_f16_raw(_p(b), s, r))


def f16_tensor_from_f32(data, shape) -> Tensor:
    d = np.ascontiguousarray(data, np.float32)
    s, r = _shape(shape)
    return Tensor(host().zt_tensor_f16_from_f32(_p(d), s, r))


def q4_tensor(raw, n, shape) -> Tensor:
    raw = np.ascontiguousarray(raw, np.uint8)
    s, r = _shape(shape)
    e = _err()
    return Tensor(_chk(host().zt_tensor_q4_raw(_p(raw), C.c_longlong(raw.size), C.c_longlong(n), s, r, e, 512), e))


def iq4nl_tensor(raw, n, shape) -> Tensor:
    raw = np.ascontiguousarray(raw, np.uint8)
    s, r = _shape(shape)
    e = _err()
    return Tensor(_chk(host().zt_tensor_iq4nl_raw(_p(raw), C.c_longlong(raw.size), C.c_longlong(n), s, r, e, 512), e))


def q4k_tensor(raw, n, shape) -> Tensor:
    """tensor.NewQ4KStorageFromRaw: 144-byte super-blocks."""
    raw = np.ascontiguousarray(raw, np.uint8)
    s, r = _shape(shape)
    e = _err()
    return Tensor(_chk(host().zt_tensor_q4k_raw(_p(raw), C.c_longlong(raw.size), C.c_longlong(n), s, r, e, 512), e))


def q5k_tensor(raw, n, shape) -> Tensor:
    """tensor.NewQ5KStorageFromRaw: 176-byte super-blocks."""
    raw = np.ascontiguousarray(raw, np.uint8)
    s, r = _shape(shape)
    e = _err()
    return Tensor(_chk(host().zt_tensor_q5k_raw(_p(raw), C.c_longlong(raw.size), C.c_longlong(n), s, r, e, 512), e))


def q6k_tensor(raw, n, shape) -> Tensor:
    """tensor.NewQ6KStorageFromRaw: 210-byte super-blocks."""
    raw = np.ascontiguousarray(raw, np.uint8)
    s, r = _shape(shape)
    e = _err()
    return Tensor(_chk(host().zt_tensor_q6k_raw(_p(raw), C.c_longlong(raw.size), C.c_longlong(n), s, r, e, 512), e))


def q8_tensor(scales, quants, n, shape) -> Tensor:
    sc = np.ascontiguousarray(scales, np.float32)
    q = np.ascontiguousarray(quants, np.int8)
    s, r = _shape(shape)
    e = _err()
    return Tensor(_chk(host().zt_tensor_q8_blocks(_p(sc), _p(q), C.c_longlong(sc.size), C.c_longlong(n), s, r, e, 512), e))


def gptq_tensor(data, scales, zeros, n, group, shape, bits=4) -> Tensor:
    d = np.ascontiguousarray(data, np.uint8)
    sc = np.ascontiguousarray(scales, np.uint16)
    z = np.ascontiguousarray(zeros, np.uint16)
    if sc.size != z.size:
        raise EngineError(f"expected {sc.size} zeros for {sc.size} groups, got {z.size}")
    s, r = _shape(shape)
    e = _err()
    return Tensor(_chk(host().zt_tensor_gptq_raw(_p(d), C.c_longlong(d.size), _p(sc), _p(z), C.c_longlong(sc.size),
                                                 C.c_longlong(n), group, bits, s, r, e, 512), e))


def awq_tensor(words, scales, zeros, n, group, shape) -> Tensor:
    w = np.ascontiguousarray(words, np.uint32)
    sc = np.ascontiguousarray(scales, np.uint16)
    z = np.ascontiguousarray(zeros, np.uint16)
    s, r = _shape(shape)
    e = _err()
    return Tensor(_chk(host().zt_tensor_awq_raw(_p(w), C.c_longlong(w.size), _p(sc), _p(z), C.c_longlong(sc.size),
                                                C.c_longlong(n), group, s, r, e, 512), e))


def w4g_device_tensor(dev_ptr: int, dev_bytes: int, meta_off: int, n: int, group, shape, awq=False, device=0) -> Tensor:
    """A GPTQ / AWQ weight already resident on the device in the layout [nibbles][pad][half2 meta at meta_off]."""
    s, r = _shape(shape)
    e = _err()
    return Tensor(_chk(host().zt_tensor_w4g_device(C.c_void_p(dev_ptr), dev_bytes, meta_off, n, group, 1 if awq else 0, device,
                                                   s, r, e, 512), e))


def ternary_tensor(values, shape, row_scale_bits=None) -> Tensor:
    v = np.ascontiguousarray(values, np.int8)
    rs = np.ascontiguousarray(row_scale_bits, np.uint16) if row_scale_bits is not None else None
    s, r = _shape(shape)
    e = _err()
    return Tensor(_chk(host().zt_tensor_ternary(_p(v), C.c_longlong(v.size), _p(rs), C.c_longlong(0 if rs is None else rs.size),
                                                s, r, e, 512), e))


class GPUEngine:
    """compute.GPUEngine[float32], the quantized-MatMul part."""

    def __init__(self, device: int = 0):
        e = _err()
        self.h = C.c_void_p(_chk(host().zt_engine_new(device, e, 512), e))

    def __del__(self):
        if getattr(self, "h", None) and _h is not None:
            _h.zt_engine_free(self.h)
            self.h = None

    @property
    def launches(self) -> int:
        return int(host().zt_engine_launches(self.h))

    def quantize(self, kind: str, src, shape, group=128) -> Tensor:
        d = np.ascontiguousarray(src, np.float32)
        s, r = _shape(shape)
        e = _err()
        return Tensor(_chk(host().zt_quantize(self.h, KIND[kind], _p(d), C.c_longlong(d.size), group, s, r, e, 512), e))

    def upload_weights(self, tensors):
        arr = (C.c_void_p * len(tensors))(*[t.h for t in tensors])
        e = _err()
        _chk(host().zt_upload_weights(self.h, arr, len(tensors), e, 512), e, False)

    def _mm(self, a, b, dst, mode):
        cap = 1 << 22
        out = np.empty(cap, np.float32)
        shp = (C.c_int * 8)()
        rank = C.c_int(0)
        matched = C.c_int(1)
        e = _err()
        _chk(host().zt_matmul(self.h, a.h, b.h, dst.h if dst is not None else None, mode, _p(out), C.c_longlong(cap), shp,
                              C.byref(rank), C.byref(matched), e, 512), e, False)
        if not matched.value:
            return None, False
        shape = tuple(shp[i] for i in range(rank.value))
        return out[: int(np.prod(shape))].reshape(shape).copy(), True

    def matmul(self, a, b, dst=None):
        return self._mm(a, b, dst, 0)[0]

    def matmul_w4a16(self, a, b, dst=None):
        return self._mm(a, b, dst, 1)[0]

    def try_w4a16_matmul(self, a, b, dst=None):
        return self._mm(a, b, dst, 2)

    # ---- the asynchronous, pooled, capturable side (what a decode loop uses) -----------------------------------
    def device_tensor(self, shape, f16=False) -> Tensor:
        """A device tensor of float32 (or fp16) elements from the engine's pool."""
        s, r = _shape(shape)
        e = _err()
        return Tensor(_chk(host().zt_device_tensor(self.h, s, r, 1 if f16 else 0, e, 512), e))

    def copy_from_host(self, t: Tensor, host_ptr: int, nbytes: int):
        e = _err()
        _chk(host().zt_copy_from_host(self.h, t.h, C.c_void_p(host_ptr), nbytes, e, 512), e, False)

    def copy_to_host(self, t: Tensor, host_ptr: int, nbytes: int):
        e = _err()
        _chk(host().zt_copy_to_host(self.h, t.h, C.c_void_p(host_ptr), nbytes, e, 512), e, False)

    def sync(self):
        e = _err()
        _chk(host().zt_engine_sync(self.h, e, 512), e, False)

    @property
    def stream(self) -> int:
        return int(host().zt_engine_stream(self.h) or 0)

    def matmul_async(self, a, b, dst=None, mode=0):
        """MatMul (mode 0), MatMulW4A16 (1) or TryW4A16MatMul (2) without any copy or wait: the result stays on the
        device (it is dst when dst is a device tensor)."""
        matched = C.c_int(1)
        e = _err()
        h = host().zt_matmul_async(self.h, a.h, b.h, dst.h if dst is not None else None, mode, C.byref(matched), e, 512)
        if not h:
            if not matched.value:
                return None
            raise EngineError(e.value.decode() or "zt_matmul_async failed")
        return Tensor(h)

    def to_host(self, t: Tensor) -> np.ndarray:
        shape = t.shape
        out = np.empty(int(np.prod(shape)), np.float32)
        e = _err()
        _chk(host().zt_tensor_to_host(self.h, t.h, _p(out), C.c_longlong(out.size), e, 512), e, False)
        return out.reshape(shape)

    def begin_capture(self):
        e = _err()
        _chk(host().zt_begin_capture(self.h, e, 512), e, False)

    def end_capture(self) -> int:
        e = _err()
        return _chk(host().zt_end_capture(self.h, e, 512), e)

    def replay_graph(self, graph: int):
        e = _err()
        _chk(host().zt_replay_graph(self.h, C.c_void_p(graph), e, 512), e, False)

    def destroy_graph(self, graph: int):
        e = _err()
        _chk(host().zt_destroy_graph(self.h, C.c_void_p(graph), e, 512), e, False)

    @property
    def pool_driver_allocs(self) -> int:
        return int(host().zt_pool_driver_allocs(self.h))

    @property
    def pool_epoch(self) -> int:
        return int(host().zt_pool_epoch(self.h))

    def pool_reset(self):
        host().zt_pool_reset(self.h)

    def pool_cached(self):
        b = C.c_longlong(0)
        n = host().zt_pool_cached(self.h, C.byref(b))
        return int(n), int(b.value)

    def ternary_gemv_gpu(self, w: Tensor, x, rows, cols):
        xv = np.ascontiguousarray(x, np.float32)
        y = np.empty(rows, np.float32)
        e = _err()
        _chk(host().zt_ternary_gemv_gpu(self.h, w.h, _p(xv), rows, cols, _p(y), e, 512), e, False)
        return y
