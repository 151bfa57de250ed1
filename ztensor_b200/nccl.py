"""ctypes front end of the host library's NCCL binding (ztensor_b200/host/ztq_nccl.h): libnccl.so.2 loaded at run
time, communicators made from a 128-byte unique id, all-reduce / broadcast on a CUDA stream.  The Python names
follow internal/nccl/nccl_purego.go (GetUniqueID, InitRank, Comm.AllReduce, ...)."""
from __future__ import annotations

import ctypes as C
import glob
import os
import sysconfig

from . import engine as _engine

INT8, UINT8, INT32, UINT32, INT64, UINT64, FLOAT16, FLOAT32, FLOAT64, BFLOAT16 = range(10)
SUM, PROD, MAX, MIN, AVG = range(5)
UNIQUE_ID_BYTES = 128


class NcclError(RuntimeError):
    pass


def find_libnccl():
    """The NCCL build next to the PyTorch in use (its communicators and ours then agree on the wire protocol),
    else whatever the loader finds under the usual names."""
    pure = sysconfig.get_paths()["purelib"]
    hits = sorted(glob.glob(os.path.join(pure, "nvidia", "nccl", "lib", "libnccl.so*")))
    return hits[0] if hits else None


def _h():
    h = _engine.host()
    if not getattr(h, "_nccl_ready", False):
        h.zt_nccl_comm_init_rank.restype = C.c_void_p
        h.zt_nccl_all_reduce.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_longlong, C.c_int, C.c_int, C.c_void_p, C.c_char_p, C.c_int]
        h.zt_nccl_broadcast.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_longlong, C.c_int, C.c_int, C.c_void_p, C.c_char_p, C.c_int]
        h.zt_nccl_comm_init_rank.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_char_p, C.c_int]
        h.zt_nccl_comm_destroy.argtypes = [C.c_void_p, C.c_char_p, C.c_int]
        h._nccl_ready = True
    return h


def _chk(rc, err):
    if rc:
        raise NcclError(err.value.decode() or "nccl call failed")


def load(path: str | None = None):
    err = C.create_string_buffer(512)
    p = path or find_libnccl()
    _chk(_h().zt_nccl_load(p.encode() if p else None, err, 512), err)


def available() -> bool:
    try:
        load()
        return True
    except NcclError:
        return False


def get_unique_id() -> bytes:
    load()
    buf = C.create_string_buffer(UNIQUE_ID_BYTES)
    err = C.create_string_buffer(512)
    _chk(_h().zt_nccl_get_unique_id(buf, err, 512), err)
    return buf.raw


def error_string(rc: int) -> str:
    out = C.create_string_buffer(256)
    _h().zt_nccl_error_string(rc, out, 256)
    return out.value.decode()


class Comm:
    """nccl.Comm: InitRank with the same id on every rank (the CUDA device of the rank must be current)."""

    def __init__(self, unique_id: bytes, n_ranks: int, rank: int):
        if len(unique_id) != UNIQUE_ID_BYTES:
            raise NcclError(f"UniqueIDFromBytes: expected {UNIQUE_ID_BYTES} bytes, got {len(unique_id)}")
        load()
        err = C.create_string_buffer(512)
        h = _h().zt_nccl_comm_init_rank(C.create_string_buffer(unique_id, UNIQUE_ID_BYTES), n_ranks, rank, err, 512)
        if not h:
            raise NcclError(err.value.decode() or "ncclCommInitRank failed")
        self.h, self.rank, self.size = C.c_void_p(h), rank, n_ranks

    def all_reduce(self, send_ptr: int, recv_ptr: int, count: int, dtype: int, op: int = SUM, stream: int = 0):
        err = C.create_string_buffer(512)
        _chk(_h().zt_nccl_all_reduce(self.h, C.c_void_p(send_ptr), C.c_void_p(recv_ptr), count, dtype, op, C.c_void_p(stream), err, 512), err)

    def broadcast(self, send_ptr: int, recv_ptr: int, count: int, dtype: int, root: int, stream: int = 0):
        err = C.create_string_buffer(512)
        _chk(_h().zt_nccl_broadcast(self.h, C.c_void_p(send_ptr), C.c_void_p(recv_ptr), count, dtype, root, C.c_void_p(stream), err, 512), err)

    def all_reduce_tensor(self, t, op: int = SUM, stream=None):
        """In-place all-reduce of a torch CUDA tensor (fp16, bf16, fp32, fp64, int32, int64) on the current stream."""
        import torch
        dt = {torch.float16: FLOAT16, torch.bfloat16: BFLOAT16, torch.float32: FLOAT32, torch.float64: FLOAT64,
              torch.int32: INT32, torch.int64: INT64}[t.dtype]
        st = torch.cuda.current_stream().cuda_stream if stream is None else stream.cuda_stream
        self.all_reduce(t.data_ptr(), t.data_ptr(), t.numel(), dt, op, st)

    def destroy(self):
        if self.h:
            err = C.create_string_buffer(512)
            h, self.h = self.h, None
            _chk(_h().zt_nccl_comm_destroy(h, err, 512), err)
