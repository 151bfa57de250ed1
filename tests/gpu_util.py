"""GPU-side helpers: upload oracle storages into the residency layouts using the
library's own repack kernels, and run each GEMV through the C-ABI."""
from __future__ import annotations

import numpy as np
import torch

from oracle import oracle as O
from ztensor_b200 import kernels as K

DEV = "cuda"


def dev_u8(a):
    return torch.from_numpy(np.ascontiguousarray(a).view(np.uint8).ravel().copy()).to(DEV)


def upload_blocks18(blocks: np.ndarray, n_blocks: int):
    """18-byte AoS blocks -> separated layout on the device (returns tensor, data_offset)."""
    off = K.q4_gpu_data_offset(n_blocks)
    sep = torch.zeros(off + n_blocks * 16, dtype=torch.uint8, device=DEV)
    K.repack_blocks18(dev_u8(blocks), sep, n_blocks)
    return sep, off


def upload_w4g(st: O.GroupQuantStorage):
    meta = torch.empty(st.num_groups() * 4, dtype=torch.uint8, device=DEV)
    K.pack_w4g_meta(dev_u8(st.scales), dev_u8(st.zeros), meta, st.num_groups())
    return dev_u8(st.data), meta


def upload_ternary(st: O.TernaryStorage, m: int, k: int):
    rows = torch.empty(m * ((k + 3) // 4), dtype=torch.uint8, device=DEV)
    K.repack_ternary_rows(dev_u8(st.data), rows, m, k)
    return rows


def x_dev(x_bits: np.ndarray):
    return torch.from_numpy(x_bits.view(np.float16).copy()).to(DEV)


def run(fn, n, batch, y_f32=True, **kw):
    y = torch.full((batch, n), float("nan"), dtype=torch.float32 if y_f32 else torch.float16, device=DEV)
    fn(y)
    torch.cuda.synchronize()
    return y.float().cpu().numpy()
