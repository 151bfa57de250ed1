"""Committed golden vectors (tests/golden/gemv_golden.npz): the oracle still reproduces them (CPU), and the
CUDA kernels reproduce them through the C-ABI (GPU)."""
import os

import numpy as np
import pytest

from oracle import oracle as O
from tests import util as U
from tests.golden.make_golden import CASES, build

GOLD = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "gemv_golden.npz"))


def test_oracle_reproduces_the_committed_vectors_bit_for_bit():
    fresh = build()
    assert set(fresh) == set(GOLD.files)
    for key in GOLD.files:
        assert np.array_equal(fresh[key], GOLD[key]), key


@pytest.mark.gpu
@pytest.mark.parametrize("fmt,n,k,batch", CASES)
def test_kernels_reproduce_the_committed_vectors(fmt, n, k, batch):
    import torch

    from tests import gpu_util as G
    from ztensor_b200 import kernels as K
    pre = f"{fmt}_{n}x{k}_b{batch}"
    xb = GOLD[pre + "/x_bits"]
    xf = O.f16_bits_to_f32(xb).reshape(batch, k)
    want = GOLD[pre + "/y"]
    w = GOLD[pre + "/w_dequant"].reshape(n, k)
    x = G.x_dev(xb)
    if fmt in ("q4_0", "iq4nl"):
        sep, off = G.upload_blocks18(GOLD[pre + "/blocks"], n * k // 32)
        fn = K.gemv_q4_0 if fmt == "q4_0" else K.gemv_iq4nl
        run = lambda y: fn(sep, off, x, y, n, k, batch, K.Y_F32)
    elif fmt == "q4k":
        nb = n * k // 256
        sep = torch.empty(nb * 144, dtype=torch.uint8, device="cuda")
        K.repack_blocks144(G.dev_u8(GOLD[pre + "/blocks"]), sep, nb)
        run = lambda y: K.gemv_q4k(sep, nb * 16, x, y, n, k, batch, K.Y_F32)
    elif fmt == "q5k":
        nb = n * k // 256
        sep = torch.empty(nb * 176, dtype=torch.uint8, device="cuda")
        K.repack_blocks176(G.dev_u8(GOLD[pre + "/blocks"]), sep, nb)
        run = lambda y: K.gemv_q5k(sep, nb * 48, x, y, n, k, batch, K.Y_F32)
    elif fmt == "q6k":
        nb = n * k // 256
        sep = torch.empty(nb * 224, dtype=torch.uint8, device="cuda")
        K.repack_blocks210(G.dev_u8(GOLD[pre + "/blocks"]), sep, nb)
        run = lambda y: K.gemv_q6k(sep, nb * 96, x, y, n, k, batch, K.Y_F32)
    elif fmt == "q8_0":
        wd = G.dev_u8(GOLD[pre + "/blocks"])
        run = lambda y: K.gemv_q8_0(wd, x, y, n, k, batch, K.Y_F32)
    elif fmt in ("gptq", "awq"):
        st = O.GroupQuantStorage(fmt, GOLD[pre + "/data"], GOLD[pre + "/scales"], GOLD[pre + "/zeros"], n * k, 128)
        qd, meta = G.upload_w4g(st)
        run = lambda y: K.gemv_w4g(qd, meta, x, y, n, k, 128, batch, K.Y_F32)
    else:
        st = O.TernaryStorage(GOLD[pre + "/data"], n * k)
        rows = G.upload_ternary(st, n, k)
        sc = G.dev_u8(GOLD[pre + "/row_scale"])
        w = w * O.f16_bits_to_f32(GOLD[pre + "/row_scale"])[:, None]
        run = lambda y: K.gemv_ternary(rows, sc, x, y, n, k, batch, K.Y_F32)
    got = G.run(run, n, batch)
    assert U.rel_err(got, want, U.absdot(w, xf)) <= U.REL_TOL
    if fmt in ("q4k", "q5k", "q6k"):                   # no device dequantizer for K-quants: the repack is checked byte for byte
        st = {"q4k": O.Q4KStorage, "q5k": O.Q5KStorage, "q6k": O.Q6KStorage}[fmt](GOLD[pre + "/blocks"], n * k)
        assert np.array_equal(sep.cpu().numpy(), st.raw_bytes_gpu())
        return
    # dequantized weights are bit-exact: codes and scales survived the residency repack
    out = torch.empty(n * k, dtype=torch.float32, device="cuda")
    if fmt in ("q4_0", "iq4nl"):
        K.dequantize(K.FMT_Q4_0 if fmt == "q4_0" else K.FMT_IQ4NL, sep, None, out, n * k, off)
    elif fmt == "q8_0":
        K.dequantize(K.FMT_Q8_0, wd, None, out, n * k, 0)
    elif fmt in ("gptq", "awq"):
        K.dequantize(K.FMT_W4G, qd, meta, out, n * k, 128)
    else:
        K.dequantize(K.FMT_TERNARY, rows, None, out, n * k, k)
    assert np.array_equal(out.cpu().numpy(), GOLD[pre + "/w_dequant"])
