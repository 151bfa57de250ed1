"""Q5_K GEMV (chunk-pair kernel) against the oracle's restatement of xblas.GemmF32Q5KNT."""
import numpy as np
import pytest
import torch

from oracle import oracle as O
from tests import util as U
from ztensor_b200 import kernels as K

pytestmark = pytest.mark.gpu


def _upload(st):
    nb = st.num_blocks()
    sep = torch.empty(nb * 176, dtype=torch.uint8, device="cuda")
    K.repack_blocks176(torch.from_numpy(st.raw).cuda(), sep, nb)
    torch.cuda.synchronize()
    assert np.array_equal(sep.cpu().numpy(), st.raw_bytes_gpu())          # side bytes then nibbles, byte for byte
    return sep, nb * 48


@pytest.mark.parametrize("n,k", [(64, 2048), (300, 4096), (96, 8192), (33, 14336), (16, 28672), (257, 2304)])
@pytest.mark.parametrize("batch", [1, 2])
@pytest.mark.parametrize("x_f32", [False, True])
def test_q5k_gemv(n, k, batch, x_f32):
    rng = U.seeded(n * 31 + k + batch)
    w = U.make_weights(rng, n, k).reshape(n, k // 32, 32)
    w = (w * rng.uniform(0.2, 3.0, (n, k // 32, 1)).astype(np.float32)).reshape(-1)   # uneven sub-block ranges
    st = O.make_q5k_blocks(w)
    assert (st.raw.reshape(-1, 176)[:, 144:] != 0).any()                             # fifth bits are in use
    if x_f32:
        xf = rng.standard_normal((batch, k)).astype(np.float32)
        x = torch.from_numpy(xf).cuda()
    else:
        from tests import gpu_util as G
        xb = U.make_x_bits(rng, batch, k)
        xf = O.f16_bits_to_f32(xb).reshape(batch, k)
        x = G.x_dev(xb)
    ref = O.gemm_f32_q5k_nt(batch, n, k, xf, st, ncpu=1).reshape(batch, n)
    absd = U.absdot(st.slice().reshape(n, k), xf)
    sep, off = _upload(st)
    y = torch.full((batch, n), float("nan"), device="cuda", dtype=torch.float32)
    fl = K.Y_F32 | (K.X_F32 if x_f32 else 0)
    K.gemv_q5k(sep, off, x, y, n, k, batch, fl)
    torch.cuda.synchronize()
    assert K.device_error() == 0
    got = y.cpu().numpy()
    assert np.isfinite(got).all()
    assert U.rel_err(got, ref, absd) <= U.REL_TOL
    again = torch.empty_like(y)
    K.gemv_q5k(sep, off, x, again, n, k, batch, fl)
    torch.cuda.synchronize()
    assert torch.equal(y, again)


def test_q5k_all_codes_at_the_top():
    """Every code 31 and the largest activations: the integer sub-block sums come close to 2^31."""
    n, k = 8, 2048
    nb = n * k // 256
    raw = np.zeros((nb, 176), dtype=np.uint8)
    raw[:, 0:2] = np.frombuffer(O.f32_to_f16_bits(np.array([0.01], np.float32)).tobytes(), np.uint8)
    raw[:, 4:8] = 63                                                          # scales of sub-blocks 0..3
    raw[:, 12:16] = 0x0F
    raw[:, 16:144] = 0xFF
    raw[:, 144:176] = 0xFF
    st = O.new_q5k_from_raw(raw.reshape(-1), n * k)
    assert st.slice().max() > 0
    xb = O.f32_to_f16_bits(np.full(k, 1000.0, np.float32)).reshape(1, k)
    xf = O.f16_bits_to_f32(xb).reshape(1, k)
    ref = O.gemm_f32_q5k_nt(1, n, k, xf, st, ncpu=1).reshape(1, n)
    from tests import gpu_util as G
    sep, off = _upload(st)
    y = torch.empty((1, n), device="cuda", dtype=torch.float32)
    K.gemv_q5k(sep, off, G.x_dev(xb), y, n, k, 1, K.Y_F32)
    torch.cuda.synchronize()
    assert U.rel_err(y.cpu().numpy(), ref, U.absdot(st.slice().reshape(n, k), xf)) <= U.REL_TOL
