"""Q4_K GEMV (chunk-pair kernel) against the oracle's restatement of xblas.GemmF32Q4KNT / GemmQ4KF32."""
import numpy as np
import pytest
import torch

from oracle import oracle as O
from tests import util as U
from ztensor_b200 import kernels as K

pytestmark = pytest.mark.gpu


def _upload(st):
    nb = st.num_blocks()
    aos = torch.from_numpy(st.raw).cuda()
    sep = torch.empty(nb * 144, dtype=torch.uint8, device="cuda")
    K.repack_blocks144(aos, sep, nb)
    torch.cuda.synchronize()
    assert np.array_equal(sep.cpu().numpy(), st.raw_bytes_gpu())          # the split layout, byte for byte
    return sep, nb * 16


@pytest.mark.parametrize("n,k", [(64, 2048), (300, 4096), (96, 8192), (33, 14336), (16, 28672), (257, 2304)])
@pytest.mark.parametrize("batch", [1, 3])
@pytest.mark.parametrize("x_f32", [False, True])
def test_q4k_gemv(n, k, batch, x_f32):
    rng = U.seeded(n * 29 + k + batch)
    st = O.quantize_q4k(U.make_weights(rng, n, k))
    if x_f32:
        xf = rng.standard_normal((batch, k)).astype(np.float32)
        x = torch.from_numpy(xf).cuda()
    else:
        xb = U.make_x_bits(rng, batch, k)
        xf = O.f16_bits_to_f32(xb).reshape(batch, k)
        from tests import gpu_util as G
        x = G.x_dev(xb)
    ref = O.gemm_f32_q4k_nt(batch, n, k, xf, st, ncpu=1).reshape(batch, n)            # weights on B, virtual transpose
    w = st.slice().reshape(n, k)
    absd = U.absdot(w, xf)
    sep, off = _upload(st)
    y = torch.full((batch, n), float("nan"), device="cuda", dtype=torch.float32)
    fl = K.Y_F32 | (K.X_F32 if x_f32 else 0)
    K.gemv_q4k(sep, off, x, y, n, k, batch, fl)
    torch.cuda.synchronize()
    assert K.device_error() == 0
    got = y.cpu().numpy()
    assert np.isfinite(got).all()
    assert U.rel_err(got, ref, absd) <= U.REL_TOL
    if batch == 1:                                                                  # weights on A: GemmQ4KF32
        ref_a = O.gemm_q4k_f32(n, 1, k, st, xf.reshape(-1)).reshape(1, n)
        assert U.rel_err(got, ref_a, absd) <= U.REL_TOL
    again = torch.empty_like(y)
    K.gemv_q4k(sep, off, x, again, n, k, batch, fl)
    torch.cuda.synchronize()
    assert torch.equal(y, again)                                                    # fixed reduction order
    y16 = torch.empty((batch, n), device="cuda", dtype=torch.float16)
    K.gemv_q4k(sep, off, x, y16, n, k, batch, fl & ~K.Y_F32)
    torch.cuda.synchronize()
    assert U.rel_err(y16.float().cpu().numpy(), U.to_f16_round(ref), absd) <= U.REL_TOL


def test_q4k_extreme_scales_and_mins():
    """Sub-blocks 4..7 carry their two high scale / min bits in other bytes: make those bits matter."""
    n, k = 40, 2048
    rng = U.seeded(99)
    w = U.make_weights(rng, n, k).reshape(n, k // 32, 32)
    w *= rng.uniform(0.05, 4.0, (n, k // 32, 1)).astype(np.float32)                   # very uneven sub-block ranges
    w += rng.uniform(-0.2, 0.05, (n, k // 32, 1)).astype(np.float32)                  # and offsets
    st = O.quantize_q4k(w.reshape(-1))
    sc, mn = st.scales_mins(3)
    assert sc.max() > 31 or mn.max() > 31                                             # the high bits are in use
    xb = U.make_x_bits(rng, 1, k)
    xf = O.f16_bits_to_f32(xb).reshape(1, k)
    ref = O.gemm_f32_q4k_nt(1, n, k, xf, st, ncpu=1).reshape(1, n)
    from tests import gpu_util as G
    sep, off = _upload(st)
    y = torch.empty((1, n), device="cuda", dtype=torch.float32)
    K.gemv_q4k(sep, off, G.x_dev(xb), y, n, k, 1, K.Y_F32)
    torch.cuda.synchronize()
    assert U.rel_err(y.cpu().numpy(), ref, U.absdot(st.slice().reshape(n, k), xf)) <= U.REL_TOL


def test_q4k_argument_errors():
    x = torch.zeros(2048, device="cuda", dtype=torch.float16)
    y = torch.zeros(8, device="cuda", dtype=torch.float16)
    w = torch.zeros(8 * 2048 // 256 * 144, dtype=torch.uint8, device="cuda")
    with pytest.raises(RuntimeError):
        K.gemv_q4k(w, 8 * 8 * 16, x, y, 8, 1024, 1, 0)        # rows shorter than 2048
    with pytest.raises(RuntimeError):
        K.gemv_q4k(w, 8 * 8 * 16, x, y, 8, 2048 + 128, 1, 0)  # K % 256
    with pytest.raises(RuntimeError):
        K.gemv_q4k(w, 8, x, y, 8, 2048, 1, 0)                 # misaligned data offset
