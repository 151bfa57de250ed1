"""RMSNorm folded into the GEMV's activation load and SwiGLU into its output store, against the oracle's
restatement of the reference's separate steps (fused_add_rmsnorm.cu, MatMul on the CPU engine, fused_swiglu.cu)."""
import numpy as np
import pytest
import torch

from oracle import oracle as O
from tests import util as U
from ztensor_b200 import kernels as K

pytestmark = pytest.mark.gpu


def _case(n, k, seed):
    from tests import gpu_util as G
    rng = U.seeded(seed)
    st = O.quantize_gptq(U.make_weights(rng, n, k), 128, 4)
    qd, meta = G.upload_w4g(st)
    w = st.slice().reshape(n, k)
    x = rng.standard_normal(k).astype(np.float32)
    res = rng.standard_normal(k).astype(np.float32)
    gain = rng.uniform(0.5, 1.5, k).astype(np.float32)
    return st, qd, meta, w, x, res, gain


@pytest.mark.parametrize("n,k", [(300, 4096), (64, 2048), (96, 8192), (40, 14336)])
@pytest.mark.parametrize("x_f32", [True, False])
@pytest.mark.parametrize("with_residual", [True, False])
def test_rmsnorm_folded_into_gemv(n, k, x_f32, with_residual):
    st, qd, meta, w, x, res, gain = _case(n, k, n + k)
    if not x_f32:                                              # fp16 stream: the values the kernel sees
        x = O.f16_bits_to_f32(O.f32_to_f16_bits(x))
        res = O.f16_bits_to_f32(O.f32_to_f16_bits(res))
    eps = 1e-5
    normed, summed = O.fused_add_rmsnorm(x, res if with_residual else None, gain, eps)
    ref = U.ref_dense_a_side(w, normed.reshape(1, k), n, k)                      # MatMul on the CPU engine
    absd = U.absdot(w, normed.reshape(1, k))
    dt = torch.float32 if x_f32 else torch.float16
    xd = torch.from_numpy(x).cuda().to(dt)
    rd = torch.from_numpy(res).cuda().to(dt) if with_residual else None
    gd = torch.from_numpy(gain).cuda()
    sd = torch.full((k,), float("nan"), device="cuda", dtype=dt)
    y = torch.full((n,), float("nan"), device="cuda", dtype=torch.float32)
    fl = K.Y_F32 | (K.X_F32 if x_f32 else 0)
    K.gemv_w4g_fused(qd, meta, xd, y, n, k, 128, fl, norm_weight=gd, eps=eps, residual=rd, sum_out=sd)
    torch.cuda.synchronize()
    assert K.device_error() == 0
    got = y.cpu().numpy().reshape(1, n)
    assert U.rel_err(got, ref, absd) <= U.REL_TOL
    want_sum = summed if x_f32 else O.f16_bits_to_f32(O.f32_to_f16_bits(summed))
    assert np.array_equal(sd.float().cpu().numpy(), want_sum)                    # x + residual: exact
    again = torch.empty_like(y)
    K.gemv_w4g_fused(qd, meta, xd, again, n, k, 128, fl, norm_weight=gd, eps=eps, residual=rd)
    torch.cuda.synchronize()
    assert torch.equal(y, again)                                                 # fixed reduction order


@pytest.mark.parametrize("f,k", [(512, 4096), (150, 2048), (37, 8192)])
def test_swiglu_folded_into_gemv(f, k):
    """gate and up interleaved row by row; the fused store equals fused_swiglu of the unfused outputs."""
    from tests import gpu_util as G
    rng = U.seeded(f * 3 + k)
    sg = O.quantize_gptq(U.make_weights(rng, f, k), 128, 4)
    su = O.quantize_gptq(U.make_weights(rng, f, k), 128, 4)
    gq, gm = G.upload_w4g(sg)
    uq, um = G.upload_w4g(su)
    pq = torch.empty(2 * f * k // 2, dtype=torch.uint8, device="cuda")
    pm = torch.empty(2 * f * (k // 128) * 4, dtype=torch.uint8, device="cuda")
    K.interleave_rows(gq, uq, pq, f, k // 2)
    K.interleave_rows(gm, um, pm, f, (k // 128) * 4)
    xb = U.make_x_bits(rng, 1, k)
    x = G.x_dev(xb).reshape(-1)
    g = torch.empty(f, device="cuda", dtype=torch.float32)
    u = torch.empty(f, device="cuda", dtype=torch.float32)
    K.gemv_w4g(gq, gm, x, g, f, k, 128, 1, K.Y_F32)
    K.gemv_w4g(uq, um, x, u, f, k, 128, 1, K.Y_F32)
    both = torch.empty(2 * f, device="cuda", dtype=torch.float32)
    K.gemv_w4g(pq, pm, x, both, 2 * f, k, 128, 1, K.Y_F32)                       # the pair layout, unfused
    y = torch.full((f,), float("nan"), device="cuda", dtype=torch.float32)
    K.gemv_w4g_fused(pq, pm, x, y, 2 * f, k, 128, K.Y_F32, swiglu=True)
    torch.cuda.synchronize()
    assert K.device_error() == 0
    assert torch.equal(both[0::2], g) and torch.equal(both[1::2], u)             # interleaving moved whole rows
    want = O.fused_swiglu(g.cpu().numpy(), u.cpu().numpy())
    got = y.cpu().numpy()
    assert np.isfinite(got).all()
    assert np.abs(got - want).max() <= 1e-5 * max(1.0, np.abs(want).max())       # expf of the device vs libm
    # and against the reference path end to end
    xf = O.f16_bits_to_f32(xb).reshape(1, k)
    rg = U.ref_dense_a_side(sg.slice().reshape(f, k), xf, f, k).reshape(-1)
    ru = U.ref_dense_a_side(su.slice().reshape(f, k), xf, f, k).reshape(-1)
    ref = O.fused_swiglu(rg, ru)
    bound = U.REL_TOL * (np.abs(ref) + 1e-3 * (np.abs(ru) + np.abs(rg) * np.abs(ru) + 1.0)) * 4 + 1e-6
    assert (np.abs(got - ref) <= bound).all()


def test_fused_argument_errors():
    from ztensor_b200 import _lib
    x = torch.zeros(4096, device="cuda", dtype=torch.float16)
    y = torch.zeros(64, device="cuda", dtype=torch.float16)
    w = torch.zeros(64 * 4096 // 2, dtype=torch.uint8, device="cuda")
    m = torch.zeros(64 * 32 * 4, dtype=torch.uint8, device="cuda")
    with pytest.raises(RuntimeError):
        K.gemv_w4g_fused(w, m, x, y, 63, 4096, 128, 0, swiglu=True)              # odd number of rows
    with pytest.raises(RuntimeError):
        K.gemv_w4g_fused(w, m, x, y, 64, 4096, 64, 0, swiglu=True)               # group 128 only
    with pytest.raises(RuntimeError):
        K.gemv_w4g_fused(w, m, x, y, 64, 4096, 128, 0, residual=x)               # residual without a norm
    g = torch.ones(4096, device="cuda")
    with pytest.raises(RuntimeError):
        K.gemv_w4g_fused(w, m, x, y, 64, 4096, 128, 0, norm_weight=g, sum_out=x)  # sum_out aliases x
