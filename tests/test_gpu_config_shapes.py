"""Parity at the shapes the benchmarks run: every CTA walks many tiles.

The small-shape tests give each CTA at most one tile.  The shapes of the benchmark configurations (W4A16 g128
4096x4096; ternary 11008x4096 with row scales; Q4_0 / Q8_0 / IQ4_NL over the 8B projections at batch 1, 4, 8; the 70B
W4A16 projections at batch 1 and 8; the 8B shapes at batch 16 / 32 on the tensor cores) run the steady state of the
pipelines instead: the ring of stages wraps (the producer waits on `empty`, the phase bits flip), a team takes four
rows per stage, the overlay stages over the activation planes come into use, a CTA makes more than one pass over its
partial-sum scratch, and a tensor-core CTA loops over several work items with and without the K split.  Each test
asks the library for the launch plan of its shape (ztq_describe_plan) and asserts the property the shape is there for.

Weights are made on the device by the library's quantizers (bit-identical to the reference quantizers, see
test_gpu_parity.py) or drawn as random packed bytes, downloaded, and handed to the oracle as the same bytes.  The
kernel always runs on the whole matrix; the oracle computes every row up to 16384 rows and otherwise the first and
last 1024 rows plus every 7th row (7 is coprime to every rows-per-stage value, so every position inside a stage,
every team and every CTA is hit).
"""
import numpy as np
import pytest
import torch

from oracle import oracle as O
from tests import util as U
from ztensor_b200 import kernels as K

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _sms():
    return torch.cuda.get_device_properties(0).multi_processor_count


def _plan(fmt, n, k, batch=1):
    return K.describe_plan(fmt, n, k, batch, 128, _sms())


def _rows(n):
    if n <= 16384:
        return np.arange(n)
    return np.unique(np.concatenate([np.arange(1024), np.arange(n - 1024, n), np.arange(0, n, 7)]))


def _x(batch, k, seed):
    g = torch.Generator(device=DEV)
    g.manual_seed(seed)
    x = torch.randn(batch, k, device=DEV, generator=g).half()
    bits = x.view(torch.int16).cpu().numpy().view(np.uint16)
    return x, bits, O.f16_bits_to_f32(bits).reshape(batch, k)


def _absdot(fmt, w, meta, n, k, aux, x, rows):
    """sum_k |w[n,k] x[b,k]| for the sampled rows, on the device (the floor of the error denominators only)."""
    out = torch.empty(x.shape[0], n, dtype=torch.float32, device=DEV)
    xa = x.float().abs()
    step = 8192
    buf = torch.empty(step * k, dtype=torch.float32, device=DEV)
    for r0 in range(0, n, step):
        r1 = min(n, r0 + step)
        cnt = (r1 - r0) * k
        if fmt == K.FMT_W4G:
            K.dequantize(fmt, w[r0 * k // 2:], meta[r0 * (k // 128) * 4:], buf, cnt, 128)
        elif fmt == K.FMT_Q8_0:
            K.dequantize(fmt, w[r0 * (k // 32) * 36:], None, buf, cnt, 0)
        elif fmt == K.FMT_TERNARY:
            K.dequantize(fmt, w[r0 * k // 4:], None, buf, cnt, k)
        else:
            raise AssertionError(fmt)
        out[:, r0:r1] = xa @ buf[:cnt].view(r1 - r0, k).abs().T
    torch.cuda.synchronize()
    return out.cpu().numpy().astype(np.float64)[:, rows]


def _check(got, ref, absd, what):
    assert np.isfinite(got).all(), f"{what}: non-finite output"
    e = U.rel_err(got, ref, absd)
    assert e <= U.REL_TOL, f"{what}: max relative error {e:.3e} > {U.REL_TOL}"


def _run(fn, n, batch, y_f32=True):
    y = torch.full((batch, n), float("nan"), dtype=torch.float32 if y_f32 else torch.float16, device=DEV)
    fn(y)
    torch.cuda.synchronize()
    return y.float().cpu().numpy()


# ---------------------------------------------------------------- W4A16 (GPTQ-4 g128)

def _w4g_device(n, k, seed, awq=False):
    from ztensor_b200.stack import quantize_matrix
    qd, meta = quantize_matrix(n, k, seed, torch.device(DEV), awq=awq)
    torch.cuda.synchronize()
    return qd, meta


def _w4g_oracle_rows(qd, meta, n, k, rows, kind="gptq"):
    data = qd.view(n, k // 2)[torch.from_numpy(rows).to(DEV)].cpu().numpy()
    m = meta.view(n, (k // 128) * 4)[torch.from_numpy(rows).to(DEV)].cpu().numpy().view(np.uint16).reshape(len(rows), k // 128, 2)
    return O.GroupQuantStorage(kind, data.ravel(), np.ascontiguousarray(m[:, :, 0]).ravel(),
                               np.ascontiguousarray(m[:, :, 1]).ravel(), len(rows) * k, 128)


def _w4a16_ref(st, ns, k, x_bits):
    batch = x_bits.shape[0]
    act = O.Float16Storage(x_bits.T.copy().ravel(), batch * k)
    return np.ascontiguousarray(O.matmul_w4a16(st, (ns, k), act, (k, batch)).T)     # compute.MatMulW4A16, weights on A


# (N, K, what the shape is there for)
W4G_B1 = [
    (4096, 4096, "config 1: the reference's own CPU-runnable case"),
    (57344, 8192, "70B gate|up: four rows per team per stage, the ring of stages wraps many times"),
    (8192, 28672, "70B down: overlay stages over the activation planes, one team of 14 warps"),
    (10240, 8192, "70B QKV"),
    (8192, 8192, "70B O"),
    (28672, 4096, "8B gate|up merged"),
    (4096, 14336, "8B down: seven warps per team"),
    (6144, 4096, "8B QKV"),
]


@pytest.mark.parametrize("n,k,why", W4G_B1)
def test_w4a16_gemv_at_benchmark_shapes_batch_1(n, k, why):
    pl = _plan("w4g", n, k, 1)
    assert pl["kernel"] == "pair"
    if (n, k) == (57344, 8192):
        assert pl["rt"] == 4 and pl["tiles_per_cta"] > 4 * (pl["stages"] + pl["overlay_stages"])
    if (n, k) == (8192, 28672):
        assert pl["overlay_stages"] >= 1 and pl["tiles_per_cta"] > pl["stages"] + pl["overlay_stages"]
    qd, meta = _w4g_device(n, k, n + k)
    rows = _rows(n)
    st = _w4g_oracle_rows(qd, meta, n, k, rows)
    x, xb, xf = _x(1, k, n * 3 + k)
    ref = _w4a16_ref(st, len(rows), k, xb)
    absd = _absdot(K.FMT_W4G, qd, meta, n, k, 128, x, rows)
    got = _run(lambda y: K.gemv_w4g(qd, meta, x, y, n, k, 128, 1, K.Y_F32), n, 1)
    _check(got[:, rows], ref, absd, f"w4a16 {n}x{k}")
    assert K.device_error() == 0
    again = _run(lambda y: K.gemv_w4g(qd, meta, x, y, n, k, 128, 1, K.Y_F32), n, 1)
    assert np.array_equal(got, again)                                     # fixed reduction order, all rows
    got16 = _run(lambda y: K.gemv_w4g(qd, meta, x, y, n, k, 128, 1, 0), n, 1, y_f32=False)
    _check(got16[:, rows], U.to_f16_round(ref), absd, f"w4a16 {n}x{k} fp16 out")
    # all rows against the one-warp-per-row kernel (different code, same arithmetic identities)
    plain = _run(lambda y: K.gemv_w4g(qd, meta, x, y, n, k, 128, 1, K.Y_F32 | K.PLAIN), n, 1)
    scale = np.abs(plain).max()
    assert np.abs(got - plain).max() <= 2e-4 * scale
    if n <= 10240:
        fp = _run(lambda y: K.gemv_w4g(qd, meta, x, y, n, k, 128, 1, K.Y_F32 | K.FP32_DECODE), n, 1)
        _check(fp[:, rows], ref, absd, f"w4a16 {n}x{k} fp32 decode")


def test_w4a16_gemv_batch_2_streams_both_rows_in_one_pass():
    n, k = 57344, 8192
    pl = _plan("w4g", n, k, 2)
    assert pl["kernel"] == "stream" and pl["rows_per_launch"] == 2 and pl["tiles_per_cta"] > 2 * pl["stages"]
    qd, meta = _w4g_device(n, k, 77)
    rows = _rows(n)
    st = _w4g_oracle_rows(qd, meta, n, k, rows)
    x, xb, xf = _x(2, k, 78)
    ref = _w4a16_ref(st, len(rows), k, xb)
    absd = _absdot(K.FMT_W4G, qd, meta, n, k, 128, x, rows)
    got = _run(lambda y: K.gemv_w4g(qd, meta, x, y, n, k, 128, 2, K.Y_F32), n, 2)
    _check(got[:, rows], ref, absd, "w4a16 57344x8192 batch 2")
    assert K.device_error() == 0


def test_w4a16_gemv_makes_two_passes_over_its_partial_sum_scratch():
    """More rows per CTA than the partial-sum scratch holds: the pass loop runs twice (and the overlay stages and
    the ring wrap are in use at the same time)."""
    n, k = 45056, 28672
    pl = _plan("w4g", n, k, 1)
    assert pl["kernel"] == "pair" and pl["passes_per_cta"] >= 2 and pl["overlay_stages"] >= 1
    wb = torch.randint(0, 256, (n * k // 2,), dtype=torch.uint8, device=DEV)
    g = torch.Generator(device=DEV)
    g.manual_seed(5)
    sz = torch.stack([torch.rand(n * k // 128, device=DEV, generator=g) * 0.008 + 0.002,
                      torch.rand(n * k // 128, device=DEV, generator=g) * 2.0 + 6.5], dim=1).half()
    meta = sz.view(torch.uint8).reshape(-1)
    rows = _rows(n)
    st = _w4g_oracle_rows(wb, meta, n, k, rows)
    x, xb, xf = _x(1, k, 6)
    ref = _w4a16_ref(st, len(rows), k, xb)
    w = st.slice().reshape(len(rows), k)
    absd = np.abs(xf.astype(np.float32)) @ np.abs(w).T
    got = _run(lambda y: K.gemv_w4g(wb, meta, x, y, n, k, 128, 1, K.Y_F32), n, 1)
    _check(got[:, rows], ref, absd, "w4a16 two passes")
    assert K.device_error() == 0


@pytest.mark.parametrize("n,k", [(57344, 8192), (8192, 28672), (10240, 8192), (8192, 8192)])
def test_w4a16_tensor_core_70b_shapes_batch_8(n, k):
    pl = _plan("w4g_tc", n, k, 8)
    if (n, k) == (57344, 8192):
        assert pl["k_slices"] == 1 and pl["items_per_cta"] >= 3           # the persistent item loop, unsplit
    if (n, k) == (8192, 28672):
        assert pl["k_slices"] >= 2                                        # K split with the last-arriver reduction
    qd, meta = _w4g_device(n, k, n + k + 8)
    rows = _rows(n)
    st = _w4g_oracle_rows(qd, meta, n, k, rows)
    x, xb, xf = _x(8, k, n + 5)
    ref = _w4a16_ref(st, len(rows), k, xb)
    absd = _absdot(K.FMT_W4G, qd, meta, n, k, 128, x, rows)
    ws = torch.empty(K.gemm_w4g_tc_workspace_bytes(n, k, 8), dtype=torch.uint8, device=DEV)
    got = _run(lambda y: K.gemm_w4g_tc(qd, meta, x, y, n, k, 128, 8, ws, K.Y_F32), n, 8)
    assert K.device_error() == 0
    _check(got[:, rows], ref, absd, f"tcgen05 {n}x{k} batch 8")
    again = _run(lambda y: K.gemm_w4g_tc(qd, meta, x, y, n, k, 128, 8, ws, K.Y_F32), n, 8)
    assert np.array_equal(got, again)
    # every row against the GEMV (the same integer arithmetic on a different path)
    gemv = _run(lambda y: K.gemv_w4g(qd, meta, x, y, n, k, 128, 8, K.Y_F32), n, 8)
    assert np.abs(got - gemv).max() <= 2e-4 * np.abs(gemv).max()


TC_8B = [(6144, 4096), (4096, 4096), (14336, 4096), (4096, 14336), (28672, 4096)]


@pytest.mark.parametrize("n,k", TC_8B)
@pytest.mark.parametrize("batch", [16, 32])
@pytest.mark.parametrize("variant", ["int8", "fp16"])
def test_w4a16_tensor_core_8b_shapes(n, k, batch, variant):
    pl = _plan("w4g_tc", n, k, batch)
    if (n, k) == (28672, 4096):
        assert pl["row_tiles"] > pl["grid"] and pl["items_per_cta"] >= 2  # 224 row tiles on 148 CTAs
    if (n, k) in ((4096, 4096), (4096, 14336)):
        assert pl["k_slices"] >= 2
    vf = K.FP32_DECODE if variant == "fp16" else 0
    qd, meta = _w4g_device(n, k, n + k + batch)
    rows = _rows(n)
    st = _w4g_oracle_rows(qd, meta, n, k, rows)
    x, xb, xf = _x(batch, k, n + batch)
    ref = _w4a16_ref(st, len(rows), k, xb)
    absd = _absdot(K.FMT_W4G, qd, meta, n, k, 128, x, rows)
    ws = torch.empty(K.gemm_w4g_tc_workspace_bytes(n, k, batch), dtype=torch.uint8, device=DEV)
    got = _run(lambda y: K.gemm_w4g_tc(qd, meta, x, y, n, k, 128, batch, ws, K.Y_F32 | vf), n, batch)
    assert K.device_error() == 0
    _check(got[:, rows], ref, absd, f"tcgen05 {variant} {n}x{k} batch {batch}")
    again = _run(lambda y: K.gemm_w4g_tc(qd, meta, x, y, n, k, 128, batch, ws, K.Y_F32 | vf), n, batch)
    assert np.array_equal(got, again)


def test_w4a16_tensor_core_split_k_with_several_items_per_cta():
    n, k, batch = 12800, 28672, 16
    pl = _plan("w4g_tc", n, k, batch)
    assert pl["k_slices"] >= 2 and pl["items_per_cta"] >= 2
    qd, meta = _w4g_device(n, k, 4242)
    rows = _rows(n)
    st = _w4g_oracle_rows(qd, meta, n, k, rows)
    x, xb, xf = _x(batch, k, 4243)
    ref = _w4a16_ref(st, len(rows), k, xb)
    absd = _absdot(K.FMT_W4G, qd, meta, n, k, 128, x, rows)
    ws = torch.empty(K.gemm_w4g_tc_workspace_bytes(n, k, batch), dtype=torch.uint8, device=DEV)
    for vf in (0, K.FP32_DECODE):
        got = _run(lambda y: K.gemm_w4g_tc(qd, meta, x, y, n, k, 128, batch, ws, K.Y_F32 | vf), n, batch)
        assert K.device_error() == 0
        _check(got[:, rows], ref, absd, f"tcgen05 split-K, several items per CTA, flags {vf}")
        assert np.array_equal(got, _run(lambda y: K.gemm_w4g_tc(qd, meta, x, y, n, k, 128, batch, ws, K.Y_F32 | vf), n, batch))


def test_fused_rmsnorm_swiglu_at_the_70b_gate_up_shape():
    """RMSNorm on the way in, SwiGLU on the way out, 57344 x 8192 (gate and up rows interleaved)."""
    n, k = 57344, 8192
    qd, meta = _w4g_device(n, k, 909)
    rng = U.seeded(910)
    xh = O.f16_bits_to_f32(O.f32_to_f16_bits(rng.standard_normal(k).astype(np.float32)))
    rh = O.f16_bits_to_f32(O.f32_to_f16_bits(rng.standard_normal(k).astype(np.float32)))
    gain = rng.uniform(0.5, 1.5, k).astype(np.float32)
    normed, summed = O.fused_add_rmsnorm(xh, rh, gain, 1e-5)
    pairs = np.unique(np.concatenate([np.arange(512), np.arange(n // 2 - 512, n // 2), np.arange(0, n // 2, 7)]))
    rows = np.stack([2 * pairs, 2 * pairs + 1], axis=1).ravel()
    st = _w4g_oracle_rows(qd, meta, n, k, rows)
    w = st.slice().reshape(len(rows), k)
    lin = U.ref_dense_a_side(w, normed.reshape(1, k), len(rows), k).reshape(-1)       # CPU-engine MatMul of the normed vector
    ref = O.fused_swiglu(lin[0::2], lin[1::2])
    xd = torch.from_numpy(xh).to(DEV).half()
    rd = torch.from_numpy(rh).to(DEV).half()
    gd = torch.from_numpy(gain).to(DEV)
    sd = torch.full((k,), float("nan"), device=DEV, dtype=torch.float16)
    y = torch.full((n // 2,), float("nan"), device=DEV, dtype=torch.float32)
    K.gemv_w4g_fused(qd, meta, xd, y, n, k, 128, K.Y_F32, norm_weight=gd, eps=1e-5, residual=rd, sum_out=sd, swiglu=True)
    torch.cuda.synchronize()
    assert K.device_error() == 0
    got = y.cpu().numpy()
    assert np.isfinite(got).all()
    g, u = lin[0::2], lin[1::2]
    bound = U.REL_TOL * (np.abs(ref) + 1e-3 * (np.abs(u) + np.abs(g) * np.abs(u) + 1.0)) * 4 + 1e-6
    assert (np.abs(got[pairs] - ref) <= bound).all()
    assert np.array_equal(sd.float().cpu().numpy(), O.f16_bits_to_f32(O.f32_to_f16_bits(summed)))
    # norm alone, all sampled rows against the plain linear outputs
    y2 = torch.full((n,), float("nan"), device=DEV, dtype=torch.float32)
    K.gemv_w4g_fused(qd, meta, xd, y2, n, k, 128, K.Y_F32, norm_weight=gd, eps=1e-5, residual=rd)
    torch.cuda.synchronize()
    absd = np.abs(normed.reshape(1, k)) @ np.abs(w).T
    _check(y2.cpu().numpy()[rows].reshape(1, -1), lin.reshape(1, -1), absd, "rmsnorm folded in, 57344x8192")


# ---------------------------------------------------------------- ternary with row scales (config 2)

def test_ternary_gemv_config_shape_with_row_scales():
    n, k = 11008, 4096
    pl = _plan("ternary", n, k, 1)
    assert pl["kernel"] == "stream" and pl["tiles_per_cta"] >= 2
    g = torch.Generator(device=DEV)
    g.manual_seed(11)
    codes = torch.randint(0, 3, (n * k,), device=DEV, generator=g, dtype=torch.int32)      # 0,1,2 = -1,0,+1
    c4 = codes.view(-1, 4)
    packed = (c4[:, 0] | (c4[:, 1] << 2) | (c4[:, 2] << 4) | (c4[:, 3] << 6)).to(torch.uint8)
    st = O.TernaryStorage(packed.cpu().numpy(), n * k)                                        # tensor/ternary_storage.go layout
    rng = U.seeded(12)
    scale_bits = O.f32_to_f16_bits(rng.uniform(0.01, 0.05, n).astype(np.float32))
    x, xb, xf = _x(1, k, 13)
    ref = U.ref_ternary(st, xf, scale_bits, n, k)
    rows = np.arange(n)
    sc = torch.from_numpy(scale_bits.view(np.int16)).to(DEV)
    absd = _absdot(K.FMT_TERNARY, packed, None, n, k, k, x, rows) * O.f16_bits_to_f32(scale_bits)[None, :]
    from tests import gpu_util as G
    wrows = G.upload_ternary(st, n, k)
    got = _run(lambda y: K.gemv_ternary(wrows, sc, x, y, n, k, 1, K.Y_F32), n, 1)
    _check(got, ref, absd, "ternary 11008x4096 with row scales")
    got16 = _run(lambda y: K.gemv_ternary(wrows, sc, x, y, n, k, 1, 0), n, 1, y_f32=False)
    _check(got16, U.to_f16_round(ref), absd, "ternary fp16 out")
    assert np.array_equal(got, _run(lambda y: K.gemv_ternary(wrows, sc, x, y, n, k, 1, K.Y_F32), n, 1))
    # the reference-named launcher (float32 in and out, no row scale), exact against TernaryGEMV
    x32 = x.float().reshape(-1)
    y = torch.full((n,), float("nan"), dtype=torch.float32, device=DEV)
    K.ternary_gemv_f32(wrows, x32, y, n, k)
    torch.cuda.synchronize()
    ref0 = O.ternary_gemv(st, xf[0], n, k)
    _check(y.cpu().numpy().reshape(1, n), ref0.reshape(1, n), absd / O.f16_bits_to_f32(scale_bits)[None, :], "ternary_gemv_f32")
    assert K.device_error() == 0


# ---------------------------------------------------------------- block formats over the 8B projections (config 3)

SHAPES_8B = [(6144, 4096), (4096, 4096), (14336, 4096), (4096, 14336)]


def _blocks18_to_aos(sep, nblk, off):
    h = sep.cpu().numpy()
    aos = np.empty((nblk, 18), np.uint8)
    aos[:, :2] = h[: nblk * 2].reshape(nblk, 2)
    aos[:, 2:] = h[off: off + nblk * 16].reshape(nblk, 16)
    return aos.ravel()


@pytest.mark.parametrize("n,k", SHAPES_8B)
def test_q4_0_gemv_8b_shapes_batch_1_4_8(n, k):
    pl = _plan("q4_0", n, k, 1)
    assert pl["kernel"] == "pair"
    if (n, k) in ((14336, 4096), (4096, 14336)):
        assert pl["tiles_per_cta"] > pl["stages"] + pl["overlay_stages"]      # the ring wraps
    g = torch.Generator(device=DEV)
    g.manual_seed(n + k)
    w = torch.empty(n * k, device=DEV).normal_(0.0, 0.02, generator=g)
    nblk = n * k // 32
    off = K.q4_gpu_data_offset(nblk)
    sep = torch.zeros(off + nblk * 16, dtype=torch.uint8, device=DEV)
    K.quantize_q4_0(w, sep, n * k)
    torch.cuda.synchronize()
    st = O.Q4Storage(_blocks18_to_aos(sep, nblk, off), n * k)
    wd = st.slice().reshape(n, k)
    for batch in (1, 4, 8):
        x, xb, xf = _x(batch, k, n + batch)
        ref = U.ref_q4_0(st, xf, n, k)                                     # CPUEngine.MatMul -> GemmF32Q4NT
        absd = np.abs(xf) @ np.abs(wd).T
        got = _run(lambda y: K.gemv_q4_0(sep, off, x, y, n, k, batch, K.Y_F32), n, batch)
        _check(got, ref, absd, f"q4_0 {n}x{k} batch {batch}")
        assert np.array_equal(got, _run(lambda y: K.gemv_q4_0(sep, off, x, y, n, k, batch, K.Y_F32), n, batch))
        if batch >= 3:                                                     # what the engine takes from three rows on
            ws = torch.empty(K.gemm_q4_0_tc_workspace_bytes(n, k, batch), dtype=torch.uint8, device=DEV)
            tc = _run(lambda y: K.gemm_q4_0_tc(sep, off, x, y, n, k, batch, ws, K.Y_F32), n, batch)
            _check(tc, ref, absd, f"q4_0 tcgen05 {n}x{k} batch {batch}")
            assert np.array_equal(tc, _run(lambda y: K.gemm_q4_0_tc(sep, off, x, y, n, k, batch, ws, K.Y_F32), n, batch))
    # the reference's own launcher name: weights on A, float32 activations [K, batch], outputs [N, batch]
    xkb = torch.randn(k, 4, device=DEV, generator=g)
    c = torch.full((n, 4), float("nan"), device=DEV)
    K.gemm_q4_f32(sep, xkb, c, n, k, 4, off)
    torch.cuda.synchronize()
    xh = xkb.cpu().numpy()
    ref = O.cpu_engine_matmul(st, (n, k), xh, (k, 4))                      # A-side: GemmQ4F32
    _check(c.cpu().numpy().T, ref.T, np.abs(xh.T) @ np.abs(wd).T, f"gemm_q4_f32 {n}x{k}x4")
    assert K.device_error() == 0


@pytest.mark.parametrize("n,k", SHAPES_8B)
def test_q8_0_gemv_8b_shapes_batch_1_4_8(n, k):
    pl = _plan("q8_0", n, k, 1)
    assert pl["kernel"] == "stream" and pl["tiles_per_cta"] >= 2
    g = torch.Generator(device=DEV)
    g.manual_seed(n + 3 * k)
    w = torch.empty(n * k, device=DEV).normal_(0.0, 0.02, generator=g)
    blocks = torch.zeros(n * k // 32 * 36, dtype=torch.uint8, device=DEV)
    K.quantize_q8_0(w, blocks, n * k)
    torch.cuda.synchronize()
    st = O.Q8Storage(blocks.cpu().numpy(), n * k)
    wd = st.slice().reshape(n, k)
    for batch in (1, 4, 8):
        x, xb, xf = _x(batch, k, n + batch + 1)
        ref = U.ref_q8_0(st, xf, n, k)
        absd = np.abs(xf) @ np.abs(wd).T
        got = _run(lambda y: K.gemv_q8_0(blocks, x, y, n, k, batch, K.Y_F32), n, batch)
        _check(got, ref, absd, f"q8_0 {n}x{k} batch {batch}")
        assert np.array_equal(got, _run(lambda y: K.gemv_q8_0(blocks, x, y, n, k, batch, K.Y_F32), n, batch))
        if batch >= 3:                                  # the path the engine takes from three rows on: tensor cores
            ws = torch.empty(K.gemm_q8_0_tc_workspace_bytes(n, k, batch), dtype=torch.uint8, device=DEV)
            tc = _run(lambda y: K.gemm_q8_0_tc(blocks, x, y, n, k, batch, ws, K.Y_F32), n, batch)
            _check(tc, ref, absd, f"q8_0 tcgen05 {n}x{k} batch {batch}")
            assert np.array_equal(tc, _run(lambda y: K.gemm_q8_0_tc(blocks, x, y, n, k, batch, ws, K.Y_F32), n, batch))
    assert K.device_error() == 0


@pytest.mark.parametrize("n,k", SHAPES_8B)
def test_iq4nl_gemv_8b_shapes_batch_1_4_8(n, k):
    """The reference has no IQ4_NL quantizer: blocks are random codes with fp16 scales, the same bytes on both sides."""
    pl = _plan("iq4nl", n, k, 1)
    assert pl["kernel"] == "stream" and pl["tiles_per_cta"] >= 2
    nblk = n * k // 32
    off = K.q4_gpu_data_offset(nblk)
    g = torch.Generator(device=DEV)
    g.manual_seed(n + 5 * k)
    sep = torch.randint(0, 256, (off + nblk * 16,), dtype=torch.uint8, device=DEV, generator=g)
    sep[: nblk * 2] = (torch.rand(nblk, device=DEV, generator=g) * 0.02 + 0.005).half().view(torch.uint8).reshape(-1)
    st = O.new_iq4nl_from_raw(_blocks18_to_aos(sep, nblk, off), n * k)
    wd = st.slice().reshape(n, k)
    for batch in (1, 4, 8):
        x, xb, xf = _x(batch, k, n + batch + 2)
        ref = U.ref_dense_a_side(wd, xf, n, k)                             # no IQ4_NL dispatch: Slice() + SgemmSimd
        absd = np.abs(xf) @ np.abs(wd).T
        got = _run(lambda y: K.gemv_iq4nl(sep, off, x, y, n, k, batch, K.Y_F32), n, batch)
        _check(got, ref, absd, f"iq4_nl {n}x{k} batch {batch}")
    assert K.device_error() == 0


def test_streaming_kernel_makes_two_passes_over_its_partial_sum_scratch():
    """Q8_0 with enough rows per CTA that the streaming kernel's pass loop runs more than once."""
    n, k = 245760, 8192
    pl = _plan("q8_0", n, k, 1)
    assert pl["kernel"] == "stream" and pl["passes_per_cta"] >= 2
    g = torch.Generator(device=DEV)
    g.manual_seed(31)
    nblk = n * k // 32
    blocks = torch.randint(0, 256, (nblk, 36), dtype=torch.uint8, device=DEV, generator=g)
    blocks[:, :4] = (torch.rand(nblk, 1, device=DEV, generator=g) * 0.001 + 0.0002).float().view(torch.uint8).reshape(-1, 4)
    blocks = blocks.reshape(-1)
    rows = _rows(n)
    sub = blocks.view(n, (k // 32) * 36)[torch.from_numpy(rows).to(DEV)].cpu().numpy()
    st = O.Q8Storage(sub.ravel(), len(rows) * k)
    x, xb, xf = _x(1, k, 32)
    ref = U.ref_q8_0(st, xf, len(rows), k)
    absd = np.abs(xf) @ np.abs(st.slice().reshape(len(rows), k)).T
    got = _run(lambda y: K.gemv_q8_0(blocks, x, y, n, k, 1, K.Y_F32), n, 1)
    _check(got[:, rows], ref, absd, "q8_0 two passes")
    assert K.device_error() == 0


# ---------------------------------------------------------------- a K-quant at the 70B gate|up shape

def test_q4k_gemv_at_the_70b_gate_up_shape():
    n, k = 57344, 8192
    pl = _plan("q4_k", n, k, 1)
    assert pl["rt"] == 4 and pl["tiles_per_cta"] > pl["stages"]
    rows = _rows(n)
    # quantize the sampled rows with the oracle's Q4_K quantizer, fill the rest with random super-blocks
    rng = U.seeded(404)
    sub = O.quantize_q4k(U.make_weights(rng, len(rows), k))
    nb_row = k // 256
    g = torch.Generator(device=DEV)
    g.manual_seed(405)
    aos = torch.randint(0, 256, (n, nb_row, 144), dtype=torch.uint8, device=DEV, generator=g)
    aos[:, :, :4] = (torch.rand(n, nb_row, 2, device=DEV, generator=g) * 0.001).half().view(torch.uint8).reshape(n, nb_row, 4)
    aos[torch.from_numpy(rows).to(DEV)] = torch.from_numpy(sub.raw.reshape(len(rows), nb_row, 144)).to(DEV)
    nb = n * nb_row
    sep = torch.empty(nb * 144, dtype=torch.uint8, device=DEV)
    K.repack_blocks144(aos.reshape(-1), sep, nb)
    x, xb, xf = _x(1, k, 406)
    ref = O.gemm_f32_q4k_nt(1, len(rows), k, xf, sub, ncpu=1).reshape(1, -1)
    absd = np.abs(xf) @ np.abs(sub.slice().reshape(len(rows), k)).T
    got = _run(lambda y: K.gemv_q4k(sep, nb * 16, x, y, n, k, 1, K.Y_F32), n, 1)
    assert np.isfinite(got).all()
    _check(got[:, rows], ref, absd, "q4_k 57344x8192")
    assert K.device_error() == 0
