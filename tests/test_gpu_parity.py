"""CUDA kernels vs the CPU oracle, through the C-ABI.  Needs a B200."""
import numpy as np
import pytest
import torch

from oracle import oracle as O
from tests import util as U
from ztensor_b200 import kernels as K

pytestmark = pytest.mark.gpu

# (N, K): streaming-kernel shapes (K multiple of 512) and plain-kernel shapes
SHAPES = [(64, 512), (96, 1024), (257, 4096), (40, 3584), (48, 8192), (33, 14336), (16, 28672),
          (50, 32), (37, 96), (20, 640), (8, 160)]
BATCHES = [1, 2, 3, 4, 8]


def _gpu():
    from tests import gpu_util as G
    return G


def _check(got, ref, absd, what):
    e = U.rel_err(got, ref, absd)
    assert np.isfinite(got).all(), f"{what}: non-finite output"
    assert e <= U.REL_TOL, f"{what}: max relative error {e:.3e} > {U.REL_TOL}"
    return e


@pytest.mark.parametrize("n,k", SHAPES)
@pytest.mark.parametrize("batch", BATCHES)
def test_q4_0_gemv(n, k, batch):
    G = _gpu()
    rng = U.seeded(n * 7 + k + batch)
    st = O.quantize_q4(U.make_weights(rng, n, k))
    xb = U.make_x_bits(rng, batch, k)
    xf = O.f16_bits_to_f32(xb).reshape(batch, k)
    ref = U.ref_q4_0(st, xf, n, k)
    absd = U.absdot(st.slice().reshape(n, k), xf)
    sep, off = G.upload_blocks18(st.blocks, st.num_blocks())
    assert np.array_equal(sep.cpu().numpy(), st.raw_bytes_gpu())          # repack == RawBytesGPU, bit for bit
    x = G.x_dev(xb)
    got32 = G.run(lambda y: K.gemv_q4_0(sep, off, x, y, n, k, batch, K.Y_F32), n, batch)
    _check(got32, ref, absd, "q4_0 f32 out")
    got16 = G.run(lambda y: K.gemv_q4_0(sep, off, x, y, n, k, batch, 0), n, batch, y_f32=False)
    _check(got16, U.to_f16_round(ref), absd, "q4_0 f16 out")
    again = G.run(lambda y: K.gemv_q4_0(sep, off, x, y, n, k, batch, K.Y_F32), n, batch)
    assert np.array_equal(got32, again)                                   # fixed reduction order
    plain = G.run(lambda y: K.gemv_q4_0(sep, off, x, y, n, k, batch, K.Y_F32 | K.PLAIN), n, batch)
    _check(plain, ref, absd, "q4_0 plain kernel")
    fp = G.run(lambda y: K.gemv_q4_0(sep, off, x, y, n, k, batch, K.Y_F32 | K.FP32_DECODE), n, batch)
    _check(fp, ref, absd, "q4_0 fp32-decode kernel")


@pytest.mark.parametrize("n,k", SHAPES)
@pytest.mark.parametrize("batch", [1, 2, 4])
def test_iq4nl_gemv(n, k, batch):
    G = _gpu()
    rng = U.seeded(n * 11 + k + batch)
    st = O.make_iq4nl_blocks(U.make_weights(rng, n, k))
    xb = U.make_x_bits(rng, batch, k)
    xf = O.f16_bits_to_f32(xb).reshape(batch, k)
    w = st.slice().reshape(n, k)
    ref = U.ref_dense_a_side(w, xf, n, k)          # no IQ4_NL case in tryQuantizedMatMul: Slice() + SgemmSimd
    absd = U.absdot(w, xf)
    sep, off = G.upload_blocks18(st.raw, st.num_blocks())
    x = G.x_dev(xb)
    got = G.run(lambda y: K.gemv_iq4nl(sep, off, x, y, n, k, batch, K.Y_F32), n, batch)
    _check(got, ref, absd, "iq4_nl")
    plain = G.run(lambda y: K.gemv_iq4nl(sep, off, x, y, n, k, batch, K.Y_F32 | K.PLAIN), n, batch)
    _check(plain, ref, absd, "iq4_nl plain")


@pytest.mark.parametrize("n,k", SHAPES)
@pytest.mark.parametrize("batch", BATCHES)
def test_q8_0_gemv(n, k, batch):
    G = _gpu()
    rng = U.seeded(n * 13 + k + batch)
    st = O.quantize_q8(U.make_weights(rng, n, k))
    xb = U.make_x_bits(rng, batch, k)
    xf = O.f16_bits_to_f32(xb).reshape(batch, k)
    ref = U.ref_q8_0(st, xf, n, k)
    absd = U.absdot(st.slice().reshape(n, k), xf)
    w = G.dev_u8(st.blocks)
    x = G.x_dev(xb)
    got = G.run(lambda y: K.gemv_q8_0(w, x, y, n, k, batch, K.Y_F32), n, batch)
    _check(got, ref, absd, "q8_0")
    got16 = G.run(lambda y: K.gemv_q8_0(w, x, y, n, k, batch, 0), n, batch, y_f32=False)
    _check(got16, U.to_f16_round(ref), absd, "q8_0 f16 out")
    plain = G.run(lambda y: K.gemv_q8_0(w, x, y, n, k, batch, K.Y_F32 | K.PLAIN), n, batch)
    _check(plain, ref, absd, "q8_0 plain")
    fp = G.run(lambda y: K.gemv_q8_0(w, x, y, n, k, batch, K.Y_F32 | K.FP32_DECODE), n, batch)
    _check(fp, ref, absd, "q8_0 fp32-decode kernel")


@pytest.mark.parametrize("kind", ["gptq", "awq"])
@pytest.mark.parametrize("n,k", [s for s in SHAPES if s[1] % 128 == 0])
@pytest.mark.parametrize("batch", BATCHES)
def test_w4a16_gemv(kind, n, k, batch):
    G = _gpu()
    rng = U.seeded(n * 17 + k + batch)
    wf = U.make_weights(rng, n, k)
    st = O.quantize_gptq(wf, 128, 4) if kind == "gptq" else O.quantize_awq(wf, 128)
    xb = U.make_x_bits(rng, batch, k)
    act = O.Float16Storage(xb.T.copy().ravel(), batch * k)          # B = activations [K, batch]
    ref = np.ascontiguousarray(O.matmul_w4a16(st, (n, k), act, (k, batch)).T)   # MatMulW4A16, weights on A
    xf = O.f16_bits_to_f32(xb).reshape(batch, k)
    absd = U.absdot(st.slice().reshape(n, k), xf)
    qd, meta = G.upload_w4g(st)
    x = G.x_dev(xb)
    got = G.run(lambda y: K.gemv_w4g(qd, meta, x, y, n, k, 128, batch, K.Y_F32), n, batch)
    _check(got, ref, absd, f"{kind} f32 out")
    got16 = G.run(lambda y: K.gemv_w4g(qd, meta, x, y, n, k, 128, batch, 0), n, batch, y_f32=False)
    _check(got16, U.to_f16_round(ref), absd, f"{kind} f16 out")
    again = G.run(lambda y: K.gemv_w4g(qd, meta, x, y, n, k, 128, batch, K.Y_F32), n, batch)
    assert np.array_equal(got, again)
    plain = G.run(lambda y: K.gemv_w4g(qd, meta, x, y, n, k, 128, batch, K.Y_F32 | K.PLAIN), n, batch)
    _check(plain, ref, absd, f"{kind} plain")
    fp = G.run(lambda y: K.gemv_w4g(qd, meta, x, y, n, k, 128, batch, K.Y_F32 | K.FP32_DECODE), n, batch)
    _check(fp, ref, absd, f"{kind} fp32-decode kernel")


@pytest.mark.parametrize("group", [32, 64, 256])
@pytest.mark.parametrize("n,k", [(40, 512), (24, 4096), (8, 96 * 4 // 3 * 2)])
def test_w4g_other_group_sizes(group, n, k):
    """QuantizeGPTQ(., 32, 4) as in compute/w4a16_test.go:60-68: groups of any power of two >= 32."""
    G = _gpu()
    if k % group:
        pytest.skip("K not a multiple of the group")
    rng = U.seeded(n + k + group)
    st = O.quantize_gptq(U.make_weights(rng, n, k), group, 4)
    xb = U.make_x_bits(rng, 2, k)
    xf = O.f16_bits_to_f32(xb).reshape(2, k)
    ref = U.ref_dense_a_side(st.slice().reshape(n, k), xf, n, k)
    absd = U.absdot(st.slice().reshape(n, k), xf)
    qd, meta = G.upload_w4g(st)
    x = G.x_dev(xb)
    for fl in (0, K.PLAIN, K.FP32_DECODE):
        got = G.run(lambda y: K.gemv_w4g(qd, meta, x, y, n, k, group, 2, K.Y_F32 | fl), n, 2)
        _check(got, ref, absd, f"w4g group {group} flags {fl}")


@pytest.mark.parametrize("n,k", [(64, 512), (300, 4096), (11, 2048), (40, 64), (9, 11008 // 64 * 64)])
@pytest.mark.parametrize("batch", [1, 2, 5])
@pytest.mark.parametrize("scaled", [False, True])
def test_ternary_gemv(n, k, batch, scaled):
    G = _gpu()
    rng = U.seeded(n * 19 + k + batch)
    st = O.new_ternary_from(rng.integers(-1, 2, size=n * k).astype(np.int8))
    scale_bits = O.f32_to_f16_bits(rng.uniform(0.01, 0.05, n).astype(np.float32)) if scaled else None
    xb = U.make_x_bits(rng, batch, k)
    xf = O.f16_bits_to_f32(xb).reshape(batch, k)
    ref = U.ref_ternary(st, xf, scale_bits, n, k)
    w = st.slice().reshape(n, k)
    if scaled:
        w = w * O.f16_bits_to_f32(scale_bits)[:, None]
    absd = U.absdot(w, xf)
    rows = G.upload_ternary(st, n, k)
    assert np.array_equal(rows.cpu().numpy(), st.data)                    # K % 4 == 0: flat == row-aligned
    sc = G.dev_u8(scale_bits) if scaled else None
    x = G.x_dev(xb)
    got = G.run(lambda y: K.gemv_ternary(rows, sc, x, y, n, k, batch, K.Y_F32), n, batch)
    _check(got, ref, absd, "ternary")
    plain = G.run(lambda y: K.gemv_ternary(rows, sc, x, y, n, k, batch, K.Y_F32 | K.PLAIN), n, batch)
    _check(plain, ref, absd, "ternary plain")
    fp = G.run(lambda y: K.gemv_ternary(rows, sc, x, y, n, k, batch, K.Y_F32 | K.FP32_DECODE), n, batch)
    _check(fp, ref, absd, "ternary fp32-decode kernel")


# ---------------- the reference's own launcher names and known answers ----------------

def test_ternary_gemv_f32_known_answers():
    """compute/ternary_gemv_test.go:25-141 through ternary_gemv_f32 (rows of any length)."""
    G = _gpu()
    cases = [
        ([1, 0, -1, 1, -1, 1, 0, 0, 0, -1, 1, -1], [2.0, 3.0, 4.0, 5.0], 3, 4, [3.0, 1.0, -4.0]),
        ([1, -1, 0, 1, -1, 0, 1, -1, 0, 1], [1.0, 2.0, 3.0, 4.0, 5.0], 2, 5, [-2.0, 4.0]),
        ([-1], [7.5], 1, 1, [-7.5]), ([0], [7.5], 1, 1, [0.0]), ([1], [7.5], 1, 1, [7.5]),
    ]
    n = 33
    ident = np.zeros((n, n), np.int8)
    ident[np.arange(n), np.arange(n)] = 1
    xi = (np.arange(n, dtype=np.float32) * 0.5 - 8.0)
    cases.append((ident.ravel().tolist(), xi.tolist(), n, n, xi.tolist()))
    cases.append((np.zeros(16 * 32, np.int8).tolist(), list(range(1, 33)), 16, 32, [0.0] * 16))
    for vals, x, m, k, want in cases:
        st = O.new_ternary_from(vals)
        rows = G.upload_ternary(st, m, k)
        xd = torch.tensor(x, dtype=torch.float32, device="cuda")
        y = torch.full((m,), float("nan"), dtype=torch.float32, device="cuda")
        K.ternary_gemv_f32(rows, xd, y, m, k)
        torch.cuda.synchronize()
        assert y.cpu().tolist() == want, (m, k)
        assert np.array_equal(y.cpu().numpy(), O.ternary_gemv(st, x, m, k))


@pytest.mark.parametrize("m,k,n", [(64, 512, 1), (130, 4096, 1), (48, 1024, 3), (17, 96, 1), (32, 4096, 8)])
def test_gemm_q4_f32_and_q8_f32_reference_signatures(m, k, n):
    """gemm_q4_f32 / gemm_q8_f32 as GPUEngine.matMulQ4 / matMulQ8 call them: A = weights [M,K],
    B = activations [K,N] float32, C [M,N] float32; inputs as in gemm_q4_test.go (modular fills)."""
    G = _gpu()
    a = ((np.arange(m * k) % 7 - 3) * np.float32(0.1)).astype(np.float32)
    b = ((np.arange(k * n) % 5 - 2) * np.float32(0.1)).astype(np.float32)
    bd = torch.from_numpy(b).cuda()
    for st, call in ((O.quantize_q4(a), "q4"), (O.quantize_q8(a), "q8")):
        ref = O.cpu_engine_matmul(st, (m, k), b, (k, n))                 # A-side quantized: GemmQ4F32 / GemmQ8F32
        absd = U.absdot(st.slice().reshape(m, k), b.reshape(k, n).T).T
        c = torch.full((m, n), float("nan"), dtype=torch.float32, device="cuda")
        if call == "q4":
            sep, off = G.upload_blocks18(st.blocks, st.num_blocks())
            K.gemm_q4_f32(sep, bd, c, m, k, n, off)
        else:
            K.gemm_q8_f32(G.dev_u8(st.blocks), bd, c, m, k, n)
        torch.cuda.synchronize()
        got = c.cpu().numpy()
        assert U.rel_err(got, ref, absd) <= U.REL_TOL
        dense = a.reshape(m, k).astype(np.float64) @ b.reshape(k, n).astype(np.float64)
        assert np.abs(got - dense).max() <= (0.15 if call == "q4" else 0.02) * max(1, k / 32)   # the reference test's own bound


def test_argument_errors_return_cuda_invalid_value():
    from ztensor_b200 import _lib
    L = _lib.lib()
    d = torch.zeros(4096, dtype=torch.uint8, device="cuda")
    p = d.data_ptr()
    assert L.gemm_q4_f32(p, p, p, 4, 33, 1, 16, None) == 1          # K % 32 (gemm_q4.cu:169-171)
    assert L.gemm_q8_f32(p, p, p, 4, 40, 1, None) == 1
    assert L.ztq_gemv_w4g(p, p, p, p, 4, 128, 48, 1, 0, None) == 1  # group size not 32 * 2^s
    assert L.ztq_gemv_w4g(p, None, p, p, 4, 128, 128, 1, 0, None) == 1
    assert L.ztq_gemv_q4_0(p, 8, p, p, 4, 32, 1, 0, None) == 1      # data offset not 16-aligned
    assert L.ztq_gemv_q4_0(p, 16, p, p, 0, 32, 1, 0, None) == 1
    assert L.ternary_gemv_f32(None, p, p, 1, 1, None) == 1
    assert L.ztq_quantize_q4_0(p, p, 33, None) == 1
    with pytest.raises(RuntimeError, match=r"gemm_q4_f32 kernel failed \(cuda error 1\)"):
        K.gemm_q4_f32(d, d, d, 4, 33, 1, 16)
    assert K.check_sm100() and K.device_error() == 0


# ---------------- integer parity: codes and scales are bit-exact ----------------

@pytest.mark.parametrize("n", [32, 4096, 128 * 1000, 4096 * 512])
def test_device_quantizers_match_reference_quantizers_bit_for_bit(n):
    G = _gpu()
    rng = U.seeded(n)
    w = (rng.standard_normal(n) * 0.02).astype(np.float32)
    w[: min(n, 64)] = 0                                              # an all-zero block / group
    if n >= 4096:
        w[128:256] = 0.5                                             # a constant group (range 0)
        w[300] = 1e-30
    src = torch.from_numpy(w).cuda()
    q4 = O.quantize_q4(w)
    sep = torch.zeros(K.q4_gpu_data_offset(n // 32) + n // 2, dtype=torch.uint8, device="cuda")
    K.quantize_q4_0(src, sep, n)
    assert np.array_equal(sep.cpu().numpy(), q4.raw_bytes_gpu())
    q8 = O.quantize_q8(w)
    b36 = torch.zeros(n // 32 * 36, dtype=torch.uint8, device="cuda")
    K.quantize_q8_0(src, b36, n)
    assert np.array_equal(b36.cpu().numpy(), q8.blocks)
    if n % 128 == 0:
        for awq in (False, True):
            st = O.quantize_awq(w, 128) if awq else O.quantize_gptq(w, 128, 4)
            qd = torch.zeros(n // 2, dtype=torch.uint8, device="cuda")
            meta = torch.zeros(n // 128 * 4, dtype=torch.uint8, device="cuda")
            K.quantize_w4g(src, qd, meta, n, 128, awq)
            assert np.array_equal(qd.cpu().numpy(), st.data)
            m = meta.cpu().numpy().view(np.uint16).reshape(-1, 2)
            assert np.array_equal(m[:, 0], st.scales) and np.array_equal(m[:, 1], st.zeros)
    if n == 4096:
        st = O.quantize_gptq(w, 32, 4)                               # generic group size
        qd = torch.zeros(n // 2, dtype=torch.uint8, device="cuda")
        meta = torch.zeros(n // 32 * 4, dtype=torch.uint8, device="cuda")
        K.quantize_w4g(src, qd, meta, n, 32, False)
        assert np.array_equal(qd.cpu().numpy(), st.data)


def test_device_dequantize_matches_storage_slice_bit_for_bit():
    G = _gpu()
    rng = U.seeded(99)
    n, k = 24, 1024
    w = U.make_weights(rng, n, k)
    out = torch.empty(n * k, dtype=torch.float32, device="cuda")

    q4 = O.quantize_q4(w)
    sep, off = G.upload_blocks18(q4.blocks, q4.num_blocks())
    K.dequantize(K.FMT_Q4_0, sep, None, out, n * k, off)
    assert np.array_equal(out.cpu().numpy(), q4.slice())

    iq = O.make_iq4nl_blocks(w)
    sep, off = G.upload_blocks18(iq.raw, iq.num_blocks())
    K.dequantize(K.FMT_IQ4NL, sep, None, out, n * k, off)
    assert np.array_equal(out.cpu().numpy(), iq.slice())

    q8 = O.quantize_q8(w)
    K.dequantize(K.FMT_Q8_0, G.dev_u8(q8.blocks), None, out, n * k, 0)
    assert np.array_equal(out.cpu().numpy(), q8.slice())

    for st in (O.quantize_gptq(w, 128, 4), O.quantize_awq(w, 128)):
        qd, meta = G.upload_w4g(st)
        K.dequantize(K.FMT_W4G, qd, meta, out, n * k, 128)
        assert np.array_equal(out.cpu().numpy(), st.slice())

    for kk in (1024, 37):                                           # 37: rows not byte aligned in the flat packing
        vals = rng.integers(-1, 2, size=n * kk).astype(np.int8)
        st = O.new_ternary_from(vals)
        rows = G.upload_ternary(st, n, kk)
        o2 = torch.empty(n * kk, dtype=torch.float32, device="cuda")
        K.dequantize(K.FMT_TERNARY, rows, None, o2, n * kk, kk)
        assert np.array_equal(o2.cpu().numpy(), vals.astype(np.float32))


@pytest.mark.parametrize("fmt", ["w4g", "q4_0"])
@pytest.mark.parametrize("n,k,splits", [(64, 4096, 4), (7, 8192, 8), (300, 14336, 7), (16, 28672, 14), (1, 2048, 2)])
def test_splitk_matches_oracle_and_is_deterministic(fmt, n, k, splits):
    """Narrow outputs: K cut into slices, fp32 partials in a caller-provided workspace, ordered second pass."""
    G = _gpu()
    rng = U.seeded(n + k + splits)
    wf = U.make_weights(rng, n, k)
    xb = U.make_x_bits(rng, 1, k)
    xf = O.f16_bits_to_f32(xb).reshape(1, k)
    x = G.x_dev(xb)
    ws = torch.full((K.splitk_workspace_bytes(n, splits) // 4,), float("nan"), dtype=torch.float32, device="cuda")
    if fmt == "w4g":
        st = O.quantize_gptq(wf, 128, 4)
        ref = U.ref_dense_a_side(st.slice().reshape(n, k), xf, n, k)
        qd, meta = G.upload_w4g(st)
        call = lambda y, fl: K.gemv_w4g_splitk(qd, meta, x, y, n, k, 128, splits, ws, fl)
        whole = lambda y: K.gemv_w4g(qd, meta, x, y, n, k, 128, 1, K.Y_F32)
    else:
        st = O.quantize_q4(wf)
        ref = U.ref_q4_0(st, xf, n, k)
        sep, off = G.upload_blocks18(st.blocks, st.num_blocks())
        call = lambda y, fl: K.gemv_q4_0_splitk(sep, off, x, y, n, k, splits, ws, fl)
        whole = lambda y: K.gemv_q4_0(sep, off, x, y, n, k, 1, K.Y_F32)
    absd = U.absdot(st.slice().reshape(n, k), xf)
    got = G.run(lambda y: call(y, K.Y_F32), n, 1)
    _check(got, ref, absd, f"{fmt} split-K")
    assert np.array_equal(got, G.run(lambda y: call(y, K.Y_F32), n, 1))          # same bits every time
    _check(G.run(lambda y: call(y, 0), n, 1, y_f32=False), U.to_f16_round(ref), absd, f"{fmt} split-K f16 out")
    _check(got, G.run(whole, n, 1), absd, f"{fmt} split-K vs unsplit kernel")
    from ztensor_b200 import _lib
    assert _lib.lib().ztq_gemv_w4g_splitk(x.data_ptr(), x.data_ptr(), x.data_ptr(), x.data_ptr(), n, k, 128, splits,
                                          ws.data_ptr(), 4, 0, None) == 1               # workspace too small


@pytest.mark.parametrize("n,k", [(128, 512), (256, 1024), (300, 4096), (1000, 2048), (64, 14336)])
@pytest.mark.parametrize("batch", [16, 17, 32, 40, 3])
@pytest.mark.parametrize("variant", ["int8", "fp16"])
def test_w4a16_tensor_core_skinny_gemm(n, k, batch, variant):
    """Batch >= 16: the tcgen05 / TMEM kernels (integer operands by default, fp16 operands under
    FP32_DECODE) against compute.MatMulW4A16 of the oracle (weights on A)."""
    vf = K.FP32_DECODE if variant == "fp16" else 0
    G = _gpu()
    rng = U.seeded(n * 23 + k + batch)
    st = O.quantize_gptq(U.make_weights(rng, n, k), 128, 4)
    xb = U.make_x_bits(rng, batch, k)
    act = O.Float16Storage(xb.T.copy().ravel(), batch * k)
    ref = np.ascontiguousarray(O.matmul_w4a16(st, (n, k), act, (k, batch)).T)
    xf = O.f16_bits_to_f32(xb).reshape(batch, k)
    absd = U.absdot(st.slice().reshape(n, k), xf)
    qd, meta = G.upload_w4g(st)
    x = G.x_dev(xb)
    ws = torch.empty(K.gemm_w4g_tc_workspace_bytes(n, k, batch), dtype=torch.uint8, device="cuda")
    got = G.run(lambda y: K.gemm_w4g_tc(qd, meta, x, y, n, k, 128, batch, ws, K.Y_F32 | vf), n, batch)
    assert K.device_error() == 0
    _check(got, ref, absd, "w4a16 tcgen05 f32 out")
    got16 = G.run(lambda y: K.gemm_w4g_tc(qd, meta, x, y, n, k, 128, batch, ws, vf), n, batch, y_f32=False)
    _check(got16, U.to_f16_round(ref), absd, "w4a16 tcgen05 f16 out")
    assert np.array_equal(got, G.run(lambda y: K.gemm_w4g_tc(qd, meta, x, y, n, k, 128, batch, ws, K.Y_F32 | vf), n, batch))


@pytest.mark.parametrize("n,k", [(128, 512), (256, 1024), (300, 4096), (1000, 2048), (64, 14336)])
@pytest.mark.parametrize("batch", [3, 4, 8, 16, 17, 40])
def test_q4_0_tensor_core_skinny_gemm(n, k, batch):
    """Three or more activation rows on Q4_0 weights: the tcgen05 / TMEM kernel with a scale per block of 32, against
    CPUEngine.MatMul -> GemmF32Q4NT of the oracle (weights on B) and against the GEMV passes."""
    G = _gpu()
    rng = U.seeded(n * 31 + k + batch)
    st = O.quantize_q4(U.make_weights(rng, n, k))
    xb = U.make_x_bits(rng, batch, k)
    xf = O.f16_bits_to_f32(xb).reshape(batch, k)
    ref = U.ref_q4_0(st, xf, n, k)
    absd = U.absdot(st.slice().reshape(n, k), xf)
    sep, off = G.upload_blocks18(st.blocks, st.num_blocks())
    x = G.x_dev(xb)
    ws = torch.empty(K.gemm_q4_0_tc_workspace_bytes(n, k, batch), dtype=torch.uint8, device="cuda")
    got = G.run(lambda y: K.gemm_q4_0_tc(sep, off, x, y, n, k, batch, ws, K.Y_F32), n, batch)
    assert K.device_error() == 0
    _check(got, ref, absd, "q4_0 tcgen05 f32 out")
    got16 = G.run(lambda y: K.gemm_q4_0_tc(sep, off, x, y, n, k, batch, ws, 0), n, batch, y_f32=False)
    _check(got16, U.to_f16_round(ref), absd, "q4_0 tcgen05 f16 out")
    assert np.array_equal(got, G.run(lambda y: K.gemm_q4_0_tc(sep, off, x, y, n, k, batch, ws, K.Y_F32), n, batch))
    gemv = G.run(lambda y: K.gemv_q4_0(sep, off, x, y, n, k, batch, K.Y_F32), n, batch)
    assert np.abs(got - gemv).max() <= 2e-4 * max(1e-6, np.abs(gemv).max())


@pytest.mark.parametrize("n,k", [(128, 512), (256, 1024), (300, 4096), (1000, 2048), (64, 14336)])
@pytest.mark.parametrize("batch", [3, 4, 8, 16, 17, 40])
def test_q8_0_tensor_core_skinny_gemm(n, k, batch):
    """Three or more activation rows on Q8_0 weights: the tcgen05 / TMEM kernel on the raw 36-byte blocks (signed int8
    operand, float scales through shared memory), against the CPU engine's Q8 path of the oracle and the GEMV passes."""
    G = _gpu()
    rng = U.seeded(n * 37 + k + batch)
    st = O.quantize_q8(U.make_weights(rng, n, k))
    xb = U.make_x_bits(rng, batch, k)
    xf = O.f16_bits_to_f32(xb).reshape(batch, k)
    ref = U.ref_q8_0(st, xf, n, k)
    absd = U.absdot(st.slice().reshape(n, k), xf)
    w = G.dev_u8(st.blocks)
    x = G.x_dev(xb)
    ws = torch.empty(K.gemm_q8_0_tc_workspace_bytes(n, k, batch), dtype=torch.uint8, device="cuda")
    got = G.run(lambda y: K.gemm_q8_0_tc(w, x, y, n, k, batch, ws, K.Y_F32), n, batch)
    assert K.device_error() == 0
    _check(got, ref, absd, "q8_0 tcgen05 f32 out")
    got16 = G.run(lambda y: K.gemm_q8_0_tc(w, x, y, n, k, batch, ws, 0), n, batch, y_f32=False)
    _check(got16, U.to_f16_round(ref), absd, "q8_0 tcgen05 f16 out")
    assert np.array_equal(got, G.run(lambda y: K.gemm_q8_0_tc(w, x, y, n, k, batch, ws, K.Y_F32), n, batch))
    gemv = G.run(lambda y: K.gemv_q8_0(w, x, y, n, k, batch, K.Y_F32), n, batch)
    assert np.abs(got - gemv).max() <= 2e-4 * max(1e-6, np.abs(gemv).max())
