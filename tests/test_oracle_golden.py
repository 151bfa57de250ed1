"""Pins the CPU oracle against the reference's own known-answer tests.

Each case restates the inputs and expectations of a test in zerfoo/ztensor
(cited per test).  Runs without a GPU."""
import numpy as np
import pytest

from oracle import oracle as O


def linspace(lo, hi, n):
    # tensor/quantized_test.go linspace helper: lo + (hi-lo)*i/(n-1) in float32
    if n == 1:
        return np.array([lo], np.float32)
    i = np.arange(n, dtype=np.float32)
    return (np.float32(lo) + (np.float32(hi) - np.float32(lo)) * i / np.float32(n - 1)).astype(np.float32)


# ---------------- ternary: compute/ternary_gemv_test.go:25-141 ----------------

def test_ternary_known_values():
    w = [1, 0, -1, 1, -1, 1, 0, 0, 0, -1, 1, -1]
    y = O.ternary_gemv(O.new_ternary_from(w), [2.0, 3.0, 4.0, 5.0], 3, 4)
    assert y.tolist() == [3.0, 1.0, -4.0]


def test_ternary_non_multiple_of_4_cols():
    w = [1, -1, 0, 1, -1, 0, 1, -1, 0, 1]
    y = O.ternary_gemv(O.new_ternary_from(w), [1.0, 2.0, 3.0, 4.0, 5.0], 2, 5)
    assert y.tolist() == [-2.0, 4.0]


def test_ternary_all_zeros():
    ts = O.new_ternary_from(np.zeros(16 * 32, np.int8))
    y = O.ternary_gemv(ts, np.arange(1, 33, dtype=np.float32), 16, 32)
    assert not y.any()


@pytest.mark.parametrize("w", [-1, 0, 1])
def test_ternary_single_element(w):
    y = O.ternary_gemv(O.new_ternary_from([w]), [7.5], 1, 1)
    assert y[0] == np.float32(w) * np.float32(7.5)


def test_ternary_identity_diagonal():
    n = 33
    vals = np.zeros((n, n), np.int8)
    vals[np.arange(n), np.arange(n)] = 1
    x = (np.arange(n, dtype=np.float32) * 0.5 - 8.0).astype(np.float32)
    y = O.ternary_gemv(O.new_ternary_from(vals), x, n, n)
    assert np.array_equal(y, x)


def test_ternary_matches_dense_float32():
    # :47-74 uses Go's PCG(42,0); the generator is not restated, the property is kept.
    rng = np.random.default_rng(42)
    rows, cols = 128, 256
    vals = rng.integers(-1, 2, size=rows * cols).astype(np.int8)
    x = (rng.random(cols, dtype=np.float32) * 2 - 1).astype(np.float32)
    got = O.ternary_gemv(O.new_ternary_from(vals), x, rows, cols)
    want = np.zeros(rows, np.float32)
    w = vals.reshape(rows, cols).astype(np.float32)
    for j in range(cols):                       # denseGEMV :11-21, sequential float32
        want = (want + w[:, j] * x[j]).astype(np.float32)
    assert np.abs(got - want).max() <= 1e-6


# ---------------- ternary storage: tensor/ternary_storage_test.go:5-70 --------

@pytest.mark.parametrize("values", [
    [-1, -1, -1, -1], [0, 0, 0, 0], [1, 1, 1, 1], [-1, 0, 1, 0], [-1], [0], [1], [-1, 0, 1],
    [1, -1, 0, 1, -1], [-1, 1, 0, -1, 1, 0, 1], [],
    [-1, 0, 1, 0, 1, -1, -1, 0, 0, 1, 1, -1, 0, 0, -1, 1],
])
def test_ternary_storage_round_trip(values):
    s = O.new_ternary_from(values)
    assert s.len == len(values)
    assert [s.get(i) for i in range(len(values))] == list(values)


def test_ternary_storage_bit_positions():
    # encoding 00=-1, 01=0, 10=+1; element i at bits 2*(i%4) of byte i/4 (ternary_storage.go:39-62)
    s = O.new_ternary_from([1, -1, 0, 1, -1])
    assert s.data.tolist() == [0b10_01_00_10, 0b00]
    with pytest.raises(ValueError):
        O.new_ternary_from([2])


# ---------------- IQ4_NL: tensor/iq4_storage_test.go:12-87,165-183 -------------

def encode_iq4nl_block(scale, nibbles):
    blk = np.zeros(18, np.uint8)
    blk[:2] = O.f32_to_f16_bits([scale]).view(np.uint8)
    n = np.asarray(nibbles, np.uint8)
    blk[2:] = (n[0::2] & 0xF) | (n[1::2] << 4)
    return blk


def test_iq4nl_dequantize_block():
    nib = np.arange(32) % 16
    st = O.new_iq4nl_from_raw(encode_iq4nl_block(2.0, nib), 32)
    want = O.f16_bits_to_f32(O.f32_to_f16_bits([2.0]))[0] * O.iq4nl_table()[nib]
    assert np.abs(st.slice() - want).max() <= 1e-6


def test_iq4nl_storage_roundtrip_and_partial():
    scales = [1.5, 0.75]
    raw, exp = [], []
    for bi in range(2):
        nib = (bi * 7 + np.arange(32) * 3) % 16
        raw.append(encode_iq4nl_block(scales[bi], nib))
        exp.append(np.float32(scales[bi]) * O.iq4nl_table()[nib])
    st = O.new_iq4nl_from_raw(np.concatenate(raw), 64)
    assert np.abs(st.slice() - np.concatenate(exp)).max() <= 1e-6
    st48 = O.new_iq4nl_from_raw(np.concatenate(raw), 48)
    assert st48.slice().size == 48 and np.array_equal(st48.slice(), st.slice()[:48])
    with pytest.raises(ValueError):
        O.new_iq4nl_from_raw(np.zeros(17, np.uint8), 32)
    with pytest.raises(ValueError):
        O.new_iq4nl_from_raw(np.zeros(18, np.uint8), 0)


def test_iq4nl_table_properties():
    t = O.iq4nl_table()
    assert np.all(np.diff(t) > 0) and t[7] == 0.0 and t[0] == -1.0 and t[15] == np.float32(1.3312578)


# ---------------- Q4_0: tensor/quantized_test.go:10-59,145-171 -----------------

@pytest.mark.parametrize("inp,max_err", [
    (linspace(-1, 1, 32), 0.1), (linspace(-0.5, 0.5, 64), 0.1),
    (np.zeros(32, np.float32), 0.001), (linspace(-1, 1, 48), 0.1),
])
def test_q4_round_trip(inp, max_err):
    q = O.quantize_q4(inp)
    assert q.len == inp.size
    assert np.abs(q.slice() - inp).max() <= max_err


def test_q4_block_layout_and_codes():
    # scale = fp16(absmax/7); byte j = (q[j]+8) | (q[j+16]+8)<<4  (quantized.go:56-88)
    inp = linspace(-1, 1, 32)
    q = O.quantize_q4(inp)
    assert q.blocks.size == 18
    scale = np.float32(1.0) / np.float32(7.0)
    assert q.scales_bits()[0] == O.f32_to_f16_bits([scale])[0]
    inv = np.float32(1.0) / scale
    want = np.clip(np.sign(inp * inv) * np.floor(np.abs((inp * inv).astype(np.float64)) + 0.5), -8, 7) + 8
    assert np.array_equal(q.codes(), want.astype(np.uint8))
    assert q.codes()[0] == 1 and q.codes()[31] == 15          # -7 and +7


def test_q4_gpu_layout_contract():
    # RawBytesGPU / Q4GPUDataOffset, quantized.go:158-199; gemm_q4_test.go repackQ4ForGPU :87-102
    q = O.quantize_q4(linspace(-1, 1, 96))
    g = q.raw_bytes_gpu()
    off = O.q4_gpu_data_offset(3)
    assert off == 16 and g.size == 16 + 48
    aos = q.blocks.reshape(3, 18)
    assert np.array_equal(g[:6], aos[:, :2].ravel()) and not g[6:16].any()
    assert np.array_equal(g[16:], aos[:, 2:].ravel())


# ---------------- Q8_0: tensor/quantized_q8_test.go ---------------------------

def test_q8_round_trip_and_blocks():
    inp = linspace(-1, 1, 64)
    q = O.quantize_q8(inp)
    assert q.blocks.size == 72
    assert np.abs(q.slice() - inp).max() <= 0.01
    assert q.scales()[0] == np.float32(1.0) / np.float32(127.0)     # f32 scale, 36-byte block
    assert q.codes()[0] == -127 and np.array_equal(q.slice(), q.codes().astype(np.float32) * np.repeat(q.scales(), 32))


# ---------------- GPTQ / AWQ: quantized_gptq_test.go, quantized_awq_test.go ---

def test_awq_known_vectors():
    # quantized_awq_test.go:88-118: scale 7/15, zero 0, codes 0,2,4,6,9,11,13,15
    q = O.quantize_awq([0, 1, 2, 3, 4, 5, 6, 7], 8)
    assert q.codes().tolist() == [0, 2, 4, 6, 9, 11, 13, 15]
    d = q.slice()
    assert abs(d[0]) <= 0.1 and abs(d[7] - 7.0) <= 0.1 and np.abs(d - np.arange(8)).max() <= 1.1


def test_awq_zero_scale_and_extremes():
    q = O.quantize_awq([3.14] * 8, 8)
    assert not q.slice().any()
    inp = np.zeros(16, np.float32)
    inp[0], inp[15] = -10.0, 10.0
    inp[1:15] = (np.arange(1, 15) - 7) * np.float32(0.1)
    q = O.quantize_awq(inp, 16)
    d = q.slice()
    assert q.codes()[0] == 0 and q.codes()[15] == 15
    assert abs(d[0] + 10) <= 0.2 and abs(d[15] - 10) <= 0.2


def test_gptq_symmetric_and_endpoints():
    inp = linspace(-1, 1, 128)
    q = O.quantize_gptq(inp, 128, 4)
    d = q.slice()
    assert q.codes()[0] == 0 and q.codes()[127] == 15
    assert np.all(d[inp > 0.15] > 0) and np.all(d[inp < -0.15] < 0)
    assert np.mean((d - inp) ** 2) < 0.01
    # GPTQ and AWQ pack the same bytes; only the rounding differs (quantized_awq.go:96-103)
    a = O.quantize_awq(inp, 128)
    assert a.data.size == q.data.size == 64 and np.array_equal(a.scales, q.scales) and np.array_equal(a.zeros, q.zeros)


def test_gptq_partial_group_sizes():
    q = O.quantize_gptq(linspace(-1, 1, 200), 128, 4)
    assert q.num_groups() == 2 and q.data.size == 64 + 36 and q.slice().size == 200


# ---------------- fp16: tensor/fp16_storage_test.go --------------------------

def test_fp16_exact_and_rounding():
    pw = np.array([1, 2, 4, 0.5, 0.25, -1, -2, 1024, 2.0 ** -14, 2.0 ** -24, 65504], np.float32)
    assert np.array_equal(O.new_float16_from_f32(pw).slice(), pw)
    v = np.random.default_rng(0).standard_normal(4096).astype(np.float32)
    bits = O.f32_to_f16_bits(v)
    assert np.array_equal(bits, v.astype(np.float16).view(np.uint16))       # IEEE RNE == numpy
    assert np.array_equal(O.f16_bits_to_f32(bits), v.astype(np.float16).astype(np.float32))
    edge = np.array([65519.9, 65520.0, 1e-8, 2.0 ** -25, 3e-8, np.inf, -np.inf, 6.1e-5], np.float32)
    assert np.array_equal(O.f32_to_f16_bits(edge), edge.astype(np.float16).view(np.uint16))
    every = np.arange(65536, dtype=np.uint16)
    dec = O.f16_bits_to_f32(every)
    ok = ~np.isnan(dec)
    assert np.array_equal(dec[ok], every.view(np.float16).astype(np.float32)[ok])
    assert O.LIB.zo_xblas_f16_bits_to_f32(0x7C00) == 0.0 and O.LIB.zo_xblas_f16_bits_to_f32(0x0001) == 2.0 ** -24


# ---------------- W4A16: compute/w4a16_test.go:32-181 -------------------------

@pytest.mark.parametrize("maker", [O.quantize_q4, lambda w: O.quantize_gptq(w, 32, 4), lambda w: O.quantize_awq(w, 32)])
def test_w4a16_a_side(maker):
    m, k, n = 2, 32, 3
    w = ((np.arange(m * k) % 7 - 3) * np.float32(0.1)).astype(np.float32)
    act = ((np.arange(k * n) % 5 - 2) * np.float32(0.1)).astype(np.float32)
    ws, fs = maker(w), O.new_float16_from_f32(act)
    got = O.matmul_w4a16(ws, (m, k), fs, (k, n))
    assert got.shape == (m, n)
    want = O.cpu_engine_matmul(ws.slice(), (m, k), fs.slice(), (k, n))
    assert np.sqrt(np.mean((got - want) ** 2)) <= 1e-6
    dense = w.reshape(m, k).astype(np.float64) @ act.reshape(k, n).astype(np.float64)
    assert np.abs(got - dense).max() <= 0.15
    with pytest.raises(ValueError):
        O.matmul_w4a16(ws.slice(), (m, k), fs, (k, n))


# ---------------- xblas: internal/xblas/gemm_quant_test.go -------------------

def _fill(n, mod, off):
    return ((np.arange(n) % mod - off) * np.float32(0.1)).astype(np.float32)


@pytest.mark.parametrize("m,k,n", [(4, 32, 8), (1, 64, 1), (3, 128, 5), (2, 256, 17), (1, 4096, 1)])
def test_gemm_q4_fused_vs_dequant_sgemm(m, k, n):
    a, b = _fill(m * k, 7, 3), _fill(k * n, 5, 2)
    q = O.quantize_q4(a)
    got = O.gemm_q4_f32(m, n, k, q, b)
    want = O.sgemm_simd(m, n, k, q.slice(), b)
    assert np.abs(got - want).max() <= 1e-5            # same values, same order
    assert np.abs(got - (a.reshape(m, k) @ b.reshape(k, n)).ravel()).max() <= 0.15 * max(1, k / 32)


@pytest.mark.parametrize("m,k,n", [(1, 64, 8), (2, 128, 16), (1, 512, 256), (4, 32, 3)])
def test_gemm_f32_q4_nt_and_q8_nt(m, k, n):
    a, w = _fill(m * k, 5, 2), _fill(n * k, 7, 3)
    q4, q8 = O.quantize_q4(w), O.quantize_q8(w)
    for q, fn, tol in ((q4, O.gemm_f32_q4_nt, 0.15), (q8, O.gemm_f32_q8_nt, 0.02)):
        got = fn(m, n, k, a, q).reshape(m, n)
        ref = a.reshape(m, k).astype(np.float64) @ q.slice().reshape(n, k).T.astype(np.float64)
        assert np.abs(got - ref).max() <= 1e-4
        assert np.abs(got - a.reshape(m, k) @ w.reshape(n, k).T).max() <= tol * max(1, k / 32)
        # the threaded m==1 fan-out returns the same bits as one thread
        assert np.array_equal(fn(m, n, k, a, q, 1), fn(m, n, k, a, q, 8))
        # CPUEngine.MatMul picks the same path for a B-side quantized weight
        assert np.array_equal(O.cpu_engine_matmul(a, (m, k), q, (k, n)).ravel(), fn(m, n, k, a, q))


def test_nt_thread_rule():
    assert O.nt_threads(4096, 4096, 8) == 8 and O.nt_threads(16, 4096, 8) == 4
    assert O.nt_threads(255, 256, 8) == 1 and O.nt_threads(8, 8192, 64) == 2


def test_sgemm_simd_order_gemv_is_sequential_unfused():
    # n == 1: every update takes the MULSS+ADDSS tail (gemm_simd_amd64.s:60-70)
    rng = np.random.default_rng(3)
    k = 1000
    a = rng.standard_normal(k).astype(np.float32)
    b = rng.standard_normal(k).astype(np.float32)
    a[::17] = 0
    got = O.sgemm_simd(1, 1, k, a, b)[0]
    s = np.float32(0)
    for p in range(k):
        if a[p] != 0:
            s = np.float32(np.float32(b[p] * a[p]) + s)
    assert got == s
    # n == 8: the lanes are fused (one rounding per update)
    n = 8
    b8 = rng.standard_normal((k, n)).astype(np.float32)
    got8 = O.sgemm_simd(1, n, k, a, b8)
    s8 = np.zeros(n, np.float64)
    for p in range(k):
        s8 = (np.float64(a[p]) * b8[p].astype(np.float64) + s8).astype(np.float32).astype(np.float64)
    assert np.array_equal(got8, s8.astype(np.float32))


def test_fused_swiglu_known_answer():
    """internal/gpuapi/metal_kernels_test.go:437-456: w1 = {0, 1, -1, 2}, w3 = 1 -> x / (1 + exp(-x)), 1e-5."""
    import math
    from oracle import oracle as O
    w1 = np.array([0, 1, -1, 2], dtype=np.float32)
    got = O.fused_swiglu(w1, np.ones(4, dtype=np.float32))
    want = np.array([x / (1.0 + math.exp(-x)) for x in (0.0, 1.0, -1.0, 2.0)], dtype=np.float32)
    assert np.abs(got - want).max() <= 1e-5


def test_fused_add_rmsnorm_known_answer():
    """internal/gpuapi/metal_kernels_test.go:458-490: input {1,2,3,4} + residual {.1,.2,.3,.4}, unit gains, eps 1e-5;
    normed within 1e-4, sum within 1e-5.  compute/gpu_bf16_fused_norm_parity_test.go:27-38 is the same formula in float64."""
    import math
    from oracle import oracle as O
    x = np.array([1, 2, 3, 4], dtype=np.float32)
    r = np.array([0.1, 0.2, 0.3, 0.4], dtype=np.float32)
    normed, summed = O.fused_add_rmsnorm(x, r, np.ones(4, dtype=np.float32), 1e-5)
    sums = [1.1, 2.2, 3.3, 4.4]
    rms = math.sqrt(sum(v * v for v in sums) / 4.0 + 1e-5)
    assert np.abs(normed - np.array([v / rms for v in sums], dtype=np.float32)).max() <= 1e-4
    assert np.abs(summed - np.array(sums, dtype=np.float32)).max() <= 1e-5
    # a longer row against the float64 statement, non-trivial gains, no residual
    rng = np.random.default_rng(11)
    xv = rng.standard_normal(4096).astype(np.float32)
    g = rng.uniform(0.5, 1.5, 4096).astype(np.float32)
    n2, s2 = O.fused_add_rmsnorm(xv, None, g, 1e-6)
    x64 = xv.astype(np.float64)
    ref = x64 / np.sqrt((x64 * x64).mean() + 1e-6) * g
    assert np.array_equal(s2, xv)
    assert np.abs(n2 - ref).max() <= 1e-5


# ---- Q4_K: tensor/quantized_kquant_test.go ---------------------------------------------------------
def test_q4k_round_trip_zeros_and_ramp():
    """TestDequantizeQ4K_RoundTrip (:134-158, sin pattern, max error 0.6), _Zeros (:160-172, exact zeros),
    TestNewQ4KStorageFromRaw (:174-206, linear ramp, max error 0.3, Len 256)."""
    import math
    from oracle import oracle as O
    v = np.array([math.sin(i * 0.1) * 2.0 for i in range(256)], dtype=np.float32)
    st = O.quantize_q4k(v)
    assert st.raw.size == 144 and np.abs(st.slice() - v).max() <= 0.6
    z = O.quantize_q4k(np.zeros(256, dtype=np.float32))
    assert not z.slice().any()
    ramp = (np.arange(256) * 0.01).astype(np.float32)
    st = O.new_q4k_from_raw(O.quantize_q4k(ramp).raw, 256)
    assert st.len == 256 and st.slice().size == 256 and np.abs(st.slice() - ramp).max() <= 0.3
    with pytest.raises(ValueError):                                   # TestNewQ4KStorageFromRaw_InvalidSize (:208-213)
        O.new_q4k_from_raw(np.zeros(10, dtype=np.uint8), 256)


def test_q4k_scale_packing_and_products():
    """The 12-byte scale region (get_scale_min_k4 layout, quantized_kquant.go:26-49) decodes to what the quantizer
    packed, and both CPU products (gemm_q4k.go) agree with dequantize-then-multiply."""
    from oracle import oracle as O
    rng = np.random.default_rng(5)
    n, k = 24, 1024
    w = (rng.standard_normal((n, k // 32, 32)) * rng.uniform(0.01, 1.0, (n, k // 32, 1))).astype(np.float32).reshape(-1)
    st = O.quantize_q4k(w)
    for b in (0, 7, st.num_blocks() - 1):
        blk = st.raw[b * 144:(b + 1) * 144]
        sc, mn = st.scales_mins(b)
        assert (sc <= 63).all() and (mn <= 63).all()
        for i in range(4):                                            # the packing QuantizeQ4K writes (:186-193)
            assert blk[4 + i] == (sc[i] & 63) | ((sc[4 + i] >> 4) << 6)
            assert blk[8 + i] == (mn[i] & 63) | ((mn[4 + i] >> 4) << 6)
            assert blk[12 + i] == (sc[4 + i] & 0xF) | ((mn[4 + i] & 0xF) << 4)
    x = rng.standard_normal(k).astype(np.float32)
    dense = st.slice().reshape(n, k).astype(np.float64) @ x.astype(np.float64)
    nt = O.gemm_f32_q4k_nt(1, n, k, x, st, ncpu=1)
    par = O.gemm_f32_q4k_nt(1, n, k, x, st, ncpu=4)
    a_side = O.gemm_q4k_f32(n, 1, k, st, x)
    assert np.array_equal(nt, par)                                    # the row fan-out changes no arithmetic
    assert np.abs(nt - dense).max() <= 1e-4 and np.abs(a_side - dense).max() <= 1e-4
    sep = st.raw_bytes_gpu()
    nb = st.num_blocks()
    assert sep.size == nb * 144
    assert np.array_equal(sep[:nb * 16].reshape(nb, 16), st.raw.reshape(nb, 144)[:, :16])


def test_q5k_round_trip_and_product():
    """TestDequantizeQ5K_RoundTrip (quantized_kquant_test.go:473-493: sin pattern, max error 0.5) with blocks built by the
    same recipe as that test's own builder (:365-470); NewQ5KStorageFromRaw sizes (:564-577); GemmF32Q5KNT equals
    dequantize-then-multiply and its row fan-out changes no arithmetic."""
    import math
    from oracle import oracle as O
    v = np.array([math.sin(i * 0.1) * 2.0 for i in range(256)], dtype=np.float32)
    st = O.make_q5k_blocks(v)
    assert st.raw.size == 176 and np.abs(st.slice() - v).max() <= 0.5
    assert np.abs(st.slice() - v).max() < np.abs(O.quantize_q4k(v).slice() - v).max()      # finer than Q4_K
    with pytest.raises(ValueError):
        O.new_q5k_from_raw(np.zeros(100, dtype=np.uint8), 256)
    rng = np.random.default_rng(9)
    n, k = 20, 1024
    w = (rng.standard_normal(n * k) * 0.02).astype(np.float32)
    st = O.make_q5k_blocks(w)
    x = rng.standard_normal(k).astype(np.float32)
    dense = st.slice().reshape(n, k).astype(np.float64) @ x.astype(np.float64)
    one = O.gemm_f32_q5k_nt(1, n, k, x, st, ncpu=1)
    assert np.array_equal(one, O.gemm_f32_q5k_nt(1, n, k, x, st, ncpu=4))
    assert np.abs(one - dense).max() <= 1e-4
    sep = st.raw_bytes_gpu()
    nb = st.num_blocks()
    assert sep.size == nb * 176 and np.array_equal(sep[:48 * nb].reshape(nb, 48)[:, 16:], st.raw.reshape(nb, 176)[:, 144:])


def test_q6k_round_trip_zeros_and_product():
    """TestDequantizeQ6K_RoundTrip (quantized_kquant_test.go:300-321: sin pattern, max error 0.3), _Zeros (:323-335),
    TestNewQ6KStorageFromRaw sizes (:337-357), with blocks built by the recipe of that file's builder (:216-298)."""
    import math
    from oracle import oracle as O
    v = np.array([math.sin(i * 0.1) * 2.0 for i in range(256)], dtype=np.float32)
    st = O.make_q6k_blocks(v)
    assert st.raw.size == 210 and np.abs(st.slice() - v).max() <= 0.3
    assert not O.make_q6k_blocks(np.zeros(256, dtype=np.float32)).slice().any()
    ramp = (np.arange(256) * 0.01).astype(np.float32)
    st = O.new_q6k_from_raw(O.make_q6k_blocks(ramp).raw, 256)
    assert st.len == 256 and st.slice().size == 256
    with pytest.raises(ValueError):
        O.new_q6k_from_raw(np.zeros(100, dtype=np.uint8), 256)
    rng = np.random.default_rng(13)
    n, k = 20, 1024
    st = O.make_q6k_blocks((rng.standard_normal(n * k) * 0.02).astype(np.float32))
    x = rng.standard_normal(k).astype(np.float32)
    dense = st.slice().reshape(n, k).astype(np.float64) @ x.astype(np.float64)
    one = O.gemm_f32_q6k_nt(1, n, k, x, st, ncpu=1)
    assert np.array_equal(one, O.gemm_f32_q6k_nt(1, n, k, x, st, ncpu=4)) and np.abs(one - dense).max() <= 1e-4
    # hand-made block: code 33 (= +1) in element 0 only, scale 2, d = 0.5 -> 1.0 at element 0, zero elsewhere
    raw = np.zeros(210, dtype=np.uint8)
    raw[0:128] = 0x00
    raw[128:192] = 0xAA                      # high bits 10 -> code 32 (= 0) everywhere
    raw[0] = 0x01                            # element 0: low nibble 1 -> code 33
    raw[192:208] = 2
    raw[208:210] = np.frombuffer(O.f32_to_f16_bits(np.array([0.5], np.float32)).tobytes(), np.uint8)
    out = O.Q6KStorage(raw, 256).slice()
    assert out[0] == 1.0 and not out[1:].any()
