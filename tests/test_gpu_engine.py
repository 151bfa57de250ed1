"""Engine-level parity: the C++ mirror of GPUEngine.MatMul / TryW4A16MatMul / TernaryGEMVGPU /
UploadWeights against the oracle's CPUEngine, following the reference's own tests."""
import numpy as np
import pytest

from oracle import oracle as O
from tests import util as U

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def eng():
    from ztensor_b200 import engine as E
    return E, E.GPUEngine(0)


def _fill(n, mod, off):
    return ((np.arange(n) % mod - off) * np.float32(0.1)).astype(np.float32)


def _w4_tensor(E, kind, w, shape, group=32):
    if kind == "q4":
        st = O.quantize_q4(w)
        return st, E.q4_tensor(st.blocks, st.len, shape)
    st = O.quantize_gptq(w, group, 4) if kind == "gptq" else O.quantize_awq(w, group)
    if kind == "gptq":
        return st, E.gptq_tensor(st.data, st.scales, st.zeros, st.len, group, shape)
    return st, E.awq_tensor(st.data.view(np.uint32), st.scales, st.zeros, st.len, group, shape)


@pytest.mark.parametrize("kind", ["q4", "gptq", "awq"])
def test_w4a16_a_side_like_reference_test(eng, kind):
    """compute/w4a16_test.go:32-124: m=2, k=32, n=3, modular fills, A = 4-bit weights, B = FP16 activations."""
    E, g = eng
    m, k, n = 2, 32, 3
    w, act = _fill(m * k, 7, 3), _fill(k * n, 5, 2)
    st, wt = _w4_tensor(E, kind, w, (m, k))
    ft = E.f16_tensor_from_f32(act, (k, n))
    assert np.array_equal(ft.bytes().view(np.uint16), O.f32_to_f16_bits(act))        # same fp16 rounding as the oracle
    before = g.launches
    got, matched = g.try_w4a16_matmul(wt, ft)
    assert matched and got.shape == (m, n) and g.launches > before
    want = O.matmul_w4a16(st, (m, k), O.new_float16_from_f32(act), (k, n))
    assert np.sqrt(np.mean((got - want) ** 2)) <= 1e-6                                # :255-348 bound
    assert np.abs(got - w.reshape(m, k) @ act.reshape(k, n)).max() <= 0.15            # :118-122 bound


@pytest.mark.parametrize("kind", ["q4", "gptq", "awq"])
@pytest.mark.parametrize("n,k,batch", [(64, 512, 1), (96, 4096, 3), (48, 1024, 8), (200, 1024, 16), (130, 2048, 40), (64, 512, 4)])
def test_engine_matmul_b_side_virtual_transpose(eng, kind, n, k, batch):
    """Engine.MatMul with the quantized weight as B: gpu_engine.go:2119-2126, logical [K,N], stored [N,K] (the
    "virtual transpose" of the reference's GPU engine).  From 3 activation rows on the engine takes the tensor-core
    kernel for GPTQ / AWQ.  (The W4A16 entry points treat a B-side weight differently: see the literal-layout
    tests below.)"""
    E, g = eng
    rng = U.seeded(n + k + batch)
    st, wt = _w4_tensor(E, kind, U.make_weights(rng, n, k), (k, n), group=128)
    xb = U.make_x_bits(rng, batch, k)
    xf = O.f16_bits_to_f32(xb).reshape(batch, k)
    xt = E.f16_tensor_from_bits(xb, (batch, k))
    assert E.host()
    got = g.matmul(xt, wt)
    if kind == "q4":
        ref = O.cpu_engine_matmul(xf, (batch, k), st, (k, n))                         # GemmF32Q4NT
    else:
        ref = U.ref_dense_a_side(st.slice().reshape(n, k), xf, n, k)
    assert U.rel_err(got, ref, U.absdot(st.slice().reshape(n, k), xf)) <= U.REL_TOL


@pytest.mark.parametrize("kind", ["q4", "gptq", "awq"])
def test_w4a16_b_side_is_a_literal_k_by_n_matrix_like_the_reference_test(eng, kind):
    """compute/w4a16_test.go:126-181 (TestW4A16_BWeights): m=2, k=32, n=3, A = FP16 activations [m,k], B = 4-bit
    weights of shape [k,n].  MatMulW4A16 dequantizes the flat slice and multiplies it as a row-major [K,N] matrix
    (compute/w4a16.go:107-119) -- no virtual transpose.  Same fills, same bound, and bit-for-bit the oracle."""
    E, g = eng
    m, k, n = 2, 32, 3
    act, w = _fill(m * k, 5, 2), _fill(k * n, 7, 3)
    st, wt = _w4_tensor(E, kind, w, (k, n), group=32)
    ft = E.f16_tensor_from_f32(act, (m, k))
    got, matched = g.try_w4a16_matmul(ft, wt)
    assert matched and got.shape == (m, n)
    want = O.matmul_w4a16(O.new_float16_from_f32(act), (m, k), st, (k, n))
    assert np.array_equal(got, want)                                                  # the same order of summation
    ref_act = O.f16_bits_to_f32(O.f32_to_f16_bits(act)).reshape(m, k)
    plain = ref_act.astype(np.float64) @ st.slice().reshape(k, n).astype(np.float64)
    assert np.abs(got - plain).max() <= 0.15                                          # the reference test's bound
    # the virtual-transpose reading of the same bytes is a different product: the two entry points must differ
    assert not np.allclose(got, ref_act @ st.slice().reshape(n, k).T)


@pytest.mark.parametrize("kind", ["q4", "gptq"])
@pytest.mark.parametrize("m,k,n", [(1, 256, 128), (5, 512, 96), (3, 128, 130)])
def test_w4a16_b_side_literal_layout_larger_shapes(eng, kind, m, k, n):
    E, g = eng
    rng = U.seeded(m + k + n)
    st, wt = _w4_tensor(E, kind, U.make_weights(rng, k, n), (k, n), group=128)
    xb = U.make_x_bits(rng, m, k)
    xt = E.f16_tensor_from_bits(xb, (m, k))
    got = g.matmul_w4a16(xt, wt)
    want = O.matmul_w4a16(O.Float16Storage(xb.ravel(), m * k), (m, k), st, (k, n))
    assert got.shape == (m, n) and np.array_equal(got, want)
    dst = g.device_tensor((m, n))
    res = g.matmul_async(xt, wt, dst=dst, mode=1)                                     # dst keeps its own buffer
    assert res.device_ptr == dst.device_ptr and np.array_equal(g.to_host(dst), want)


def test_matmul_is_pooled_asynchronous_and_capturable(eng):
    """compute/gpu_engine_matmul.go:89-100 and compute/gpu_engine.go:1179-1259: outputs come from the pool, nothing
    waits, and a run of MatMuls records into a CUDA graph.  After one warm-up pass the driver is not asked for
    memory again, in or out of capture."""
    E, g = eng
    import torch
    rng = U.seeded(4711)
    dims = [(256, 4096), (512, 2048), (96, 1024), (300, 4096), (128, 8192), (64, 512), (2048, 2048), (40, 3584)]
    ws, xs, refs = [], [], []
    for n, k in dims:
        st = O.quantize_gptq(U.make_weights(rng, n, k), 128, 4)
        wt = E.gptq_tensor(st.data, st.scales, st.zeros, st.len, 128, (k, n))
        xb = U.make_x_bits(rng, 1, k)
        xt = g.device_tensor((1, k), f16=True)
        pinned = torch.from_numpy(xb.view(np.int16).copy()).pin_memory()
        g.copy_from_host(xt, pinned.data_ptr(), k * 2)
        ws.append(wt)
        xs.append((xt, pinned))
        xf = O.f16_bits_to_f32(xb).reshape(1, k)
        refs.append((U.ref_dense_a_side(st.slice().reshape(n, k), xf, n, k), U.absdot(st.slice().reshape(n, k), xf)))
    g.upload_weights(ws)
    outs = [g.matmul_async(x, w) for (x, _), w in zip(xs, ws)]                        # warm-up pass: fills the pool
    g.sync()
    for o, (ref, absd) in zip(outs, refs):
        assert U.rel_err(g.to_host(o), ref, absd) <= U.REL_TOL
    dsts = [g.device_tensor((1, n)) for n, _ in dims]
    del outs                                                                          # buffers go back to the pool
    allocs = g.pool_driver_allocs
    launches = g.launches
    g.begin_capture()
    for (x, _), w, d in zip(xs, ws, dsts):
        r = g.matmul_async(x, w, dst=d)
        assert r.device_ptr == d.device_ptr                                           # dst's own storage, not re-homed
    tmp = g.matmul_async(xs[0][0], ws[0])                                             # a pool-backed result inside the capture
    graph = g.end_capture()
    assert g.launches == launches + len(dims) + 1 and g.pool_driver_allocs == allocs
    for _ in range(3):
        g.replay_graph(graph)
    g.sync()
    for d, (ref, absd) in zip(dsts, refs):
        assert U.rel_err(g.to_host(d), ref, absd) <= U.REL_TOL
    assert U.rel_err(g.to_host(tmp), refs[0][0], refs[0][1]) <= U.REL_TOL
    g.destroy_graph(graph)
    # host activations cannot be staged while capturing: an error, not a silent synchronisation
    g.begin_capture()
    with pytest.raises(E.EngineError, match="cannot be staged during stream capture"):
        g.matmul_async(E.f16_tensor_from_bits(U.make_x_bits(rng, 1, 4096), (1, 4096)), ws[0])
    g.destroy_graph(g.end_capture())
    # steady state outside capture: many calls, no new driver allocations
    del tmp
    for (x, _), w in zip(xs, ws):
        g.matmul_async(x, w)
    allocs = g.pool_driver_allocs
    for _ in range(20):
        for (x, _), w in zip(xs, ws):
            g.matmul_async(x, w)
    g.sync()
    assert g.pool_driver_allocs == allocs


def test_gpu_storage_views_share_a_reference_count_and_respect_the_pool_epoch(eng):
    """tensor/gpu_storage.go:25-46, :136-170, :467-529 and internal/gpuapi/mempool.go:26-50."""
    E, g = eng
    t = g.device_tensor((4, 256))
    assert t.refcount == 1
    v = t.view(256, 512, (2, 256))
    assert t.refcount == 2 and v.refcount == 2 and v.device_ptr == t.device_ptr + 256 * 4
    cached0, _ = g.pool_cached()
    t.free_storage()                                                                  # the view still holds the buffer
    assert v.refcount == 1 and g.pool_cached()[0] == cached0
    v.free_storage()                                                                  # last reference: back to the pool
    assert g.pool_cached()[0] == cached0 + 1
    v.free_storage()                                                                  # Free is idempotent
    assert g.pool_cached()[0] == cached0 + 1
    # a Free that arrives after the Reset that reclaimed its allocation is dropped (an engine of its own: Reset
    # reclaims every buffer of the pool)
    g = E.GPUEngine(0)
    keep = g.device_tensor((1, 1000))
    a = g.device_tensor((1, 1000))
    ptr = a.device_ptr
    epoch = g.pool_epoch
    g.pool_reset()
    assert g.pool_epoch == epoch + 1
    n_after_reset, _ = g.pool_cached()
    b = g.device_tensor((1, 1000))                                                    # may be handed a's bytes again
    a.free_storage()                                                                  # stale epoch: must not re-enter the free list
    assert g.pool_cached()[0] == n_after_reset - 1
    if b.device_ptr == ptr:
        c = g.device_tensor((1, 1000))
        assert c.device_ptr != ptr                                                    # b's buffer was not issued twice


def test_w4a16_not_matched_and_errors(eng):
    """compute/w4a16_test.go:183-205: float32 x float32 is not a W4A16 pair."""
    E, g = eng
    a = E.cpu_tensor(np.ones(8, np.float32), (2, 4))
    b = E.cpu_tensor(np.ones(8, np.float32), (4, 2))
    res, matched = g.try_w4a16_matmul(a, b)
    assert res is None and not matched
    with pytest.raises(E.EngineError, match="MatMulW4A16: inputs are not W4A16"):
        g.matmul_w4a16(a, b)
    with pytest.raises(E.EngineError, match="neither operand is a quantized weight"):
        g.matmul(a, b)
    st = O.quantize_q4(_fill(64, 7, 3))
    wt = E.q4_tensor(st.blocks, 64, (2, 32))
    with pytest.raises(E.EngineError, match=r"invalid shapes for matrix multiplication: a.Shape\(\)=\[2 32\], b.Shape\(\)=\[16 1\]"):
        g.matmul(wt, E.cpu_tensor(np.ones(16, np.float32), (16, 1)))
    with pytest.raises(E.EngineError, match="Q4_0 raw data too short: need 36 bytes for 2 blocks, got 18"):
        E.q4_tensor(st.blocks[:18], 64, (2, 32))
    with pytest.raises(E.EngineError, match="numElements must be positive"):
        E.iq4nl_tensor(np.zeros(18, np.uint8), 0, (1, 32))
    with pytest.raises(E.EngineError, match="tensor: TernaryStorage value must be -1, 0, or 1"):
        E.ternary_tensor([2], (1, 1))
    # no CPU fallback: a shape the kernels refuse surfaces as the kernel error (K % 32 != 0)
    t48 = E.q8_tensor(np.ones(3, np.float32), np.ones(96, np.int8), 96, (2, 48))
    with pytest.raises(E.EngineError, match=r"ztq_gemv_q8_0 kernel failed \(cuda error 1\)"):
        g.matmul(t48, E.cpu_tensor(np.ones(48, np.float32), (48, 1)))


@pytest.mark.parametrize("m,k,n", [(4, 32, 8), (1, 64, 1), (3, 128, 5), (64, 4096, 1)])
def test_q4_q8_a_side_float32_like_xblas_tests(eng, m, k, n):
    """internal/xblas/gemm_quant_test.go:45-138 / compute/cpu_engine_quant_test.go:12-73 through Engine.MatMul."""
    E, g = eng
    a, b = _fill(m * k, 7, 3), _fill(k * n, 5, 2)
    for st, t in ((O.quantize_q4(a), None), (O.quantize_q8(a), None)):
        if isinstance(st, O.Q4Storage):
            t = E.q4_tensor(st.blocks, st.len, (m, k))
        else:
            t = E.q8_tensor(st.scales(), st.codes(), st.len, (m, k))
        got = g.matmul(t, E.cpu_tensor(b, (k, n)))
        ref = O.cpu_engine_matmul(st, (m, k), b, (k, n))
        absd = U.absdot(st.slice().reshape(m, k), b.reshape(k, n).T).T
        assert got.shape == (m, n) and U.rel_err(got, ref, absd) <= U.REL_TOL
        assert np.abs(got - a.reshape(m, k) @ b.reshape(k, n)).max() <= (0.15 if isinstance(st, O.Q4Storage) else 0.02) * max(1, k / 32)


def test_iq4nl_and_q8_b_side_and_dst_contract(eng):
    E, g = eng
    rng = U.seeded(77)
    n, k, batch = 80, 1024, 2
    w = U.make_weights(rng, n, k)
    xb = U.make_x_bits(rng, batch, k)
    xf = O.f16_bits_to_f32(xb).reshape(batch, k)
    iq = O.make_iq4nl_blocks(w)
    got = g.matmul(E.cpu_tensor(xf, (batch, k)), E.iq4nl_tensor(iq.raw, iq.len, (k, n)))
    assert U.rel_err(got, U.ref_dense_a_side(iq.slice().reshape(n, k), xf, n, k), U.absdot(iq.slice().reshape(n, k), xf)) <= U.REL_TOL
    q8 = O.quantize_q8(w)
    t8 = E.q8_tensor(q8.scales(), q8.codes(), q8.len, (k, n))
    ref8 = O.cpu_engine_matmul(xf, (batch, k), q8, (k, n))
    # dst contract (compute/gpu_kernels.go:248-272): the result lands in dst's own storage, which is not re-homed
    dst = E.cpu_tensor(np.full(batch * n, np.nan, np.float32), (batch, n))
    got8 = g.matmul(E.f16_tensor_from_bits(xb, (batch, k)), t8, dst=dst)
    assert got8.shape == (batch, n) and U.rel_err(got8, ref8, U.absdot(q8.slice().reshape(n, k), xf)) <= U.REL_TOL
    with pytest.raises(E.EngineError, match="dst storage does not match"):
        g.matmul(E.cpu_tensor(xf, (batch, k)), t8, dst=E.cpu_tensor(np.zeros(3, np.float32), (3,)))


@pytest.mark.parametrize("n,k,batch", [(96, 4096, 3), (200, 1024, 8), (130, 2048, 17), (64, 544, 4)])
def test_engine_matmul_q8_b_side_batches(eng, n, k, batch):
    """Engine.MatMul with Q8_0 weights as B and 3 or more fp16 activation rows: the tensor-core kernel on the raw
    blocks when K % 512 == 0, GEMV passes otherwise; both against CPUEngine.MatMul of the oracle."""
    E, g = eng
    rng = U.seeded(3 * n + k + batch)
    q8 = O.quantize_q8(U.make_weights(rng, n, k))
    xb = U.make_x_bits(rng, batch, k)
    xf = O.f16_bits_to_f32(xb).reshape(batch, k)
    t8 = E.q8_tensor(q8.scales(), q8.codes(), q8.len, (k, n))
    ref = O.cpu_engine_matmul(xf, (batch, k), q8, (k, n))
    got = g.matmul(E.f16_tensor_from_bits(xb, (batch, k)), t8)
    assert got.shape == (batch, n) and U.rel_err(got, ref, U.absdot(q8.slice().reshape(n, k), xf)) <= U.REL_TOL


def test_ternary_gemv_gpu_known_answers(eng):
    """compute/ternary_gemv_gpu_test.go repeats compute/ternary_gemv_test.go:25-141 through TernaryGEMVGPU."""
    E, g = eng
    cases = [([1, 0, -1, 1, -1, 1, 0, 0, 0, -1, 1, -1], [2.0, 3.0, 4.0, 5.0], 3, 4, [3.0, 1.0, -4.0]),
             ([1, -1, 0, 1, -1, 0, 1, -1, 0, 1], [1.0, 2.0, 3.0, 4.0, 5.0], 2, 5, [-2.0, 4.0]),
             ([-1], [7.5], 1, 1, [-7.5]), ([1], [7.5], 1, 1, [7.5])]
    for vals, x, r, c, want in cases:
        t = E.ternary_tensor(vals, (r, c))
        assert g.ternary_gemv_gpu(t, x, r, c).tolist() == want
        assert t.resident                                               # uploaded once, cached on the storage
    rng = U.seeded(3)
    rows, cols = 128, 256
    vals = rng.integers(-1, 2, size=rows * cols).astype(np.int8)
    x = (rng.random(cols, dtype=np.float32) * 2 - 1).astype(np.float32)
    t = E.ternary_tensor(vals, (rows, cols))
    got = g.ternary_gemv_gpu(t, x, rows, cols)
    want = O.ternary_gemv(O.new_ternary_from(vals), x, rows, cols)
    assert np.abs(got - want).max() <= 1e-5
    with pytest.raises(E.EngineError, match="rows\\*cols does not match"):
        g.ternary_gemv_gpu(t, x, rows, cols + 1)
    # row scales (benchmark configuration) through Engine.MatMul, weights on B
    sc = O.f32_to_f16_bits(rng.uniform(0.01, 0.05, rows).astype(np.float32))
    ts = E.ternary_tensor(vals, (cols, rows), row_scale_bits=sc)
    xb = U.make_x_bits(rng, 1, cols)
    xf = O.f16_bits_to_f32(xb).reshape(1, cols)
    got = g.matmul(E.f16_tensor_from_bits(xb, (1, cols)), ts)
    ref = U.ref_ternary(O.new_ternary_from(vals), xf, sc, rows, cols)
    wd = vals.reshape(rows, cols).astype(np.float32) * O.f16_bits_to_f32(sc)[:, None]
    assert U.rel_err(got, ref, U.absdot(wd, xf)) <= U.REL_TOL


def test_engine_quantizers_and_upload_weights_residency(eng):
    E, g = eng
    rng = U.seeded(11)
    n, k = 32, 512
    w = U.make_weights(rng, n, k)
    q4 = g.quantize("q4", w, (n, k))
    assert np.array_equal(q4.bytes(), O.quantize_q4(w).blocks)                       # bit-identical to tensor.QuantizeQ4
    q8 = g.quantize("q8", w, (n, k))
    assert np.array_equal(q8.bytes(), O.quantize_q8(w).blocks)
    for kind, ref in (("gptq", O.quantize_gptq(w, 128, 4)), ("awq", O.quantize_awq(w, 128))):
        t = g.quantize(kind, w, (n, k))
        assert np.array_equal(t.bytes(0), ref.data)
        assert np.array_equal(t.bytes(1).view(np.uint16), ref.scales) and np.array_equal(t.bytes(2).view(np.uint16), ref.zeros)
    iq = O.make_iq4nl_blocks(w)
    tern = E.ternary_tensor(rng.integers(-1, 2, size=n * k).astype(np.int8), (n, k))
    weights = [q4, q8, g.quantize("gptq", w, (n, k)), g.quantize("awq", w, (n, k)), E.iq4nl_tensor(iq.raw, iq.len, (n, k)), tern]
    assert not any(t.resident for t in weights)
    g.upload_weights(weights)                                                        # packed residency for every format
    assert all(t.resident for t in weights)
    xb = U.make_x_bits(rng, 1, k)
    xt = E.f16_tensor_from_bits(xb.T.copy(), (k, 1))
    for t in weights:                                                                # weights on A, resident
        assert g.matmul(t, xt).shape == (n, 1)
    with pytest.raises(E.EngineError, match="multiple of 32"):
        g.quantize("q4", np.ones(33, np.float32), (33,))


@pytest.mark.parametrize("n,k,batch", [(64, 2048, 1), (100, 4096, 3)])
def test_q4k_through_the_engine(eng, n, k, batch):
    """Q4KStorage on the B side (xblas.GemmF32Q4KNT, cpu_engine.go:2391-2399) and, for one column, on the A side
    (GemmQ4KF32, cpu_engine.go:2305-2311); UploadWeights keeps the packed super-blocks on the device."""
    E, g = eng
    rng = U.seeded(n + k + batch + 5)
    st = O.quantize_q4k(U.make_weights(rng, n, k))
    wt = E.q4k_tensor(st.raw, n * k, (k, n))                                          # logical [K, N], stored [N, K]
    g.upload_weights([wt])
    x = rng.standard_normal((batch, k)).astype(np.float32)
    got = g.matmul(E.cpu_tensor(x, (batch, k)), wt)
    ref = O.gemm_f32_q4k_nt(batch, n, k, x, st, ncpu=1).reshape(batch, n)
    absd = U.absdot(st.slice().reshape(n, k), x)
    assert got.shape == (batch, n) and U.rel_err(got, ref, absd) <= U.REL_TOL
    if batch == 1:
        wa = E.q4k_tensor(st.raw, n * k, (n, k))
        got_a = g.matmul(wa, E.cpu_tensor(x.reshape(k, 1), (k, 1)))
        ref_a = O.gemm_q4k_f32(n, 1, k, st, x.reshape(-1)).reshape(n, 1)
        assert got_a.shape == (n, 1) and U.rel_err(got_a.reshape(1, n), ref_a.reshape(1, n), absd) <= U.REL_TOL
    with pytest.raises(RuntimeError, match="Q4_K raw data too short"):
        E.q4k_tensor(st.raw[:100], n * k, (k, n))


def test_q5k_through_the_engine(eng):
    """Q5KStorage on the B side (xblas.GemmF32Q5KNT, cpu_engine.go:2435-2449)."""
    E, g = eng
    n, k, batch = 72, 2048, 2
    rng = U.seeded(123)
    st = O.make_q5k_blocks(U.make_weights(rng, n, k))
    wt = E.q5k_tensor(st.raw, n * k, (k, n))
    g.upload_weights([wt])
    x = rng.standard_normal((batch, k)).astype(np.float32)
    got = g.matmul(E.cpu_tensor(x, (batch, k)), wt)
    ref = O.gemm_f32_q5k_nt(batch, n, k, x, st, ncpu=1).reshape(batch, n)
    assert got.shape == (batch, n) and U.rel_err(got, ref, U.absdot(st.slice().reshape(n, k), x)) <= U.REL_TOL
    with pytest.raises(RuntimeError, match="Q5_K raw data too short"):
        E.q5k_tensor(st.raw[:100], n * k, (k, n))


def test_q6k_through_the_engine(eng):
    """Q6KStorage on the B side (xblas.GemmF32Q6KNT, cpu_engine.go:2475-2489)."""
    E, g = eng
    n, k, batch = 40, 4096, 2
    rng = U.seeded(321)
    st = O.make_q6k_blocks(U.make_weights(rng, n, k))
    wt = E.q6k_tensor(st.raw, n * k, (k, n))
    g.upload_weights([wt])
    x = rng.standard_normal((batch, k)).astype(np.float32)
    got = g.matmul(E.cpu_tensor(x, (batch, k)), wt)
    ref = O.gemm_f32_q6k_nt(batch, n, k, x, st, ncpu=1).reshape(batch, n)
    assert got.shape == (batch, n) and U.rel_err(got, ref, U.absdot(st.slice().reshape(n, k), x)) <= U.REL_TOL
    with pytest.raises(RuntimeError, match="Q6_K raw data too short"):
        E.q6k_tensor(st.raw[:100], n * k, (k, n))
