"""The allocation-free split-K entry point against the workspace-taking one.

Some callers of this library cannot allocate device memory when they need a GEMV: a runtime that serves
all buffers from an arena fixed at start-up, or code that is already capturing a CUDA graph.  For them
ztq_gemv_w4g_splitk_static keeps its partial sums in an array built into the library.  The array is
shared by all calls and never cleared, so the check runs the call twice in a row, with a different
problem in between, and expects the bits of the workspace version every time."""
import numpy as np
import pytest
import torch

from oracle import oracle as O
from tests import util as U
from ztensor_b200 import _lib
from ztensor_b200 import kernels as K

pytestmark = pytest.mark.gpu


def _case(seed, n, k):
    from tests import gpu_util as G
    rng = U.seeded(seed)
    st = O.quantize_gptq(U.make_weights(rng, n, k), 128, 4)
    xb = U.make_x_bits(rng, 1, k)
    qd, meta = G.upload_w4g(st)
    xf = O.f16_bits_to_f32(xb).reshape(1, k)
    ref = U.ref_dense_a_side(st.slice().reshape(n, k), xf, n, k)
    return qd, meta, G.x_dev(xb), ref, U.absdot(st.slice().reshape(n, k), xf)


def test_static_scratch_splitk_matches_workspace_splitk_twice_in_a_row():
    n, k, splits = 96, 8192, 8
    qd, meta, x, ref, absd = _case(501, n, k)
    ws = torch.empty(K.splitk_workspace_bytes(n, splits) // 4, dtype=torch.float32, device="cuda")
    want = torch.empty(1, n, dtype=torch.float32, device="cuda")
    K.gemv_w4g_splitk(qd, meta, x, want, n, k, 128, splits, ws, K.Y_F32)
    torch.cuda.synchronize()
    want = want.cpu().numpy()
    assert U.rel_err(want, ref, absd) <= U.REL_TOL

    other = _case(502, 40, 4096)                       # a different problem leaves other contents in the scratch
    # set-up call: the first call on a device looks up the scratch array (and loads the kernels); it comes before
    # the measurement of free memory, the way a caller makes it before its arena is frozen
    y0 = torch.empty(1, n, dtype=torch.float32, device="cuda")
    K.gemv_w4g_splitk_static(qd, meta, x, y0, n, k, 128, splits, K.Y_F32)
    torch.cuda.synchronize()
    before = torch.cuda.memory_allocated()
    for attempt in range(2):
        y = torch.full((1, n), float("nan"), dtype=torch.float32, device="cuda")
        torch.cuda.synchronize()
        mark = torch.cuda.memory_allocated()
        free_before, _ = torch.cuda.mem_get_info()     # the driver's view: sees a cudaMalloc inside the library too
        K.gemv_w4g_splitk_static(qd, meta, x, y, n, k, 128, splits, K.Y_F32)
        torch.cuda.synchronize()
        free_after, _ = torch.cuda.mem_get_info()
        assert free_after >= free_before, "the call took device memory from the driver"
        assert torch.cuda.memory_allocated() == mark  # nothing was allocated through torch either
        got = y.cpu().numpy()
        assert U.rel_err(got, want, absd) <= U.REL_TOL, f"call {attempt}"
        assert np.array_equal(got, want), f"call {attempt}: same kernels, same order: same bits"
        y2 = torch.empty(1, 40, dtype=torch.float32, device="cuda")
        K.gemv_w4g_splitk_static(other[0], other[1], other[2], y2, 40, 4096, 128, 4, K.Y_F32)
        torch.cuda.synchronize()
        assert U.rel_err(y2.cpu().numpy(), other[3], other[4]) <= U.REL_TOL
    assert torch.cuda.memory_allocated() >= before
    assert K.device_error() == 0


def test_static_scratch_rejects_problems_beyond_its_size():
    n = K.STATIC_SCRATCH_BYTES // 4 // 2 + 1            # n * 2 splits * 4 bytes is just over the limit
    d = torch.zeros(64, dtype=torch.uint8, device="cuda")
    rc = _lib.lib().ztq_gemv_w4g_splitk_static(d.data_ptr(), d.data_ptr(), d.data_ptr(), d.data_ptr(), n, 1024, 128, 2, 0, None)
    assert rc == 1                                       # cudaErrorInvalidValue, nothing launched
    with pytest.raises(RuntimeError, match=r"ztq_gemv_w4g_splitk_static kernel failed \(cuda error 1\)"):
        K.gemv_w4g_splitk_static(d, d, d, d, n, 1024, 128, 2)
