"""The fused all-reduce of the row-parallel kernels on ONE GPU.

The {value, tag} cells a peer would push are written into this rank's slot buffer before the launch, with the tags of
the launches to come, and the "peer's" slot buffer is a second local buffer.  The kernel under test therefore never
waits for another kernel: it pushes its own cells to both buffers, finds every cell it polls already there, adds in
rank order and stores.  Checked: y == own partial + peer partial (exact in fp32, rank order), the cells that reached
the peer buffer (values, tags, parity), the launch sequence word, for the GEMV kernels and for the tensor-core kernel
(K split and unsplit, 8 and 16 columns, ragged last row tile), alternating on one descriptor.
"""
import ctypes as C

import numpy as np
import pytest
import torch

from oracle import oracle as O
from tests import util as U

pytestmark = pytest.mark.gpu


def _mods():
    from tests import gpu_util as G
    from ztensor_b200 import kernels as K
    from ztensor_b200.collective import ZtqAllReduce
    return G, K, ZtqAllReduce


class _LocalAR:
    """world = 2, this process is `rank`; the other rank's partial sums are supplied by the test."""

    def __init__(self, max_elems, rank):
        _, _, ZtqAllReduce = _mods()
        self.world, self.rank, self.stride = 2, rank, (max_elems + 31) // 32 * 32
        cells = 2 * self.world * self.stride
        self.own = torch.zeros(cells, 2, dtype=torch.int32, device="cuda")     # {value bits, tag}
        self.peer = torch.zeros(cells, 2, dtype=torch.int32, device="cuda")
        self.state = torch.zeros(4, dtype=torch.int32, device="cuda")
        self.desc = ZtqAllReduce()
        self.desc.world, self.desc.rank, self.desc.slot_stride = self.world, rank, self.stride
        self.desc.slots[rank] = self.own.data_ptr()
        self.desc.slots[1 - rank] = self.peer.data_ptr()
        self.desc.state = self.state.data_ptr()
        self.seq = 0

    def ptr(self):
        return C.byref(self.desc)

    def region(self, buf, seq, r):
        o = ((seq & 1) * self.world + r) * self.stride
        return buf[o:o + self.stride]

    def expect_peer(self, partial: torch.Tensor):
        """Write the other rank's cells of the next launch (partial: [batch, N] float32 on the device)."""
        reg = self.region(self.own, self.seq, 1 - self.rank)
        flat = partial.reshape(-1)
        reg[:flat.numel(), 0] = flat.view(torch.int32)
        reg[:flat.numel(), 1] = self.seq + 1
        torch.cuda.synchronize()

    def check_pushed(self, partial: torch.Tensor):
        """After a launch: both buffers hold this rank's cells with this launch's tag."""
        flat = partial.reshape(-1)
        for buf in (self.own, self.peer):
            reg = self.region(buf, self.seq, self.rank)
            assert torch.equal(reg[:flat.numel(), 0], flat.view(torch.int32))
            assert bool((reg[:flat.numel(), 1] == self.seq + 1).all())
        self.seq += 1
        st = self.state.cpu().numpy()
        assert st[0] == self.seq and st[1] == 0


def _w4g(n, k, batch, seed):
    G, K, _ = _mods()
    rng = U.seeded(seed)
    st = O.quantize_gptq(U.make_weights(rng, n, k), 128, 4)
    xb = U.make_x_bits(rng, batch, k)
    qd, meta = G.upload_w4g(st)
    return st, xb, qd, meta, G.x_dev(xb)


@pytest.mark.parametrize("rank", [0, 1])
def test_gemv_and_tensor_core_allreduce_alternate_on_one_descriptor(rank):
    G, K, _ = _mods()
    ar = _LocalAR(16 * 8192, rank)
    g = torch.Generator(device="cuda")
    g.manual_seed(5 + rank)
    # (n, k, batch): GEMV, tensor cores unsplit and split, 16 columns, a ragged tile, GEMV again, two rows per pass
    cases = [(2048, 4096, 1), (8192, 1024, 8), (8192, 3584, 8), (1000, 2048, 5), (4096, 4096, 16), (512, 8192, 2),
             (8192, 4096, 3)]
    for ci, (n, k, batch) in enumerate(cases):
        st, xb, qd, meta, x = _w4g(n, k, batch, 77 * ci + n + k)
        tc = batch >= 3
        own = torch.empty(batch, n, dtype=torch.float32, device="cuda")
        if tc:
            ws = torch.empty(K.gemm_w4g_tc_workspace_bytes(n, k, batch), dtype=torch.uint8, device="cuda")
            K.gemm_w4g_tc(qd, meta, x, own, n, k, 128, batch, ws, K.Y_F32)
        else:
            K.gemv_w4g(qd, meta, x, own, n, k, 128, batch, K.Y_F32)
        other = torch.randn(batch, n, device="cuda", generator=g) * own.abs().mean()
        for rep in range(2):                                   # both parities of the cell buffers
            ar.expect_peer(other)
            y = torch.full((batch, n), float("nan"), dtype=torch.float32, device="cuda")
            if tc:
                K.gemm_w4g_tc_allreduce(qd, meta, x, y, n, k, 128, batch, ws, ar, K.Y_F32)
            else:
                K.gemv_w4g_allreduce(qd, meta, x, y, n, k, 128, batch, ar, K.Y_F32)
            torch.cuda.synchronize()
            assert K.device_error() == 0
            want = (own + other) if rank == 0 else (other + own)           # rank order; fp32 addition commutes anyway
            assert torch.equal(y, want), f"case {ci} rep {rep}: max diff {(y - want).abs().max().item()}"
            ar.check_pushed(own)
        # fp16 output of the reduced sum
        ar.expect_peer(other)
        y16 = torch.full((batch, n), float("nan"), dtype=torch.float16, device="cuda")
        if tc:
            K.gemm_w4g_tc_allreduce(qd, meta, x, y16, n, k, 128, batch, ws, ar, 0)
        else:
            K.gemv_w4g_allreduce(qd, meta, x, y16, n, k, 128, batch, ar, 0)
        torch.cuda.synchronize()
        assert torch.equal(y16, (own + other).half())
        ar.check_pushed(own)


def test_tensor_core_allreduce_argument_checks():
    G, K, _ = _mods()
    ar = _LocalAR(4 * 1024, 0)
    st, xb, qd, meta, x = _w4g(1024, 1024, 4, 9)
    ws = torch.empty(K.gemm_w4g_tc_workspace_bytes(1024, 1024, 4), dtype=torch.uint8, device="cuda")
    y = torch.zeros(4, 1024, dtype=torch.float32, device="cuda")
    with pytest.raises(RuntimeError):                          # fp16 operands have no all-reduce variant
        K.gemm_w4g_tc_allreduce(qd, meta, x, y, 1024, 1024, 128, 4, ws, ar, K.Y_F32 | K.FP32_DECODE)
    with pytest.raises(RuntimeError):                          # nor do the fp32-decode GEMV kernels
        K.gemv_w4g_allreduce(qd, meta, x, y, 1024, 1024, 128, 1, ar, K.Y_F32 | K.FP32_DECODE)
    small = _LocalAR(1024, 0)                                   # slots too small for 4 x 1024 cells
    with pytest.raises(RuntimeError):
        K.gemm_w4g_tc_allreduce(qd, meta, x, y, 1024, 1024, 128, 4, ws, small, K.Y_F32)
    torch.cuda.synchronize()
    assert K.device_error() == 0 and int(ar.state[0].item()) == 0
