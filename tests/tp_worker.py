"""Worker of the tensor-parallel parity test (launched by torchrun, one rank per GPU).

A GPTQ-4bit [N, K] matrix is quantized by the oracle on every rank from the same
seed; rank r holds columns [r K/w, (r+1) K/w) (row-parallel shard).  The fused
GEMV+all-reduce must reproduce the oracle's full product within the parity
tolerance, be bit-identical on all ranks and from call to call, and agree with
the NCCL path."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from oracle import oracle as O            # noqa: E402
from tests import gpu_util as G           # noqa: E402
from tests import util as U               # noqa: E402
from ztensor_b200 import kernels as K     # noqa: E402
from ztensor_b200.collective import FusedAllReduce   # noqa: E402


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    ar = FusedAllReduce(max_elems=16 * 8192)
    ok = True
    cases = [(512, 4096 * world, 1), (2048, 1024 * world, 1), (1000, 2048 * world, 2), (300, 3584 * world, 1)]
    # the row-parallel projections of the 70B-shaped stack as this world size shards them (O: K = 8192, down:
    # K = 28672): every CTA walks several tiles and passes, the cells carry 8192 rows
    cases += [(8192, 8192, 1), (8192, 28672, 1)]
    # three or more activation rows: the tensor-core kernel with the all-reduce in its epilogue, alternating with the
    # GEMV launches above on the same slots and sequence word (K split and unsplit plans, 8 and 16 columns, a ragged
    # last row tile)
    cases += [(8192, 8192, 8), (8192, 28672, 8), (1000, 2048 * world, 5), (8192, 8192, 1), (8192, 28672, 16)]
    for ci, (n, k, batch) in enumerate(cases):
        tc = batch >= 3
        if ci == 3:
            ar.resync()                    # sequence back to 0 on every rank, buffers clean: the next launches still agree
        rng = U.seeded(n + k)
        st = O.quantize_gptq(U.make_weights(rng, n, k), 128, 4)
        xb = U.make_x_bits(rng, batch, k)
        xf = O.f16_bits_to_f32(xb).reshape(batch, k)
        act = O.Float16Storage(xb.T.copy().ravel(), batch * k)
        ref = np.ascontiguousarray(O.matmul_w4a16(st, (n, k), act, (k, batch)).T)
        absd = U.absdot(st.slice().reshape(n, k), xf)
        ks = k // world
        c0 = rank * ks
        data = st.data.reshape(n, k // 2)[:, c0 // 2:(c0 + ks) // 2].copy()
        sc = st.scales.reshape(n, k // 128)[:, c0 // 128:(c0 + ks) // 128].copy()
        zr = st.zeros.reshape(n, k // 128)[:, c0 // 128:(c0 + ks) // 128].copy()
        shard = O.GroupQuantStorage("gptq", data.ravel(), sc.ravel(), zr.ravel(), n * ks, 128)
        qd, meta = G.upload_w4g(shard)
        x = G.x_dev(np.ascontiguousarray(xb[:, c0:c0 + ks]))
        y = torch.zeros(batch, n, dtype=torch.float32, device="cuda")
        outs = []
        for _ in range(3):
            y.fill_(float("nan"))
            if tc:
                ws = torch.empty(K.gemm_w4g_tc_workspace_bytes(n, ks, batch), dtype=torch.uint8, device="cuda")
                K.gemm_w4g_tc_allreduce(qd, meta, x, y, n, ks, 128, batch, ws, ar, K.Y_F32)
            else:
                K.gemv_w4g_allreduce(qd, meta, x, y, n, ks, 128, batch, ar, K.Y_F32)
            torch.cuda.synchronize()
            outs.append(y.cpu().numpy().copy())
        e = U.rel_err(outs[0], ref, absd)
        same_calls = all(np.array_equal(outs[0], o) for o in outs[1:])
        gathered = [torch.zeros_like(y) for _ in range(world)]
        dist.all_gather(gathered, y)
        same_ranks = all(torch.equal(gathered[0], g) for g in gathered[1:])
        y2 = torch.zeros(batch, n, dtype=torch.float32, device="cuda")
        if tc:
            K.gemm_w4g_tc(qd, meta, x, y2, n, ks, 128, batch, ws, K.Y_F32)
        else:
            K.gemv_w4g(qd, meta, x, y2, n, ks, 128, batch, K.Y_F32)
        dist.all_reduce(y2)
        e_nccl = U.rel_err(outs[0], y2.cpu().numpy(), absd)
        good = e <= U.REL_TOL and same_calls and same_ranks and e_nccl <= U.REL_TOL and K.device_error() == 0
        ok = ok and good
        if rank == 0:
            print(f"tp{world} {'tensor-core ' if tc else ''}n={n} k={k} b={batch}: err={e:.2e} vs_nccl={e_nccl:.2e} same_calls={same_calls} "
                  f"same_ranks={same_ranks} -> {'ok' if good else 'FAIL'}", flush=True)
    # the host library's own NCCL binding (libnccl loaded by libztq_host.so, the id handed over by pointer): fp16 and
    # fp32 all-reduces agree with torch.distributed's
    from ztensor_b200 import nccl as HN
    ids = [HN.get_unique_id() if rank == 0 else None]
    dist.broadcast_object_list(ids, src=0)
    comm = HN.Comm(ids[0], world, rank)
    for dt in (torch.float16, torch.float32):
        g = torch.Generator(device="cuda")
        g.manual_seed(100 + rank)
        a = torch.randn(8192, device="cuda", generator=g).to(dt)
        b = a.clone()
        comm.all_reduce_tensor(a)
        dist.all_reduce(b)
        torch.cuda.synchronize()
        same = torch.equal(a, b)
        ok = ok and same
        if rank == 0:
            print(f"host-library ncclAllReduce {dt}: {'ok' if same else 'FAIL'}", flush=True)
    comm.destroy()
    ar.close()
    if rank == 0:
        print("TP_PARITY_OK" if ok else "TP_PARITY_FAIL", flush=True)
    sys.stdout.flush()
    os._exit(0 if ok else 1)


if __name__ == "__main__":
    main()
