"""Run one GEMV shape a few times on random packed weights: `python -m ztensor_b200.probe w4g 57344 8192`.

A small driver for profilers and for checking that a shape launches: it calls
the same C-ABI entry point, with the same launch plan, as the engine and the
benchmark do.  Weights are random bytes with sane scales (no parity check here).

    python -m ztensor_b200.probe <w4g|w4g_tc|w4g_splitk|q4_0|iq4nl|q8_0|ternary> N K [batch] [flags] [launches]

`w4g_tc` is the tensor-core entry point (ztq_gemm_w4g_tc), `w4g_splitk` the split-K GEMV (the batch argument
is then the number of K slices); the others are the GEMV entry points.
"""
from __future__ import annotations

import sys

import torch

from . import kernels as K


def make_case(fmt: str, n: int, k: int, batch: int, flags: int, nbuf: int = 3, dev: str = "cuda"):
    def rnd(nbytes):
        return torch.randint(0, 256, (nbytes,), dtype=torch.uint8, device=dev)

    x = torch.randn(batch, k, device=dev).half()
    y = torch.empty(batch, n, device=dev, dtype=torch.half)
    if fmt in ("w4g", "w4g_tc", "w4g_splitk"):
        qd = [rnd(n * k // 2) for _ in range(nbuf)]
        meta = [(torch.rand(n * k // 128, 2, device=dev) * 0.01 + 0.001).half().view(torch.uint8).reshape(-1)
                for _ in range(nbuf)]
        if fmt == "w4g_splitk":
            splits = batch
            x1 = torch.randn(1, k, device=dev).half()
            y1 = torch.empty(1, n, device=dev, dtype=torch.half)
            ws = torch.empty(K.splitk_workspace_bytes(n, splits), dtype=torch.uint8, device=dev)
            return lambda i: K.gemv_w4g_splitk(qd[i % nbuf], meta[i % nbuf], x1, y1, n, k, 128, splits, ws, flags)
        if fmt == "w4g_tc":
            ws = torch.empty(K.gemm_w4g_tc_workspace_bytes(n, k, batch), dtype=torch.uint8, device=dev)
            return lambda i: K.gemm_w4g_tc(qd[i % nbuf], meta[i % nbuf], x, y, n, k, 128, batch, ws, flags)
        return lambda i: K.gemv_w4g(qd[i % nbuf], meta[i % nbuf], x, y, n, k, 128, batch, flags)
    if fmt in ("q4_0", "iq4nl"):
        nb = n * k // 32
        off = K.q4_gpu_data_offset(nb)
        bufs = []
        for _ in range(nbuf):
            b = rnd(off + nb * 16)
            b[:nb * 2] = (torch.rand(nb, device=dev) * 0.01).half().view(torch.uint8).reshape(-1)
            bufs.append(b)
        fn = K.gemv_q4_0 if fmt == "q4_0" else K.gemv_iq4nl
        return lambda i: fn(bufs[i % nbuf], off, x, y, n, k, batch, flags)
    if fmt == "q8_0":
        nb = n * k // 32
        bufs = []
        for _ in range(nbuf):
            b = rnd(nb * 36).view(-1, 36)
            b[:, :4] = (torch.rand(nb, 1, device=dev) * 0.001).float().view(torch.uint8).reshape(-1, 4)
            bufs.append(b.reshape(-1))
        return lambda i: K.gemv_q8_0(bufs[i % nbuf], x, y, n, k, batch, flags)
    if fmt == "ternary":
        bufs = []
        for _ in range(nbuf):
            hi = rnd(n * k // 4) & 0xAA                       # code 2 where set
            lo = rnd(n * k // 4) & 0x55 & ~(hi >> 1)          # code 1 elsewhere, never code 3
            bufs.append(hi | lo)
        sc = (torch.rand(n, device=dev) * 0.04 + 0.01).half()
        return lambda i: K.gemv_ternary(bufs[i % nbuf], sc, x, y, n, k, batch, flags)
    raise SystemExit(f"unknown format {fmt}")


def main(argv):
    if len(argv) < 4:
        raise SystemExit(__doc__)
    fmt, n, k = argv[1], int(argv[2]), int(argv[3])
    batch = int(argv[4]) if len(argv) > 4 else 1
    flags = int(argv[5]) if len(argv) > 5 else 0
    launches = int(argv[6]) if len(argv) > 6 else 6
    run = make_case(fmt, n, k, batch, flags)
    for i in range(launches):
        run(i)
    torch.cuda.synchronize()
    print(f"{fmt} N={n} K={k} batch={batch}: {launches} launches, device error {K.device_error()}")


if __name__ == "__main__":
    main(sys.argv)
