"""Per-shape throughput of the quantized GEMV kernels: every (format, K -> N, batch) of the benchmark
configurations, as achieved GB/s of algorithmic bytes (packed weights + scales + fp16 x + fp16 y, each once).

Method: per shape, enough distinct weight buffers to exceed L2 several times over (> 600 MB in total) are
cycled through by `iters` back-to-back launches recorded into one CUDA graph; one replay is timed with CUDA
events on the launching stream after a warm-up replay.  The figure therefore includes the launch-to-launch
gap of a stream of dependent kernels (programmatic dependent launch), which is what a decode step pays.
Weights are random codes with small positive scales: throughput does not depend on the values.
"""
from __future__ import annotations

import torch

from . import kernels as K

# K -> N of the Llama-3-8B decode projections (QKV, O, gate, up, down) and of the 70B ones
SHAPES_8B = [(6144, 4096), (4096, 4096), (14336, 4096), (4096, 14336)]
SHAPES_70B = [(10240, 8192), (8192, 8192), (57344, 8192), (8192, 28672)]


def _rnd_u8(n, dev):
    return torch.randint(0, 256, (n,), dtype=torch.uint8, device=dev)


def _time_graph(fn_for_buf, nbuf, iters):
    s = torch.cuda.Stream()
    with torch.cuda.stream(s):
        for i in range(min(nbuf, 4)):
            fn_for_buf(i % nbuf)
        s.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=s):
            for i in range(iters):
                fn_for_buf(i % nbuf)
        g.replay()
        s.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(s)
        g.replay()
        e1.record(s)
        s.synchronize()
    del g
    return e0.elapsed_time(e1) * 1e3 / iters


def launch_floor(iters: int = 200):
    """Microseconds per launch of a stream of empty kernels with the two launch shapes the GEMVs use (one
    544-thread CTA per SM with 207 KB of shared memory; two 288-thread CTAs per SM with 104 KB), with and without
    the programmatic-dependent-launch attribute, graph-replayed like the shapes of the suite."""
    sms = torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count
    out = {}
    for name, grid, threads, smem in (("one_cta_per_sm", sms, 544, 207 * 1024), ("two_ctas_per_sm", 2 * sms, 288, 104 * 1024)):
        for pdl in (True, False):
            us = _time_graph(lambda i: K.probe_launch(grid, threads, smem, 0 if pdl else K.NO_PDL), 2, iters)
            out[f"{name}_{'pdl' if pdl else 'plain'}_us"] = round(us, 2)
    return out


def _nbuf(total_bytes):
    return max(2, int(600e6 // total_bytes) + 1)


def _row(fmt, n, k, batch, us, alg, peak, kernel):
    return {"format": fmt, "N": n, "K": k, "batch": batch, "us": round(us, 2), "gbs": round(alg / us / 1e3, 1),
            "frac_of_measured_peak": round(alg / us / 1e3 / peak, 3), "frac_of_8tbs": round(alg / us / 1e3 / 8000.0, 3),
            "kernel": kernel}


def parse_only(spec: str):
    """`<format>:<N>x<K>:<batch>` -> (format, N, K, batch); formats: w4g, w4g_fused, q4_0, q8_0, iq4nl, ternary,
    q4_k, q5_k, q6_k."""
    fmt, shape, batch = spec.split(":")
    n, k = shape.lower().split("x")
    return fmt, int(n), int(k), int(batch)


def run(peak_gbs: float, iters: int = 100, quick: bool = False, only: str | None = None):
    """only: one `<format>:<N>x<K>:<batch>` case instead of the whole suite (four plain launches first, then the
    timed graph: what a profiler is pointed at)."""
    dev = torch.device("cuda", torch.cuda.current_device())
    rows = []

    def w4g(n, k, batch):
        wb, mb = n * k // 2, n * k // 128 * 4
        nb = _nbuf(wb + mb)
        qd = [_rnd_u8(wb, dev) for _ in range(nb)]
        meta = [(torch.rand(n * k // 128, 2, device=dev) * 0.01 + 0.001).half().view(torch.uint8).reshape(-1) for _ in range(nb)]
        x = torch.randn(batch, k, device=dev).half()
        y = torch.empty(batch, n, device=dev, dtype=torch.half)
        alg = wb + mb + 2 * batch * (k + n)
        if batch >= 3:
            ws = torch.empty(K.gemm_w4g_tc_workspace_bytes(n, k, batch), dtype=torch.uint8, device=dev)
            us = _time_graph(lambda i: K.gemm_w4g_tc(qd[i], meta[i], x, y, n, k, 128, batch, ws, 0), nb, iters)
            rows.append(_row("w4a16-g128", n, k, batch, us, alg, peak_gbs, "tcgen05"))
        else:
            us = _time_graph(lambda i: K.gemv_w4g(qd[i], meta[i], x, y, n, k, 128, batch, 0), nb, iters)
            rows.append(_row("w4a16-g128", n, k, batch, us, alg, peak_gbs, "gemv"))

    def blocks18(n, k, batch, which):
        nblk = n * k // 32
        off = K.q4_gpu_data_offset(nblk)
        tot = off + nblk * 16
        nb = _nbuf(tot)
        bufs = []
        for _ in range(nb):
            b = _rnd_u8(tot, dev)
            b[:nblk * 2] = (torch.rand(nblk, device=dev) * 0.01).half().view(torch.uint8).reshape(-1)
            bufs.append(b)
        x = torch.randn(batch, k, device=dev).half()
        y = torch.empty(batch, n, device=dev, dtype=torch.half)
        if which == "q4_0" and batch >= 3 and k % 512 == 0:
            ws = torch.empty(K.gemm_q4_0_tc_workspace_bytes(n, k, batch), dtype=torch.uint8, device=dev)
            us = _time_graph(lambda i: K.gemm_q4_0_tc(bufs[i], off, x, y, n, k, batch, ws, 0), nb, iters)
            rows.append(_row(which, n, k, batch, us, nblk * 18 + 2 * batch * (k + n), peak_gbs, "tcgen05"))
            return
        fn = K.gemv_q4_0 if which == "q4_0" else K.gemv_iq4nl
        us = _time_graph(lambda i: fn(bufs[i], off, x, y, n, k, batch, 0), nb, iters)
        rows.append(_row(which, n, k, batch, us, nblk * 18 + 2 * batch * (k + n), peak_gbs, "gemv"))

    def q4k(n, k, batch):
        nblk = n * k // 256
        nb = _nbuf(nblk * 144)
        bufs = []
        for _ in range(nb):
            b = _rnd_u8(nblk * 144, dev)
            hdr = b[:nblk * 16].view(-1, 16)
            hdr[:, :4] = (torch.rand(nblk, 2, device=dev) * 0.001).half().view(torch.uint8).reshape(-1, 4)   # d, dmin
            bufs.append(b)
        x = torch.randn(batch, k, device=dev).half()
        y = torch.empty(batch, n, device=dev, dtype=torch.half)
        us = _time_graph(lambda i: K.gemv_q4k(bufs[i], nblk * 16, x, y, n, k, batch, 0), nb, iters)
        rows.append(_row("q4_k", n, k, batch, us, nblk * 144 + 2 * batch * (k + n), peak_gbs, "gemv"))

    def q5k(n, k, batch):
        nblk = n * k // 256
        nb = _nbuf(nblk * 176)
        bufs = []
        for _ in range(nb):
            b = _rnd_u8(nblk * 176, dev)
            side = b[:nblk * 48].view(-1, 48)
            side[:, :4] = (torch.rand(nblk, 2, device=dev) * 0.001).half().view(torch.uint8).reshape(-1, 4)  # d, dmin
            bufs.append(b)
        x = torch.randn(batch, k, device=dev).half()
        y = torch.empty(batch, n, device=dev, dtype=torch.half)
        us = _time_graph(lambda i: K.gemv_q5k(bufs[i], nblk * 48, x, y, n, k, batch, 0), nb, iters)
        rows.append(_row("q5_k", n, k, batch, us, nblk * 176 + 2 * batch * (k + n), peak_gbs, "gemv"))

    def q6k(n, k, batch):
        nblk = n * k // 256
        nb = _nbuf(nblk * 224)
        bufs = []
        for _ in range(nb):
            b = _rnd_u8(nblk * 224, dev)
            side = b[:nblk * 96].view(-1, 96)
            side[:, 80:82] = (torch.rand(nblk, 1, device=dev) * 0.0001).half().view(torch.uint8).reshape(-1, 2)   # d
            bufs.append(b)
        x = torch.randn(batch, k, device=dev).half()
        y = torch.empty(batch, n, device=dev, dtype=torch.half)
        us = _time_graph(lambda i: K.gemv_q6k(bufs[i], nblk * 96, x, y, n, k, batch, 0), nb, iters)
        rows.append(_row("q6_k", n, k, batch, us, nblk * 210 + 2 * batch * (k + n), peak_gbs, "gemv"))

    def q8(n, k, batch):
        nblk = n * k // 32
        tot = nblk * 36
        nb = _nbuf(tot)
        bufs = []
        for _ in range(nb):
            b = _rnd_u8(tot, dev).view(-1, 36)
            b[:, :4] = (torch.rand(nblk, 1, device=dev) * 0.001).float().view(torch.uint8).reshape(-1, 4)
            bufs.append(b.reshape(-1))
        x = torch.randn(batch, k, device=dev).half()
        y = torch.empty(batch, n, device=dev, dtype=torch.half)
        if batch >= 3 and k % 512 == 0:
            ws = torch.empty(K.gemm_q8_0_tc_workspace_bytes(n, k, batch), dtype=torch.uint8, device=dev)
            us = _time_graph(lambda i: K.gemm_q8_0_tc(bufs[i], x, y, n, k, batch, ws, 0), nb, iters)
            rows.append(_row("q8_0", n, k, batch, us, tot + 2 * batch * (k + n), peak_gbs, "tcgen05"))
            return
        us = _time_graph(lambda i: K.gemv_q8_0(bufs[i], x, y, n, k, batch, 0), nb, iters)
        rows.append(_row("q8_0", n, k, batch, us, tot + 2 * batch * (k + n), peak_gbs, "gemv"))

    def ternary(n, k, batch):
        tot = n * k // 4
        nb = _nbuf(tot)
        bufs = []
        for _ in range(nb):
            hi = _rnd_u8(tot, dev) & 0xAA                       # 10 = +1
            lo = _rnd_u8(tot, dev) & 0x55 & ~(hi >> 1)          # 01 = 0, never 11
            bufs.append(hi | lo)
        sc = (torch.rand(n, device=dev) * 0.04 + 0.01).half()
        x = torch.randn(batch, k, device=dev).half()
        y = torch.empty(batch, n, device=dev, dtype=torch.half)
        us = _time_graph(lambda i: K.gemv_ternary(bufs[i], sc, x, y, n, k, batch, 0), nb, iters)
        rows.append(_row("ternary", n, k, batch, us, tot + 2 * n + 2 * batch * (k + n), peak_gbs, "gemv"))

    def w4g_fused(n, k):
        """gate|up with RMSNorm folded into the activation load and SwiGLU into the store (rows interleaved)."""
        wb, mb = n * k // 2, n * k // 128 * 4
        nb = _nbuf(wb + mb)
        qd = [_rnd_u8(wb, dev) for _ in range(nb)]
        meta = [(torch.rand(n * k // 128, 2, device=dev) * 0.01 + 0.001).half().view(torch.uint8).reshape(-1) for _ in range(nb)]
        x = torch.randn(k, device=dev).half()
        res = torch.randn(k, device=dev).half()
        gain = torch.rand(k, device=dev) + 0.5
        y = torch.empty(n // 2, device=dev, dtype=torch.half)
        alg = wb + mb + 2 * 2 * k + 4 * k + 2 * (n // 2)
        us = _time_graph(lambda i: K.gemv_w4g_fused(qd[i], meta[i], x, y, n, k, 128, 0, norm_weight=gain, eps=1e-5,
                                                    residual=res, swiglu=True), nb, iters)
        rows.append(_row("w4a16-g128", n, k, 1, us, alg, peak_gbs, "gemv + rmsnorm in + swiglu out"))

    if only:
        fmt, n, k, b = parse_only(only)
        table = {"w4g": lambda: w4g(n, k, b), "w4g_fused": lambda: w4g_fused(n, k), "q4_0": lambda: blocks18(n, k, b, "q4_0"),
                 "iq4nl": lambda: blocks18(n, k, b, "iq4nl"), "q8_0": lambda: q8(n, k, b), "ternary": lambda: ternary(n, k, b),
                 "q4_k": lambda: q4k(n, k, b), "q5_k": lambda: q5k(n, k, b), "q6_k": lambda: q6k(n, k, b)}
        if fmt not in table:
            raise SystemExit(f"--only: unknown format {fmt!r}")
        table[fmt]()
        return rows
    w4g(4096, 4096, 1)                                          # the reference's own CPU-runnable case
    ternary(11008, 4096, 1)                                     # BitNet-style, per-row scale
    batches = (1,) if quick else (1, 4, 8)
    for (n, k) in SHAPES_8B:
        for b in batches:
            blocks18(n, k, b, "q4_0")
            q8(n, k, b)
            blocks18(n, k, b, "iq4nl")
    for (n, k) in SHAPES_8B:
        for b in (1, 16, 32):
            w4g(n, k, b)
    for (n, k) in SHAPES_70B:
        for b in ((1,) if quick else (1, 8)):
            w4g(n, k, b)
    for (n, k) in SHAPES_8B + [(57344, 8192)]:                  # Q4_K: the format GGUF checkpoints ship with
        q4k(n, k, 1)
        q5k(n, k, 1)
        q6k(n, k, 1)
    w4g(28672, 4096, 1)                                         # merged gate|up of the 8B shapes, plain and fused
    w4g_fused(28672, 4096)
    w4g_fused(57344, 8192)
    return rows


def to_markdown(doc: dict) -> str:
    """The JSON object of `bench.py --suite shapes` as a markdown table."""
    lines = ["# Per-shape throughput of the quantized GEMV / skinny-GEMM kernels (configs 0-4)\n",
             "Command: `python bench.py --suite shapes --steps 60 > shapes.json` on one B200, then "
             "`python -m ztensor_b200.shapes_bench shapes.json` (one case: `--only <format>:<N>x<K>:<batch>`).  Method: " + doc["method"] + "\n",
             f"Peak = {doc['peak']} GB/s ({doc['peak_kind']} copy bandwidth); the column after it is the fraction of the "
             f"nominal 8 TB/s.  device_error = {doc['device_error']}.  CPU columns: the reference CPU engine as restated by "
             "the oracle, on the same host, with the threads the reference would use, timed on a sample of the rows and "
             "scaled (batch-1 rows only).\n",
             *([] if "launch_floor" not in doc else [
                 "Launch floor, measured in the same way (a graph of back-to-back launches of a kernel that does nothing, same "
                 "grid, block and shared-memory carve-out as the GEMV kernels): "
                 + ", ".join(f"{k.replace('_us', '').replace('_', ' ')} {v:.2f} us" for k, v in doc["launch_floor"].items())
                 + ".  A dependent launch that also reads a vector every CTA needs and writes its slice costs 1.8 us; "
                 "what the small shapes pay above that is the activation conversion, the DRAM ramp and the final sums.\n"]),
             "| format | K -> N | batch | us / launch | GB/s | of measured peak | of 8 TB/s | kernel | CPU us | CPU threads | GPU / CPU |",
             "|---|---|---|---|---|---|---|---|---|---|---|"]
    for r in doc["rows"]:
        cpu = (f"{r['cpu_us']:.0f} | {r['cpu_threads']} | {r['speedup_vs_cpu']:.0f}x" if "cpu_us" in r else " | | ")
        lines.append(f"| {r['format']} | {r['K']} -> {r['N']} | {r['batch']} | {r['us']:.2f} | {r['gbs']:.0f} | "
                     f"{r['frac_of_measured_peak'] * 100:.1f} % | {r['frac_of_8tbs'] * 100:.1f} % | {r['kernel']} | {cpu} |")
    return "\n".join(lines) + "\n"


if __name__ == "__main__":
    import json
    import sys
    print(to_markdown(json.load(open(sys.argv[1]))), end="")
