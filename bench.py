#!/usr/bin/env python
"""Benchmark of the weight-quantized GEMV hot path.

Default workload: the Llama-3-70B-shaped 80-layer W4A16 (GPTQ-style 4-bit,
group 128) projection stack at batch 1, sharded tensor-parallel over N GPUs of
one node with an all-reduce after every row-parallel projection.  A step is one
decode token through all 320 projections.  Weights are seeded random-init and
quantized on the device; activations are seeded fp16 N(0,1) buffers.

    python bench.py --gpus 1 --steps 20 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...
    python bench.py --impl reference          # CPU restatement of the reference path

One JSON line is printed by rank 0.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "w4a16_decode_stack_tokens_per_s"
UNIT = "tok/s"


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


# --------------------------------------------------------------------------- clocks
class ClockSampler:
    """nvidia-smi sampled every 200 ms while the timed region runs."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.gpu), f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._pump, daemon=True).start()
        except OSError:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.25)
        self.proc.terminate()
        sm, smax, reasons = [], [], set()
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                smax.append(float(f[2]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(smax) if smax else None,
                "reasons": sorted(reasons), "samples": len(sm)}


# --------------------------------------------------------------------------- CPU arm
def cpu_reference_pass(model: str, batch: int, frac: int, rng_seed: int = 7):
    """One bounded pass of the reference CPU path (compute.MatMulW4A16, compute/w4a16.go:71-119:
    GPTQStorage.Slice() + Float16Storage.Slice() + CPUEngine.MatMul -> SgemmSimd, one thread on
    amd64) over 1/frac of the rows of every projection of one layer (frac = 1: the whole layer).
    Returns (seconds, weights)."""
    import numpy as np

    from oracle import oracle as O
    from ztensor_b200.stack import SHAPES
    _, h, f, qh, kvh = SHAPES[model]
    dims = [((qh + 2 * kvh) * 128, h), (h, h), (2 * f, h), (h, f)]
    rng = np.random.default_rng(rng_seed)
    total_t, total_w = 0.0, 0
    for n, k in dims:
        ns = max(1, n // frac)
        st = O.GroupQuantStorage(
            "gptq", rng.integers(0, 256, ns * k // 2, dtype=np.uint8),
            O.f32_to_f16_bits(rng.uniform(0.002, 0.01, ns * k // 128).astype(np.float32)),
            O.f32_to_f16_bits(rng.uniform(6.5, 8.5, ns * k // 128).astype(np.float32)), ns * k, 128)
        act = O.new_float16_from_f32(rng.standard_normal(k * batch).astype(np.float32))
        t0 = time.perf_counter()
        O.matmul_w4a16(st, (ns, k), act, (k, batch))          # weights on A, activations [K, batch] on B
        total_t += time.perf_counter() - t0
        total_w += ns * k
    return total_t, total_w


def shapes_cpu_rows(rows_cap: int = 2048):
    """The reference CPU engine beside every batch-1 shape: the oracle's restatement of the dispatch of
    compute/cpu_engine.go:2236-2470 (test infrastructure, used here only as the timed baseline), with the threads
    the reference would use: GemmF32Q4NT / GemmF32Q8NT / GemmF32Q4KNT fan out over min(cores, N/4) goroutines
    (internal/xblas/gemm_quant.go:99-105), MatMulW4A16 and IQ4_NL go through Slice() + SgemmSimd on one thread,
    TernaryGEMV is one thread.  Each shape is timed on its first `rows_cap` output rows and scaled to N rows
    (the work is linear in rows); returns {(format, N, K): (microseconds for N rows, threads, sample rows)}."""
    import time

    import numpy as np

    from oracle import oracle as O
    from ztensor_b200.shapes_bench import SHAPES_8B, SHAPES_70B
    rng = np.random.default_rng(3)
    out = {}
    ncpu = O.num_cpu()

    def timed(fn):
        t0 = time.perf_counter()
        fn()
        return (time.perf_counter() - t0) * 1e6

    def add(fmt, n, k, us_sample, ns, threads):
        out[(fmt, n, k)] = (us_sample * n / ns, threads, ns)

    for (n, k) in [(4096, 4096)] + SHAPES_8B + SHAPES_70B + [(28672, 4096)]:
        ns = min(n, rows_cap)
        x = rng.standard_normal(k).astype(np.float32)
        st = O.GroupQuantStorage("gptq", rng.integers(0, 256, ns * k // 2, dtype=np.uint8),
                                 O.f32_to_f16_bits(rng.uniform(0.002, 0.01, ns * k // 128).astype(np.float32)),
                                 O.f32_to_f16_bits(rng.uniform(6.5, 8.5, ns * k // 128).astype(np.float32)), ns * k, 128)
        act = O.new_float16_from_f32(x)
        add("w4a16-g128", n, k, timed(lambda: O.matmul_w4a16(st, (ns, k), act, (k, 1))), ns, 1)
    for (n, k) in SHAPES_8B:
        ns = min(n, rows_cap)
        x = rng.standard_normal(k).astype(np.float32)
        w = (rng.standard_normal(ns * k) * 0.02).astype(np.float32)
        q4, q8, q4k, iq = O.quantize_q4(w), O.quantize_q8(w), O.quantize_q4k(w), O.make_iq4nl_blocks(w)
        q5k, q6k = O.make_q5k_blocks(w), O.make_q6k_blocks(w)
        th = O.nt_threads(ns, k, ncpu)
        add("q4_0", n, k, timed(lambda: O.gemm_f32_q4_nt(1, ns, k, x, q4, ncpu)), ns, th)
        add("q8_0", n, k, timed(lambda: O.gemm_f32_q8_nt(1, ns, k, x, q8, ncpu)), ns, th)
        add("q4_k", n, k, timed(lambda: O.gemm_f32_q4k_nt(1, ns, k, x, q4k, ncpu)), ns, th)
        add("q5_k", n, k, timed(lambda: O.gemm_f32_q5k_nt(1, ns, k, x, q5k, ncpu)), ns, th)
        add("q6_k", n, k, timed(lambda: O.gemm_f32_q6k_nt(1, ns, k, x, q6k, ncpu)), ns, th)
        add("iq4nl", n, k, timed(lambda: O.sgemm_simd(ns, 1, k, iq.slice(), x)), ns, 1)
    n, k = 11008, 4096
    ns = min(n, rows_cap)
    tern = O.new_ternary_from(rng.integers(-1, 2, size=ns * k).astype(np.int8))
    x = rng.standard_normal(k).astype(np.float32)
    add("ternary", n, k, timed(lambda: O.ternary_gemv(tern, x, ns, k)), ns, 1)
    return out


REF_MAX_STEPS = 3          # a whole 70B-shaped layer is about 30 s on one CPU thread


def run_reference_arm(args):
    from ztensor_b200.stack import SHAPES
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    layers = args.layers_effective
    if args.warmup > 0:
        cpu_reference_pass(args.model, args.batch, 16)            # warm-up: a sixteenth of a layer (page-in, threads)
    steps = max(1, min(args.steps, REF_MAX_STEPS))
    t = 0.0
    for i in range(steps):
        dt, _ = cpu_reference_pass(args.model, args.batch, 1, rng_seed=7 + i)
        t += dt
    per_token = (t / steps) * layers
    value = args.batch / per_token
    sample = (f"every row of the 4 projections of one whole layer per step ({steps} steps timed of the {args.steps} asked "
              f"for: a layer takes about half a minute), scaled by {layers} layers; restatement of compute.MatMulW4A16 on "
              "the CPU engine (Slice dequant + SgemmSimd), single thread as on amd64")
    out = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": steps, "warmup": min(args.warmup, 1), "ms_per_step": per_token * 1e3, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(args, args.gpus),
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": 1, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    _emit(out)


def workload_config(args, world):
    return {"workload": f"{args.model}-shaped W4A16 (GPTQ-4bit g128) projection stack, decode batch {args.batch}",
            "layers": args.layers_effective, "batch": args.batch, "parallelism": f"tp{world}",
            "gate_up_merged": True, "l2": "inputs (packed weights) exceed L2 many times over; no flush needed",
            "activations": "independent fixed fp16 N(0,1) input buffer per projection, as the configuration specifies; "
                           "launches are ordered by the stream (each waits for the one before)",
            "collective": (f"{getattr(args, 'allreduce', 'fused')} all-reduce after O and down" if world > 1 else "none")}


# --------------------------------------------------------------------------- untimed correctness sample
def parity_spot_check(stack, fused, world, dev, stream, samples=256):
    """After the timed loops: the four projections of layer 0 once more, through the very launches the timed
    step makes, and `samples` of their output rows against the CPU oracle (the checker; nothing here is timed).

    Column-parallel projections: every rank checks rows of its own shard.  Row-parallel projections (O, down):
    every rank computes the oracle's partial product of the sampled rows over ITS columns, the partials are
    summed over the ranks in float64, and every rank compares its all-reduced output with that sum.  The error
    measure is the parity tests': |got - ref| / max(|ref|, 1e-3 sum_k |w x|), outputs and reference rounded to
    fp16 alike.  Returns {projection: max error over rows and ranks}."""
    import numpy as np
    import torch
    import torch.distributed as dist

    from oracle import oracle as O
    b = stack.batch
    out = {}
    with torch.cuda.stream(stream):
        for p in stack.layers[0]:
            y = torch.full((b, p.n), float("nan"), dtype=torch.float16, device=dev)
            stack.run_projection(p, fused, y)
            stream.synchronize()
            rows = np.unique(np.linspace(0, p.n - 1, samples).astype(np.int64))
            ridx = torch.from_numpy(rows).to(dev)
            data = p.qdata.view(p.n, p.k // 2)[ridx].cpu().numpy()
            m = p.meta.view(p.n, (p.k // 128) * 4)[ridx].cpu().numpy().view(np.uint16).reshape(len(rows), p.k // 128, 2)
            st = O.GroupQuantStorage("gptq", data.ravel(), np.ascontiguousarray(m[:, :, 0]).ravel(),
                                     np.ascontiguousarray(m[:, :, 1]).ravel(), len(rows) * p.k, 128)
            xb = stack.x[p.name].view(torch.int16).cpu().numpy().view(np.uint16)             # [b, k] fp16 bits
            act = O.Float16Storage(xb.T.copy().ravel(), b * p.k)
            ref = np.ascontiguousarray(O.matmul_w4a16(st, (len(rows), p.k), act, (p.k, b)).T).astype(np.float64)   # [b, rows]
            xf = O.f16_bits_to_f32(xb).reshape(b, p.k)
            absd = (np.abs(xf) @ np.abs(st.slice().reshape(len(rows), p.k)).T).astype(np.float64)
            if p.row_parallel and world > 1:
                t = torch.from_numpy(np.stack([ref, absd])).to(dev)
                dist.all_reduce(t)
                ref, absd = t.cpu().numpy()
            ref16 = O.f16_bits_to_f32(O.f32_to_f16_bits(ref.astype(np.float32))).reshape(ref.shape).astype(np.float64)
            got = y.float().cpu().numpy().astype(np.float64)[:, rows]
            den = np.maximum(np.abs(ref16), 1e-3 * absd)
            den = np.where(den > 0, den, 1.0)
            err = float((np.abs(got - ref16) / den).max()) if np.isfinite(got).all() else float("inf")
            if world > 1:
                t = torch.tensor([err], device=dev, dtype=torch.float64)
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
                err = float(t.item())
            out[p.name] = err
    return out


# --------------------------------------------------------------------------- end to end through the engine
class EngineStep:
    """The same token-step issued through the engine mirror (libztq_host.so: GPUEngine.MatMul per projection, the
    reference's entry point), recorded once into a CUDA graph with the engine's own capture calls.  The weights are
    the stack's device buffers, adopted in place; activations and outputs are device tensors from the engine's pool
    (outputs float32, the reference's result type)."""

    def __init__(self, stack, device_index):
        import torch

        from ztensor_b200 import engine as E
        self.E, self.g = E, E.GPUEngine(device_index)
        g = self.g
        self.x, self.y, self.ops = {}, {}, []
        for p in stack.layers[0]:
            xt = g.device_tensor((stack.batch, p.k), f16=True)
            h = stack.x[p.name].cpu().pin_memory()
            g.copy_from_host(xt, h.data_ptr(), h.numel() * 2)
            g.sync()
            self.x[p.name] = xt
            self.y[p.name] = g.device_tensor((stack.batch, p.n))
        for layer in stack.layers:
            for p in layer:
                w = E.w4g_device_tensor(p.packed.data_ptr(), p.packed.numel(), p.meta_off, p.n * p.k, 128, (p.k, p.n),
                                        device=device_index)
                self.ops.append((self.x[p.name], w, self.y[p.name]))
        self._run()                                            # uncaptured pass: kernels loaded, pool warm
        g.sync()
        g.begin_capture()
        self._run()
        self.graph = g.end_capture()
        self.stream = torch.cuda.ExternalStream(g.stream)
        self.out_bytes = stack.batch * stack.hidden * 4

    def _run(self):
        for x, w, y in self.ops:
            self.g.matmul_async(x, w, dst=y)                   # weights on B: the virtual transpose of gpu_engine.go:2119-2126

    def step(self, x_host, y_host):
        g = self.g
        g.copy_from_host(self.x["qkv"], x_host.data_ptr(), x_host.numel() * 2)
        g.replay_graph(self.graph)
        g.copy_to_host(self.y["down"], y_host.data_ptr(), self.out_bytes)
        g.sync()                                               # the caller reads the result before the next token

    def close(self):
        self.g.destroy_graph(self.graph)


# --------------------------------------------------------------------------- per-layer time budget
def run_layer_budget(args, world, rank, dev, hbm_peak):
    """Where a layer's time goes on this rank count: each of the four projections of the sharded layer alone
    (a graph of back-to-back launches cycling through distinct weights), the row-parallel ones also with the fused
    and with the NCCL all-reduce, the whole layer, and a stream of empty kernels of the same launch shape as the
    floor.  Times are CUDA events on the launching stream, max over ranks."""
    import torch
    import torch.distributed as dist

    from ztensor_b200 import kernels as K
    from ztensor_b200.shapes_bench import _time_graph, launch_floor
    from ztensor_b200.stack import shard_dims
    fused = None
    if world > 1:
        from ztensor_b200.collective import FusedAllReduce
        fused = FusedAllReduce(max_elems=args.batch * 8192)
    dims = shard_dims(args.model, args.shard_as or world)      # --shard-as: one GPU running another rank count's shapes
    b = args.batch
    rows = []
    bufs = {}
    for name, n, k, rowp in dims:
        wb, mb = n * k // 2, n * k // 128 * 4
        nbuf = max(8, int(500e6 // (wb + mb)) + 1)
        qd = [torch.randint(0, 256, (wb,), dtype=torch.uint8, device=dev) for _ in range(nbuf)]
        meta = [(torch.rand(n * k // 128, 2, device=dev) * 0.01 + 0.001).half().view(torch.uint8).reshape(-1) for _ in range(nbuf)]
        x = torch.randn(b, k, device=dev).half()
        y = torch.empty(b, n, device=dev, dtype=torch.half)
        bufs[name] = (qd, meta, x, y, n, k, nbuf, rowp)

    def reduce_max(v):
        if world == 1:
            return v
        t = torch.tensor([v], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    # three or more activation rows: the tensor-core kernels, as the stack runner chooses
    use_tc = b >= 3 and all(k % 512 == 0 for _, _, k, _ in dims)
    ws = torch.empty(max(K.gemm_w4g_tc_workspace_bytes(n, k, b) for _, n, k, _ in dims), dtype=torch.uint8, device=dev) if use_tc else None

    def plain(qd, meta, x, y, n, k):
        if use_tc:
            K.gemm_w4g_tc(qd, meta, x, y, n, k, 128, b, ws, 0)
        else:
            K.gemv_w4g(qd, meta, x, y, n, k, 128, b, 0)

    def reduced(qd, meta, x, y, n, k):
        if use_tc:
            K.gemm_w4g_tc_allreduce(qd, meta, x, y, n, k, 128, b, ws, fused)
        else:
            K.gemv_w4g_allreduce(qd, meta, x, y, n, k, 128, b, fused)

    iters = max(40, args.steps)
    for name, n, k, rowp in dims:
        qd, meta, x, y, _, _, nbuf, _ = bufs[name]
        r = {"projection": name, "N": n, "K": k, "row_parallel": rowp, "weight_mb": round((n * k // 2 + n * k // 32) / 1e6, 2),
             "hbm_us_at_peak": round((n * k // 2 + n * k // 32) / hbm_peak / 1e3, 2)}
        r["us_gemv"] = round(reduce_max(_time_graph(lambda i: plain(qd[i], meta[i], x, y, n, k), nbuf, iters)), 2)
        if rowp and world > 1:
            r["us_gemv_fused_allreduce"] = round(reduce_max(_time_graph(lambda i: reduced(qd[i], meta[i], x, y, n, k), nbuf, iters)), 2)

            def with_nccl(i):
                plain(qd[i], meta[i], x, y, n, k)
                dist.all_reduce(y)
            r["us_gemv_nccl_allreduce"] = round(reduce_max(_time_graph(with_nccl, nbuf, iters)), 2)
        rows.append(r)

    def layer(i):
        for name, n, k, rowp in dims:
            qd, meta, x, y, _, _, nbuf, _ = bufs[name]
            if rowp and world > 1:
                reduced(qd[i % nbuf], meta[i % nbuf], x, y, n, k)
            else:
                plain(qd[i % nbuf], meta[i % nbuf], x, y, n, k)
    layer_us = reduce_max(_time_graph(layer, 8, iters))
    floor = launch_floor(iters=200)
    err = K.device_error()
    if rank == 0:
        _emit({"suite": "budget", "model": args.model, "batch": b, "n_gpus": world,
               "kernel": "tensor cores (ztq_gemm_w4g_tc)" if use_tc else "gemv", "rows": rows,
               "layer_us": round(layer_us, 2), "sum_of_rows_us": round(sum(r.get("us_gemv_fused_allreduce", r["us_gemv"]) for r in rows), 2),
               "shapes_of_ranks": args.shard_as or world, "launch_floor": floor, "device_error": err,
               "method": "each row: a CUDA graph of back-to-back launches of that projection alone over distinct weight "
                         "buffers (> 500 MB in total), one replay timed with CUDA events, max over ranks; layer_us: the four "
                         "projections in stack order, fused all-reduce where row-parallel"})
    if fused is not None:
        fused.close()


# --------------------------------------------------------------------------- GPU arm
_RESULT_FD = None


def _claim_stdout():
    """Libraries (NCCL's version banner) write to file descriptor 1; the contract is ONE JSON line on stdout.
    Keep a private copy of stdout for the result and point descriptor 1 at stderr for everybody else."""
    global _RESULT_FD
    if _RESULT_FD is None:
        sys.stdout.flush()
        _RESULT_FD = os.dup(1)
        os.dup2(2, 1)


def _emit(obj):
    line = (json.dumps(obj) + "\n").encode()
    if _RESULT_FD is None:
        sys.stdout.write(line.decode())
        sys.stdout.flush()
    else:
        os.write(_RESULT_FD, line)


def main():
    _claim_stdout()
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--model", default="llama3-70b", choices=["llama3-70b", "llama3-8b"])
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--layers", type=int, default=0, help="override the layer count (debugging only)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-parity-check", action="store_true", help="skip the untimed oracle sample after the timed loops")
    ap.add_argument("--suite", default="stack", choices=["stack", "shapes", "budget"],
                    help="stack: the decode stack (the one JSON line of the contract); shapes: per-shape GB/s of every "
                         "quantized GEMV of the benchmark configurations, one JSON object with a row per shape; budget: the "
                         "four projections of one sharded layer timed one by one, with and without their all-reduce, "
                         "beside the launch floor (any number of ranks)")
    ap.add_argument("--shard-as", type=int, default=0,
                    help="with --suite budget on one GPU: the per-rank shapes of this many ranks (no all-reduce)")
    ap.add_argument("--only", default=None, metavar="FMT:NxK:BATCH",
                    help="with --suite shapes: one case, e.g. w4g:57344x8192:1 (formats: w4g, w4g_fused, q4_0, q8_0, "
                         "iq4nl, ternary, q4_k, q5_k, q6_k); no CPU column")
    ap.add_argument("--allreduce", default="fused", choices=["fused", "nccl"],
                    help="all-reduce after the row-parallel projections: fused into the GEMV kernel, or NCCL")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup

    from ztensor_b200.stack import SHAPES
    args.layers_effective = args.layers or SHAPES[args.model][0]

    if args.impl == "reference":
        run_reference_arm(args)
        return

    import torch
    import torch.distributed as dist

    from ztensor_b200 import _lib
    from ztensor_b200 import kernels as K
    from ztensor_b200.stack import ProjectionStack

    _lib.lib()                                     # fail loudly if the CUDA library is not built
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
    if not K.check_sm100():
        raise RuntimeError("this benchmark needs an sm_100 device")
    hbm_peak, peak_kind = load_peaks()

    if args.suite == "shapes":
        if world > 1:
            raise SystemExit("--suite shapes is a single-GPU measurement")
        from ztensor_b200 import shapes_bench
        rows = shapes_bench.run(hbm_peak, iters=max(20, args.steps), only=args.only)
        if not args.no_cpu_baseline and not args.only:  # the reference CPU engine (oracle port) beside the batch-1 rows
            cpu = shapes_cpu_rows()
            for r in rows:
                c = cpu.get((r["format"], r["N"], r["K"]))
                if c and r["batch"] == 1 and "rmsnorm" not in r["kernel"]:
                    r["cpu_us"], r["cpu_threads"], r["cpu_sample_rows"] = round(c[0], 1), c[1], c[2]
                    r["speedup_vs_cpu"] = round(c[0] / r["us"], 1)
        _emit({"suite": "shapes", "unit": "GB/s", "peak": hbm_peak, "peak_kind": peak_kind,
                          "launch_floor": shapes_bench.launch_floor(),
                          "method": shapes_bench.__doc__.split("Method:")[1].strip().split("\n\n")[0].replace("\n", " "),
                          "device_error": K.device_error(), "rows": rows})
        return

    if args.suite == "budget":
        run_layer_budget(args, world, rank, dev, hbm_peak)
        _teardown(world, None)
        return

    host_comm = None
    if world > 1 and args.allreduce == "nccl":
        # the NCCL arm calls ncclAllReduce through the host library's own binding (internal/nccl's counterpart)
        from ztensor_b200 import nccl as host_nccl
        ids = [host_nccl.get_unique_id() if rank == 0 else None]
        dist.broadcast_object_list(ids, src=0)
        host_comm = host_nccl.Comm(ids[0], world, rank)
    stack = ProjectionStack(args.model, args.batch, rank, world, layers=args.layers or None, device=dev, host_nccl=host_comm)
    fused = None
    if world > 1 and args.allreduce == "fused":
        from ztensor_b200.collective import FusedAllReduce
        fused = FusedAllReduce(max_elems=args.batch * stack.hidden)
    stream = torch.cuda.Stream(device=dev)
    x_host = torch.randn(args.batch, stack.hidden).half().pin_memory()
    y_host = torch.empty(args.batch, stack.hidden, dtype=torch.float16).pin_memory()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    with torch.cuda.stream(stream):
        for _ in range(2):                         # eager warm-up (module loading, NCCL channels)
            stack.step(fused)
            stack.step(None)
        stream.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            stack.step(fused)
        for _ in range(args.warmup):
            graph.replay()
        stream.synchronize()

        # ---- the same step with NCCL all-reduces instead of the fused one (reported beside it)
        ms_nccl = None
        if fused is not None:
            graph_nccl = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph_nccl, stream=stream):
                stack.step(None)
            for _ in range(args.warmup):
                graph_nccl.replay()
            barrier()
            n0, n1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            n0.record(stream)
            for _ in range(args.steps):
                graph_nccl.replay()
            n1.record(stream)
            stream.synchronize()
            barrier()
            ms_nccl = n0.elapsed_time(n1)
            del graph_nccl

        # ---- device-resident throughput
        sampler = ClockSampler(local)
        barrier()
        if rank == 0:
            sampler.start()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(args.steps):
            graph.replay()
        e1.record(stream)
        stream.synchronize()
        barrier()
        ms = e0.elapsed_time(e1)
        clocks = sampler.stop() if rank == 0 else None

        # ---- end to end: pinned host input in, result out, every step.  One GPU: through the engine mirror's
        # MatMul (libztq_host.so), the reference-facing call; several GPUs: through the stack runner (the engine
        # mirror has no collective)
        barrier()
        e2e_via = "stack runner over the C-ABI"
        if world == 1:
            es = EngineStep(stack, local)
            y32_host = torch.empty(args.batch, stack.hidden, dtype=torch.float32).pin_memory()
            for _ in range(args.warmup):
                es.step(x_host, y32_host)
            f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            f0.record(es.stream)
            for _ in range(args.steps):
                es.step(x_host, y32_host)
            f1.record(es.stream)
            es.stream.synchronize()
            ms_e2e = f0.elapsed_time(f1)
            d2h_bytes = y32_host.numel() * 4
            e2e_via = "GPUEngine.MatMul of the engine mirror (libztq_host.so), one captured graph of 320 calls"
            # the engine path computes the same products: compare its last output with the stack's
            stack.set_input(x_host)
            graph.replay()
            stream.synchronize()
            e2e_diff = float((y32_host.to(dev) - stack.y["down"].float()).abs().max().item() /
                             max(1e-30, stack.y["down"].float().abs().max().item()))
            es.close()
        else:
            f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            f0.record(stream)
            for _ in range(args.steps):
                stack.set_input(x_host)
                graph.replay()
                y_host.copy_(stack.y["down"], non_blocking=True)
                stream.synchronize()                    # the caller reads the result before the next token
            f1.record(stream)
            stream.synchronize()
            ms_e2e = f0.elapsed_time(f1)
            d2h_bytes = y_host.numel() * 2
            e2e_diff = None
        barrier()

        # ---- dominant kernel alone: gate|up GEMV of every layer in turn (distinct weights >> L2)
        gu = [layer[2] for layer in stack.layers]
        reps = max(1, 160 // len(gu))
        for p in gu[:4]:
            K.gemv_w4g(p.qdata, p.meta, stack.x[p.name], stack.y[p.name], p.n, p.k, 128, 1, 0)
        stream.synchronize()
        k0, k1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        k0.record(stream)
        for _ in range(reps):
            for p in gu:
                K.gemv_w4g(p.qdata, p.meta, stack.x[p.name], stack.y[p.name], p.n, p.k, 128, 1, 0)
        k1.record(stream)
        stream.synchronize()
        kernel_ms = k0.elapsed_time(k1) / (reps * len(gu))
        err = K.device_error()
    parity = None if args.no_parity_check else parity_spot_check(stack, fused, world, dev, stream)

    if world > 1:
        t = torch.tensor([ms, ms_e2e, kernel_ms, ms_nccl or 0.0], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, ms_e2e, kernel_ms, ms_nccl_max = t.tolist()
        ms_nccl = ms_nccl_max if ms_nccl is not None else None

    if rank == 0:
        p0 = gu[0]
        alg_bytes = p0.weight_bytes + 2 * (p0.k + p0.n)               # weights + scales/zeros + x + y, once each
        achieved = alg_bytes / (kernel_ms * 1e-3) / 1e9
        value = args.batch * args.steps / (ms * 1e-3)
        e2e_value = args.batch * args.steps / (ms_e2e * 1e-3)
        step_bytes = stack.algorithmic_bytes_per_step()
        out = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "int8xint4 exact block dot, fp32 scales and accumulation",
            "data": "synthetic", "config": workload_config(args, world),
            "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": x_host.numel() * 2,
                    "d2h_bytes_per_step": d2h_bytes, "via": e2e_via, "max_rel_diff_vs_stack_runner": e2e_diff},
            "gpu_launches": stack.kernel_launches_per_step * args.steps,
            "stack_gbs_per_gpu": step_bytes / (ms / args.steps * 1e-3) / 1e9,
            "stack_frac_of_hbm_peak": step_bytes / (ms / args.steps * 1e-3) / 1e9 / hbm_peak,
            "roofline": {"bound": "hbm", "kernel": f"gemv_w4pair_kernel (gate|up {p0.k}->{p0.n}, batch 1)",
                         "achieved": achieved, "peak": hbm_peak, "peak_kind": peak_kind, "unit": "GB/s",
                         "frac": achieved / hbm_peak, "frac_of_8tbs": achieved / 8000.0,
                         "algorithmic_bytes_per_launch": alg_bytes, "us_per_launch": kernel_ms * 1e3,
                         "traffic": None},
            "clocks": clocks, "device_error": err,
        }
        if parity is not None:
            out["parity_sample_max_rel_err"] = max(parity.values())
            out["parity_sample"] = {"per_projection": parity, "tolerance": 2e-3, "rows_per_projection": 256,
                                    "what": "layer 0, outputs of the launches the timed step makes vs the CPU oracle "
                                            "(after all-reduce where there is one), untimed"}
        if world > 1:
            out["allreduce"] = {"mode": args.allreduce, "per_step": stack.collectives_per_step,
                                "payload_bytes": 2 * args.batch * stack.hidden,
                                "nccl_arm": "ncclAllReduce (fp16) through the host library's binding of libnccl.so.2"}
            if ms_nccl is not None:
                out["allreduce"]["nccl_value"] = args.batch * args.steps / (ms_nccl * 1e-3)
                out["allreduce"]["nccl_ms_per_step"] = ms_nccl / args.steps
        if world == 1 and not args.no_cpu_baseline:
            t_cpu, _ = cpu_reference_pass(args.model, args.batch, 1)
            per_token = t_cpu * args.layers_effective
            out["cpu_baseline"] = {
                "value": args.batch / per_token, "unit": UNIT, "cores": 1, "kind": "port",
                "sample": f"every row of the 4 projections of one whole layer, timed once, scaled by "
                          f"{args.layers_effective} layers; reference path compute.MatMulW4A16 on the CPU engine "
                          "(dequantize + SgemmSimd), one thread as on amd64"}
        traffic_file = os.path.join(ROOT, "profiles", "traffic.json")
        if os.path.exists(traffic_file):
            with open(traffic_file) as f:
                out["roofline"]["traffic"] = json.load(f).get(f"w4g_{p0.k}x{p0.n}")
        _emit(out)

    del graph
    _teardown(world, fused)


def _teardown(world, fused):
    """Release the captured graph before the communicator, and never let a stuck communicator teardown outlive the
    measurement (the JSON line is already out)."""
    import torch
    import torch.distributed as dist
    sys.stdout.flush()
    torch.cuda.synchronize()
    if fused is not None:
        fused.close()
    if world > 1:
        threading.Timer(20.0, lambda: os._exit(0)).start()
        try:
            dist.barrier()
            dist.destroy_process_group()
        finally:
            os._exit(0)


if __name__ == "__main__":
    main()
