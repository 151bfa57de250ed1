"""Llama-shaped W4A16 projection stacks, sharded tensor-parallel over the ranks
of one node.

Per layer the decode path runs four quantized projections (hidden H, FFN F,
Q/KV heads of 128):

    QKV      H -> (q + 2 kv) * 128     column-parallel (rows split, no exchange)
    O        H -> H                    row-parallel    (K split, all-reduce of the output)
    gate|up  H -> 2 F                  column-parallel (gate and up rows concatenated)
    down     F -> H                    row-parallel    (K split, all-reduce of the output)

Weights are GPTQ-style 4-bit, group 128 along K (tensor/quantized_gptq.go layout,
residency layout of include/ztq.h), quantized on the device by the library's own
quantizer from seeded N(0, 0.02) float32 matrices.  Only the projections run:
activations between them are fixed fp16 N(0,1) buffers, as the benchmark
configuration specifies.  The all-reduce after O and down is NCCL (through
torch.distributed) on the same stream as the kernels, so the whole step can be
recorded into one CUDA graph per rank.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from . import kernels as K

TC_MIN_BATCH = 3      # activation rows from which the stack takes ztq_gemm_w4g_tc instead of ztq_gemv_w4g

SHAPES = {
    # name: (layers, hidden, ffn, q_heads, kv_heads)
    "llama3-8b": (32, 4096, 14336, 32, 8),
    "llama3-70b": (80, 8192, 28672, 64, 8),
}


@dataclass
class Projection:
    name: str
    n: int                 # output rows on this rank
    k: int                 # input columns on this rank
    qdata: torch.Tensor
    meta: torch.Tensor
    row_parallel: bool
    packed: torch.Tensor = None   # the one allocation behind qdata and meta: [nibbles][pad to 256][half2 meta]
    meta_off: int = 0

    @property
    def weight_bytes(self) -> int:
        return self.qdata.numel() + self.meta.numel()


def shard_dims(model: str, world: int):
    """Per-rank (name, N, K, row_parallel) of the four projections."""
    _, h, f, qh, kvh = SHAPES[model]
    if qh % world or kvh % world or f % world or (h // world) % 128 or (f // world) % 128:
        raise ValueError(f"{model} does not shard over {world} ranks")
    qkv_rows = (qh + 2 * kvh) * 128 // world
    return [
        ("qkv", qkv_rows, h, False),
        ("o", h, h // world, True),
        ("gate_up", 2 * f // world, h, False),
        ("down", h, f // world, True),
    ]


def quantize_matrix(n: int, k: int, seed: int, device, awq: bool = False, chunk_rows: int = 8192, with_packed: bool = False):
    """Seeded N(0, 0.02) float32 [n, k] -> (qdata, meta) with the device quantizer.  Both live in one allocation
    laid out as the engine keeps resident GPTQ / AWQ weights: [nibbles][pad to 256 bytes][half2 {scale, zero}]
    (with_packed: also return that allocation and the offset of the meta array)."""
    moff = (n * k // 2 + 255) & ~255
    packed = torch.empty(moff + n * k // 128 * 4, dtype=torch.uint8, device=device)
    qdata = packed[: n * k // 2]
    meta = packed[moff:]
    gen = torch.Generator(device=device)
    gen.manual_seed(seed)
    for r0 in range(0, n, chunk_rows):
        r1 = min(n, r0 + chunk_rows)
        w = torch.empty((r1 - r0) * k, dtype=torch.float32, device=device)
        w.normal_(0.0, 0.02, generator=gen)
        K.quantize_w4g(w, qdata[r0 * k // 2:], meta[r0 * k // 128 * 4:], (r1 - r0) * k, 128, awq)
    if with_packed:
        return qdata, meta, packed, moff
    return qdata, meta


class ProjectionStack:
    def __init__(self, model: str, batch: int = 1, rank: int = 0, world: int = 1, layers: int | None = None,
                 device=None, group=None, seed: int = 0x5EED, host_nccl=None):
        self.model, self.batch, self.rank, self.world = model, batch, rank, world
        # NCCL arm: a communicator of the host library's own binding (ztensor_b200.nccl.Comm: ncclAllReduce on fp16
        # called straight from libztq_host.so) when given, else torch.distributed
        self.host_nccl = host_nccl
        self.device = device or torch.device("cuda", torch.cuda.current_device())
        self.group = group
        nl = SHAPES[model][0] if layers is None else layers
        self.hidden = SHAPES[model][1]
        dims = shard_dims(model, world)
        self.layers: list[list[Projection]] = []
        for li in range(nl):
            projs = []
            for pi, (name, n, k, rowp) in enumerate(dims):
                qd, mt, packed, moff = quantize_matrix(n, k, seed + 1000003 * li + 101 * pi + 7 * rank, self.device, with_packed=True)
                projs.append(Projection(name, n, k, qd, mt, rowp, packed, moff))
            self.layers.append(projs)
        g = torch.Generator(device=self.device)
        g.manual_seed(seed + 99 + rank)
        # fixed fp16 N(0,1) inputs of each projection and their outputs
        self.x = {name: torch.randn(batch, k, device=self.device, generator=g).half() for name, _, k, _ in dims}
        self.y = {name: torch.zeros(batch, n, device=self.device, dtype=torch.float16) for name, n, _, _ in dims}
        # From TC_MIN_BATCH activation rows on the tensor-core kernel wins (one pass over the weights per 32 rows
        # against one GEMV pass per 2 rows); it needs a scratch for its activation tiles
        self.tc_ws = None
        if batch >= TC_MIN_BATCH:
            nbytes = max(K.gemm_w4g_tc_workspace_bytes(n, k, batch) for _, n, k, _ in dims)
            self.tc_ws = torch.empty(nbytes, dtype=torch.uint8, device=self.device)
        self.kernel_launches_per_step = 0
        self.collectives_per_step = 0
        self._count()

    def _count(self):
        # GEMV: one launch per pair of rows; tensor-core path: activation preparation + GEMM per 32 rows
        per_proj = (self.batch + 1) // 2 if self.batch < TC_MIN_BATCH else 2 * ((self.batch + 31) // 32)
        self.kernel_launches_per_step = len(self.layers) * 4 * per_proj
        self.collectives_per_step = len(self.layers) * 2 if self.world > 1 else 0

    @property
    def weight_bytes(self) -> int:
        return sum(p.weight_bytes for layer in self.layers for p in layer)

    def algorithmic_bytes_per_step(self) -> int:
        """Packed weights + scales/zeros + fp16 activations in + fp16 outputs out, each once."""
        total = 0
        for layer in self.layers:
            for p in layer:
                total += p.weight_bytes + 2 * self.batch * (p.k + p.n)
        return total

    def set_input(self, x_host_pinned: torch.Tensor, stream=None):
        """Host -> device copy of the hidden-state input of the step (QKV and gate|up read it)."""
        self.x["qkv"].copy_(x_host_pinned, non_blocking=True)

    def _nccl_all_reduce(self, y):
        if self.host_nccl is not None:
            self.host_nccl.all_reduce_tensor(y)
        else:
            import torch.distributed as dist
            dist.all_reduce(y, group=self.group)

    def run_projection(self, p: Projection, fused=None, y=None):
        """One projection on the current stream (the launches step() makes for it), into y (default: its buffer)."""
        b = self.batch
        y = self.y[p.name] if y is None else y
        if self.tc_ws is not None and p.k % 512 == 0:
            if p.row_parallel and self.world > 1 and fused is not None:
                K.gemm_w4g_tc_allreduce(p.qdata, p.meta, self.x[p.name], y, p.n, p.k, 128, b, self.tc_ws, fused)
                return y
            K.gemm_w4g_tc(p.qdata, p.meta, self.x[p.name], y, p.n, p.k, 128, b, self.tc_ws, 0)
            if p.row_parallel and self.world > 1:
                self._nccl_all_reduce(y)
            return y
        if p.row_parallel and self.world > 1 and fused is not None:
            K.gemv_w4g_allreduce(p.qdata, p.meta, self.x[p.name], y, p.n, p.k, 128, b, fused)
            return y
        K.gemv_w4g(p.qdata, p.meta, self.x[p.name], y, p.n, p.k, 128, b, 0)
        if p.row_parallel and self.world > 1:
            self._nccl_all_reduce(y)
        return y

    def step(self, fused=None):
        """One token-step: every projection of every layer, in order, on the current stream.

        fused: a collective.FusedAllReduce -> the all-reduce after O and down runs inside the
        GEMV kernel; None -> NCCL all-reduce (torch.distributed) after the kernel."""
        for layer in self.layers:
            for p in layer:
                self.run_projection(p, fused)
        return self.y["down"]
