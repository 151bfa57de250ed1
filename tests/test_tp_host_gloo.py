"""Tensor-parallel host logic on CPU: two and four gloo ranks, the oracle doing the arithmetic.

Column-parallel shards concatenate to the full product; row-parallel shards sum
(all-reduce) to it.  This is the N>1 data path minus the GPU kernels."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def _worker(rank, world, port, q):
    from oracle import oracle as O
    from tests import util as U
    from ztensor_b200 import shard as S
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        n, k, batch = 96, 1024, 2
        rng = U.seeded(5)
        st = O.quantize_gptq(U.make_weights(rng, n, k), 128, 4)
        xb = U.make_x_bits(rng, batch, k)
        xf = O.f16_bits_to_f32(xb).reshape(batch, k)
        full = U.ref_dense_a_side(st.slice().reshape(n, k), xf, n, k)                 # [batch, n]
        absd = U.absdot(st.slice().reshape(n, k), xf)

        # row-parallel: partial products, summed by the all-reduce
        d, s, z, nl, kl = S.shard_w4g(st.data, st.scales, st.zeros, n, k, 128, rank, world, True)
        sh = O.GroupQuantStorage("gptq", d, s, z, nl * kl, 128)
        part = U.ref_dense_a_side(sh.slice().reshape(nl, kl), S.shard_activations(xf, rank, world, True), nl, kl)
        t = torch.from_numpy(part.copy())
        dist.all_reduce(t)
        assert U.rel_err(t.numpy(), full, absd) <= 1e-4

        # column-parallel: row blocks, concatenated by an all-gather
        d, s, z, nl, kl = S.shard_w4g(st.data, st.scales, st.zeros, n, k, 128, rank, world, False)
        sh = O.GroupQuantStorage("gptq", d, s, z, nl * kl, 128)
        blk = torch.from_numpy(U.ref_dense_a_side(sh.slice().reshape(nl, kl), xf, nl, kl).copy())
        parts = [torch.zeros_like(blk) for _ in range(world)]
        dist.all_gather(parts, blk)
        assert np.array_equal(torch.cat(parts, dim=1).numpy(), full)                  # same rows, same arithmetic
        q.put((rank, "ok"))
    except Exception as e:  # noqa: BLE001
        q.put((rank, f"fail: {e!r}"))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
def test_sharding_matches_full_product(world):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29600 + (os.getpid() + 7 * world) % 200
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = [q.get(timeout=180) for _ in procs]
    for p in procs:
        p.join(timeout=30)
    assert sorted(res) == [(r, "ok") for r in range(world)], res


def test_shard_dims_and_errors():
    from ztensor_b200 import shard as S
    from ztensor_b200.stack import shard_dims
    for w in (1, 2, 4, 8):
        dims = {name: (n, k, rp) for name, n, k, rp in shard_dims("llama3-70b", w)}
        assert dims["qkv"] == (10240 // w, 8192, False)
        assert dims["o"] == (8192, 8192 // w, True)
        assert dims["gate_up"] == (2 * 28672 // w, 8192, False)
        assert dims["down"] == (8192, 28672 // w, True)
    with pytest.raises(ValueError):
        shard_dims("llama3-70b", 3)
    with pytest.raises(ValueError):
        S.check_shardable(64, 384, 2, 128, True)        # 192 columns per rank: not group aligned
    with pytest.raises(ValueError):
        S.check_shardable(65, 256, 2, 128, False)
