"""Tensor-parallel sharding of packed GPTQ/AWQ (W4G) weights -- host side, numpy only.

A weight is [N, K] row-major with groups of `group` consecutive k inside a row
(tensor/quantized_gptq.go:45-130): `data` holds K/2 bytes per row, `scales` and
`zeros` K/group fp16 values per row.

  column-parallel (split N, no exchange):  rank r takes rows [r N/w, (r+1) N/w)
  row-parallel    (split K, all-reduce):   rank r takes columns [r K/w, (r+1) K/w);
                                           K/w must be a multiple of the group size
"""
from __future__ import annotations

import numpy as np


def check_shardable(n: int, k: int, world: int, group: int, row_parallel: bool) -> None:
    if world < 1:
        raise ValueError("world must be >= 1")
    if row_parallel:
        if k % world or (k // world) % group:
            raise ValueError(f"K={k} does not split into {world} group-aligned column shards (group {group})")
    elif n % world:
        raise ValueError(f"N={n} does not split into {world} row shards")


def shard_w4g(data: np.ndarray, scales: np.ndarray, zeros: np.ndarray, n: int, k: int, group: int,
              rank: int, world: int, row_parallel: bool):
    """Return (data, scales, zeros, n_local, k_local) of one rank's shard."""
    check_shardable(n, k, world, group, row_parallel)
    d = np.asarray(data, np.uint8).reshape(n, k // 2)
    s = np.asarray(scales, np.uint16).reshape(n, k // group)
    z = np.asarray(zeros, np.uint16).reshape(n, k // group)
    if row_parallel:
        ks = k // world
        c0 = rank * ks
        return (np.ascontiguousarray(d[:, c0 // 2:(c0 + ks) // 2]).ravel(),
                np.ascontiguousarray(s[:, c0 // group:(c0 + ks) // group]).ravel(),
                np.ascontiguousarray(z[:, c0 // group:(c0 + ks) // group]).ravel(), n, ks)
    ns = n // world
    r0 = rank * ns
    return (np.ascontiguousarray(d[r0:r0 + ns]).ravel(), np.ascontiguousarray(s[r0:r0 + ns]).ravel(),
            np.ascontiguousarray(z[r0:r0 + ns]).ravel(), ns, k)


def shard_activations(x: np.ndarray, rank: int, world: int, row_parallel: bool) -> np.ndarray:
    """x [batch, K]: a row-parallel shard reads only its K/w columns."""
    if not row_parallel:
        return x
    ks = x.shape[1] // world
    return np.ascontiguousarray(x[:, rank * ks:(rank + 1) * ks])
