"""Shared helpers of the parity tests: seeded inputs, residency upload through
the C-ABI repack kernels, oracle references and the error measure."""
from __future__ import annotations

import numpy as np

from oracle import oracle as O

REL_TOL = 2e-3          # the bar: max relative error on fp16 / fp32 outputs
FLOOR = 1e-3            # denominators are floored at FLOOR * sum_k |w x| of the row


def seeded(seed):
    return np.random.default_rng(0x5EED + seed)


def make_weights(rng, n, k, std=0.02):
    return (rng.standard_normal((n, k)) * std).astype(np.float32)


def make_x_bits(rng, batch, k):
    """fp16 activations ~N(0,1) as uint16 bit patterns [batch, k]."""
    return O.f32_to_f16_bits(rng.standard_normal((batch, k)).astype(np.float32)).reshape(batch, k)


def rel_err(got, ref, absdot):
    got = np.asarray(got, np.float64)
    ref = np.asarray(ref, np.float64)
    den = np.maximum(np.abs(ref), FLOOR * np.asarray(absdot, np.float64))
    den = np.where(den > 0, den, 1.0)
    return float((np.abs(got - ref) / den).max())


def absdot(w_deq, x):
    """sum_k |w[n,k] x[b,k]| -> [batch, n] (float64)."""
    return np.abs(x.astype(np.float64)) @ np.abs(w_deq.astype(np.float64)).T


# ---------------------------------------------------------------- oracle references (weights [N,K], x [B,K] -> y [B,N])

def ref_q4_0(st: O.Q4Storage, x_f32, n, k):
    """B-side Q4 weight: CPUEngine.MatMul -> GemmF32Q4NT (cpu_engine.go:2405-2411)."""
    b = x_f32.shape[0]
    return O.cpu_engine_matmul(x_f32, (b, k), st, (k, n))


def ref_q8_0(st: O.Q8Storage, x_f32, n, k):
    b = x_f32.shape[0]
    return O.cpu_engine_matmul(x_f32, (b, k), st, (k, n))


def ref_dense_a_side(w_deq, x_f32, n, k):
    """Weights on the A side, [N,K] x [K,B] (w4a16.go:96-106 / IQ4_NL fallthrough): SgemmSimd."""
    b = x_f32.shape[0]
    out = O.cpu_engine_matmul(w_deq, (n, k), np.ascontiguousarray(x_f32.T), (k, b))   # [N,B]
    return np.ascontiguousarray(out.T)


def ref_ternary(st: O.TernaryStorage, x_f32, row_scale_bits, n, k):
    ys = []
    for b in range(x_f32.shape[0]):
        y = O.ternary_gemv(st, x_f32[b], n, k)
        if row_scale_bits is not None:
            y = (y * O.f16_bits_to_f32(row_scale_bits)).astype(np.float32)
        ys.append(y)
    return np.stack(ys)


def to_f16_round(a):
    return O.f16_bits_to_f32(O.f32_to_f16_bits(a)).reshape(np.shape(a))
