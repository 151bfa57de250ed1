"""Generates tests/golden/gemv_golden.npz: small seeded cases of every format with the oracle's outputs.

The reference (Go) cannot run where this was made, so the vectors come from the CPU oracle, which is itself
pinned to the reference's known-answer tests (tests/test_oracle_golden.py).  They freeze today's oracle
arithmetic: a later change to the oracle or to a kernel that moves any value shows up against this file.

    python tests/golden/make_golden.py
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from oracle import oracle as O      # noqa: E402
from tests import util as U         # noqa: E402

CASES = [("q4_0", 48, 512, 2), ("q8_0", 40, 256, 3), ("iq4nl", 24, 512, 1), ("gptq", 32, 1024, 2), ("awq", 32, 512, 1),
         ("ternary", 36, 256, 2), ("q4k", 24, 2048, 2), ("q5k", 16, 2048, 1), ("q6k", 16, 2048, 1)]


def build():
    out = {}
    for fmt, n, k, batch in CASES:
        rng = U.seeded(sum(map(ord, fmt)))
        w = U.make_weights(rng, n, k)
        xb = U.make_x_bits(rng, batch, k)
        xf = O.f16_bits_to_f32(xb).reshape(batch, k)
        pre = f"{fmt}_{n}x{k}_b{batch}"
        out[pre + "/x_bits"] = xb
        if fmt == "q4_0":
            st = O.quantize_q4(w)
            out[pre + "/blocks"] = st.blocks
            y = U.ref_q4_0(st, xf, n, k)
        elif fmt == "q4k":
            st = O.quantize_q4k(w)
            out[pre + "/blocks"] = st.raw
            y = O.gemm_f32_q4k_nt(batch, n, k, xf, st, ncpu=1).reshape(batch, n)
        elif fmt == "q5k":
            st = O.make_q5k_blocks(w)
            out[pre + "/blocks"] = st.raw
            y = O.gemm_f32_q5k_nt(batch, n, k, xf, st, ncpu=1).reshape(batch, n)
        elif fmt == "q6k":
            st = O.make_q6k_blocks(w)
            out[pre + "/blocks"] = st.raw
            y = O.gemm_f32_q6k_nt(batch, n, k, xf, st, ncpu=1).reshape(batch, n)
        elif fmt == "q8_0":
            st = O.quantize_q8(w)
            out[pre + "/blocks"] = st.blocks
            y = U.ref_q8_0(st, xf, n, k)
        elif fmt == "iq4nl":
            st = O.make_iq4nl_blocks(w)
            out[pre + "/blocks"] = st.raw
            y = U.ref_dense_a_side(st.slice().reshape(n, k), xf, n, k)
        elif fmt in ("gptq", "awq"):
            st = O.quantize_gptq(w, 128, 4) if fmt == "gptq" else O.quantize_awq(w, 128)
            out[pre + "/data"], out[pre + "/scales"], out[pre + "/zeros"] = st.data, st.scales, st.zeros
            act = O.Float16Storage(xb.T.copy().ravel(), batch * k)
            y = np.ascontiguousarray(O.matmul_w4a16(st, (n, k), act, (k, batch)).T)
        else:
            vals = rng.integers(-1, 2, size=n * k).astype(np.int8)
            st = O.new_ternary_from(vals)
            sc = O.f32_to_f16_bits(rng.uniform(0.01, 0.05, n).astype(np.float32))
            out[pre + "/data"], out[pre + "/row_scale"] = st.data, sc
            y = U.ref_ternary(st, xf, sc, n, k)
        out[pre + "/w_dequant"] = st.slice().astype(np.float32)
        out[pre + "/y"] = y.astype(np.float32)
    return out


if __name__ == "__main__":
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "gemv_golden.npz")
    np.savez_compressed(path, **build())
    print("wrote", path, os.path.getsize(path), "bytes")
