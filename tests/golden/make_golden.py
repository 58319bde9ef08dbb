"""Regenerates tests/golden/qk_golden.npz from the CPU oracle.

    python tests/golden/make_golden.py

The reference is Rust and cannot be run where this was written, so these
vectors are outputs of oracle/qk_oracle.c (itself pinned to the reference's
known-answer tests by tests/test_oracle_kat.py) on seeded synthetic inputs.
They freeze the oracle's answers so that a later change to it, or to the CUDA
path, shows up as a diff against committed bytes.
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

import oracle_lib as O  # noqa: E402
from oxillama_b200 import synth as S  # noqa: E402

CASES = []
for t in S.ALL_TYPES:
    bs = S.BLOCK_SIZE[t]
    CASES.append((t, 19, 768))                 # whole blocks, rows not a multiple of 8
    CASES.append((t, 5, bs + bs // 2 + 3))     # partial last block


def main():
    out = {}
    for i, (t, rows, cols) in enumerate(CASES):
        key = f"{S.NAMES[t]}_{rows}x{cols}"
        w = S.gen_weight(t, rows, cols, seed=100, stream=i)
        x = S.gen_acts(3, cols, seed=100, stream=1000 + i)
        out[key + "_w"] = w
        out[key + "_x"] = x
        out[key + "_dequant"] = O.dequant_matrix(t, w, rows, cols)
        st, y = O.gemm(t, w, x, 3, rows, cols)
        assert st == 0
        out[key + "_gemm"] = y
        # Q8_0 activations cover whole 32-blocks: pad x row 0 with zeros
        kp = -(-cols // S.BLOCK_SIZE[t]) * S.BLOCK_SIZE[t]
        xp = np.zeros(kp, np.float32)
        xp[:cols] = x[0]
        st, a = O.quantize_q8_0(xp)
        assert st == 0
        out[key + "_q8"] = a
        init = np.linspace(-1, 1, rows, dtype=np.float32)
        st, f = O.matvec_q8_fused(t, w, a, init, rows, cols)
        assert st == 0
        out[key + "_fused_init"] = init
        out[key + "_fused"] = f
    np.savez_compressed(os.path.join(HERE, "qk_golden.npz"), **out)
    print("wrote", len(out), "arrays")


if __name__ == "__main__":
    main()
