"""The committed golden vectors are what the oracle answers today (no GPU needed)."""
import os

import numpy as np
import pytest

import oracle_lib as O
from oxillama_b200 import synth as S

G = np.load(os.path.join(os.path.dirname(__file__), "golden", "qk_golden.npz"))
KEYS = sorted({k.rsplit("_", 1)[0] for k in G.files if k.endswith("_w")})
TYPE_OF = {v: k for k, v in S.NAMES.items()}


def parse(key):
    name, shape = key.rsplit("_", 1)
    rows, cols = (int(v) for v in shape.split("x"))
    return TYPE_OF[name], rows, cols


@pytest.mark.parametrize("key", KEYS)
def test_oracle_reproduces_golden(key):
    t, rows, cols = parse(key)
    w, x = G[key + "_w"], G[key + "_x"]
    assert np.array_equal(O.dequant_matrix(t, w, rows, cols).view(np.uint32), G[key + "_dequant"].view(np.uint32))
    st, y = O.gemm(t, w, x, 3, rows, cols)
    assert st == 0 and np.array_equal(y.view(np.uint32), G[key + "_gemm"].view(np.uint32))
    st, f = O.matvec_q8_fused(t, w, G[key + "_q8"], G[key + "_fused_init"], rows, cols)
    assert st == 0 and np.array_equal(f.view(np.uint32), G[key + "_fused"].view(np.uint32))
