"""The CPU baseline's SIMD rows (oracle/qk_cpu_simd.c: restatements of the reference's
gemv_row_avx2 / gemv_row_avx512 for all five formats) against the scalar oracle, at the bar
the reference holds its own SIMD tiers to (1e-3, e.g. simd/avx2/q4_k.rs:766-1028), on full,
ragged and multi-threaded shapes."""
import ctypes as C
import os
import subprocess

import numpy as np
import pytest

import oracle_lib as O
from oxillama_b200 import synth as S

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def simd():
    so = os.path.join(ROOT, "oracle", "_build", "libqk_cpu_simd.so")
    src = os.path.join(ROOT, "oracle", "qk_cpu_simd.c")
    if not os.path.exists(so) or os.path.getmtime(so) < os.path.getmtime(src):
        subprocess.check_call(["make", "-s", "-C", os.path.join(ROOT, "oracle")])
    return C.CDLL(so)


def run(simd, t, tier, threads, w, rows, cols, x):
    y = np.full(rows, np.nan, np.float32)
    used = C.c_int(-1)
    st = simd.qk_cpu_gemv(t, tier, threads, C.c_void_p(w.ctypes.data), C.c_size_t(rows), C.c_size_t(cols),
                          C.c_void_p(x.ctypes.data), C.c_void_p(y.ctypes.data), C.byref(used))
    assert st == 0
    return y, used.value


@pytest.mark.parametrize("t", S.ALL_TYPES)
@pytest.mark.parametrize("rows,cols", [(64, 4096), (7, 256 + 96 + 5), (33, 1024), (3, 40)])
def test_simd_rows_match_the_scalar_oracle(simd, t, rows, cols):
    best = simd.qk_cpu_best_tier()
    w = S.gen_weight(t, rows, cols, seed=41)
    x = S.gen_acts(1, cols, seed=41)[0]
    st, ref = O.gemv(t, w, rows, cols, x)
    assert st == 0
    den = float(np.abs(ref).max()) or 1.0
    for tier in range(best + 1):
        for threads in (1, 3):
            y, used = run(simd, t, tier, threads, w, rows, cols, x)
            assert used == tier          # every format has every tier the CPU has
            assert float(np.abs(y - ref).max()) / den <= 1e-3, (tier, threads)
    y0, used = run(simd, t, 0, 1, w, rows, cols, x)
    assert used == 0 and np.array_equal(y0, ref)   # tier 0 is the oracle row itself


def test_pool_survives_many_calls_and_thread_counts(simd):
    t, rows, cols = S.Q4_K, 96, 512
    w = S.gen_weight(t, rows, cols, seed=42)
    x = S.gen_acts(1, cols, seed=42)[0]
    want, _ = run(simd, t, simd.qk_cpu_best_tier(), 1, w, rows, cols, x)
    for i in range(200):
        y, _ = run(simd, t, simd.qk_cpu_best_tier(), 1 + i % 6, w, rows, cols, x)
        assert np.array_equal(y, want)   # a row's sum does not depend on who computes it
