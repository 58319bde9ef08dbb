"""CPU-side checks of the boundary: the library loads, exports every symbol the
header declares, the getters answer without a GPU, and compute entry points
fail loudly (never fall back) when no CUDA device is present."""
import ctypes as C
import os
import re

import numpy as np
import pytest

from oxillama_b200 import _lib, synth as S

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    src = open(os.path.join(ROOT, "include", "qk_cuda.h")).read()
    src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
    return sorted(set(re.findall(r"\b(qk_[a-z0-9_]+)\s*\(", src)))


@pytest.fixture(scope="module")
def lib():
    from oxillama_b200 import build
    build.build()
    return _lib.load()


def test_exports_every_declared_symbol(lib):
    declared = _declared_symbols()
    assert len(declared) >= 20
    for name in declared:
        assert hasattr(lib, name), f"{name} declared in include/qk_cuda.h but not exported"
    assert sorted(_lib.SIGNATURES) == declared


def test_trait_getters_need_no_gpu(lib):
    # crates/oxillama-gguf/src/types.rs:199-259
    for t in S.ALL_TYPES + S.NEXT_TYPES:
        assert lib.qk_block_size(t) == S.BLOCK_SIZE[t]
        assert lib.qk_block_bytes(t) == S.BLOCK_BYTES[t]
        assert lib.qk_name(t).decode() == S.NAMES[t]
    assert lib.qk_block_size(16) == 0 and lib.qk_name(16) is None   # IQ2_XXS: not served


def test_no_cpu_fallback(lib):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    h = C.c_void_p()
    assert lib.qk_init(0, C.byref(h)) == 100  # QK_CUDA_ERROR
    assert not h.value
    from oxillama_b200.kernels import Context, QuantError
    with pytest.raises(QuantError):
        Context(0)


def test_null_context_is_rejected(lib):
    x = np.zeros(32, np.float32)
    assert lib.qk_gemv(None, S.Q4_0, None, 0, 0, 0, C.c_void_p(x.ctypes.data), 32,
                       C.c_void_p(x.ctypes.data), 32) == 102


def test_synth_blocks_are_legal():
    for t in S.ALL_TYPES:
        w = S.gen_weight(t, 5, 600, seed=3)
        assert w.size == S.weight_nbytes(t, 5, 600)
        bb = S.BLOCK_BYTES[t]
        off = 208 if t == S.Q6_K else 0
        d = w.reshape(-1, bb)[:, off:off + 2].copy().view(np.float16).astype(np.float32)
        assert np.all(np.isfinite(d)) and np.all(d > 0)
    assert np.array_equal(S.gen_weight(S.Q4_K, 2, 256, 7), S.gen_weight(S.Q4_K, 2, 256, 7))
    assert not np.array_equal(S.gen_weight(S.Q4_K, 2, 256, 7), S.gen_weight(S.Q4_K, 2, 256, 8))
