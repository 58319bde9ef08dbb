"""The allocation-free entry point, `qk_gemm_dev_noalloc`, against `qk_gemm_dev`.

Who needs it: a caller that may not allocate device memory once it is running —
a serving process that gave all of HBM to its own pools at start-up, a job under
a fixed memory budget, a loop that must not take the driver's allocator lock.
The entry point keeps its scratch in a 96 KiB array built into the library, so
this test checks (through the C ABI, as a binding would call it) that it returns
what the regular entry point returns, on two calls in a row — the second call
finds the array full of the first call's data — and that it refuses a request
whose scratch would not fit.

Collected last on purpose: a run that stops at the first failure has by then
run every other test.  It also passes alone in a fresh process.
"""
import ctypes as C

import numpy as np
import pytest

from oxillama_b200 import synth as S

pytestmark = pytest.mark.gpu

TOL_F32 = 2e-5  # the bar the other GPU tests hold the decode kernels to


def _setup(rows, cols, m, seed):
    import torch
    from oxillama_b200.device import DeviceWeights
    from oxillama_b200.kernels import default_context
    ctx = default_context()
    w = S.gen_weight(S.Q4_K, rows, cols, seed=seed)
    dw = DeviceWeights(S.Q4_K, w, rows, cols, ctx=ctx)
    x = torch.from_numpy(S.gen_acts(m, cols, seed=seed)).cuda()
    return torch, ctx, dw, x


def _noalloc(ctx, dw, x, y, m, ldy):
    import torch
    return ctx.lib.qk_gemm_dev_noalloc(ctx.handle, dw.handle, C.c_void_p(x.data_ptr()),
                                       C.c_void_p(y.data_ptr()), m, ldy,
                                       C.c_void_p(torch.cuda.current_stream().cuda_stream))


@pytest.mark.parametrize("rows,cols,m", [(64, 4096, 1), (203, 2048, 3), (72, 8192, 3)])
def test_noalloc_matches_regular_entry_point_twice(rows, cols, m):
    torch, ctx, dw, x = _setup(rows, cols, m, seed=51)
    y_ref = torch.full((m, rows), float("nan"), device="cuda")
    dw.gemm(x, y_ref, m)
    torch.cuda.synchronize()
    ref = y_ref.cpu().numpy()
    den = np.abs(ref).max()
    for call in range(2):  # the second call starts from the first call's scratch contents
        y = torch.full((m, rows), float("nan"), device="cuda")
        xin = x if call == 0 else x * 0.5
        assert _noalloc(ctx, dw, xin, y, m, rows) == 0, ctx.last_error()
        torch.cuda.synchronize()
        got = y.cpu().numpy()
        want = ref if call == 0 else ref * 0.5
        assert np.all(np.isfinite(got))
        assert np.abs(got - want).max() / den <= TOL_F32
    from oxillama_b200.device import check_device_status
    check_device_status(ctx)
    dw.free()


def test_noalloc_refuses_what_does_not_fit():
    # 4 rows of 8 192 columns split into 3 digit planes: ~107 KB of scratch > 96 KiB,
    # a shape the regular entry point serves
    torch, ctx, dw, x = _setup(8, 8192, 4, seed=52)
    y_ok = torch.zeros((4, 8), device="cuda")
    dw.gemm(x, y_ok, 4)
    y = torch.zeros((4, 8), device="cuda")
    assert _noalloc(ctx, dw, x, y, 4, 8) == 102  # QK_INVALID_ARGUMENT
    assert "built-in scratch" in ctx.last_error()
    assert _noalloc(ctx, dw, x, y, 5, 8) == 102  # more activation rows than the decode kernel takes
    dw.free()
    # other formats are not served here
    from oxillama_b200.device import DeviceWeights
    w8 = DeviceWeights(S.Q8_0, S.gen_weight(S.Q8_0, 8, 256, seed=53), 8, 256, ctx=ctx)
    x8 = torch.zeros((1, 256), device="cuda")
    assert _noalloc(ctx, w8, x8, y, 1, 8) == 1  # QK_UNSUPPORTED_TYPE
    w8.free()
