"""Mirror of the reference's second operator surface, `GpuKernel`
(crates/oxillama-gpu/src/kernels/mod.rs:91-106) and `batched_gemv_f32`
(kernels/batched_gemv.rs:36-50), served by the CUDA library.

The reference's implementations dequantise on the host and dispatch an f32 shader through
a graphics API; here the same call (raw weight bytes, input, output, rows, cols) runs the
fused CUDA kernels.  Element order follows the CPU crate (`oxillama-quant`), as `qk_gemv`
does.  Errors are `GpuError` with the reference's variant names.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from .kernels import Context, default_context
from .synth import IQ4_XS, Q4_0, Q4_K, Q6_K, Q8_0


class GpuError(Exception):
    """`GpuError` (crates/oxillama-gpu/src/error.rs:7-31): `.kind` is the variant name."""

    def __init__(self, kind: str, detail: str = ""):
        self.kind = kind
        super().__init__(f"{kind}{': ' + detail if detail else ''}")


class GpuContext:
    """Stands where `GpuContext` (device + queue) stands; wraps one CUDA context."""

    def __init__(self, ctx: Context | None = None):
        self.ctx = ctx or default_context()


def _raise(gctx: GpuContext, st: int):
    if st == 0:
        return
    detail = gctx.ctx.last_error()
    if st == 6:
        raise GpuError("BufferSize", detail)
    if st == 1:
        raise GpuError("UnsupportedType", detail)
    raise GpuError("DeviceRequest", f"status {st}: {detail}")


class _Kernel:
    tensor_type = 0

    def gemv(self, ctx: GpuContext, weight_bytes, input, output: np.ndarray, rows: int, cols: int) -> None:
        """output[i] = sum_j weight[i*cols + j] * input[j] (mod.rs:97-105); output is written in place."""
        w = np.ascontiguousarray(weight_bytes, dtype=np.uint8).reshape(-1)
        x = np.ascontiguousarray(input, dtype=np.float32).reshape(-1)
        if not (isinstance(output, np.ndarray) and output.dtype == np.float32 and output.flags.c_contiguous):
            raise TypeError("output must be a C-contiguous float32 ndarray")
        y = output.reshape(-1)
        lib, h = ctx.ctx.lib, ctx.ctx.handle
        _raise(ctx, lib.qk_gpu_gemv(h, self.tensor_type, C.c_void_p(w.ctypes.data), w.size, C.c_void_p(x.ctypes.data),
                                    x.size, C.c_void_p(y.ctypes.data), y.size, rows, cols))


class Q4_0GpuKernel(_Kernel):
    tensor_type = Q4_0


class Q8_0GpuKernel(_Kernel):
    tensor_type = Q8_0


class Q4_KGpuKernel(_Kernel):
    tensor_type = Q4_K


class Q6_KGpuKernel(_Kernel):
    tensor_type = Q6_K


class Iq4XsGpuKernel(_Kernel):
    tensor_type = IQ4_XS


def batched_gemv(ctx: GpuContext, tensor_type: int, weight_bytes, vectors, rows: int, cols: int,
                 batch_size: int) -> np.ndarray:
    """Y[b, r] = sum_c A[r, c] X[b, c] (batched_gemv.rs:36-50) for a quantised A; returns Y [batch x rows]."""
    w = np.ascontiguousarray(weight_bytes, dtype=np.uint8).reshape(-1)
    x = np.ascontiguousarray(vectors, dtype=np.float32).reshape(-1)
    y = np.zeros((batch_size, rows), np.float32)
    lib, h = ctx.ctx.lib, ctx.ctx.handle
    _raise(ctx, lib.qk_gpu_gemv_batched(h, tensor_type, C.c_void_p(w.ctypes.data), w.size, C.c_void_p(x.ctypes.data),
                                        x.size, C.c_void_p(y.ctypes.data), y.size, rows, cols, batch_size))
    return y
