"""Device-resident side of the C ABI: weights uploaded once, torch tensors as buffers.

PyTorch is only the owner of device memory and streams here; every kernel is
launched by libqk_cuda.so on the stream torch reports as current.
"""
from __future__ import annotations

import ctypes as C

import numpy as np
import torch

from .kernels import Context, QuantError, default_context


def _stream_ptr(stream=None) -> C.c_void_p:
    s = stream if stream is not None else torch.cuda.current_stream()
    return C.c_void_p(s.cuda_stream)


class DeviceWeights:
    """Rows [row_begin, row_end) of a [n_rows x n_cols] GGUF-layout matrix, resident in HBM."""

    def __init__(self, tensor_type: int, data: np.ndarray, n_rows: int, n_cols: int,
                 row_begin: int = 0, row_end: int | None = None, ctx: Context | None = None):
        self.ctx = ctx or default_context()
        self.tensor_type = tensor_type
        data = np.ascontiguousarray(data, dtype=np.uint8).reshape(-1)
        row_end = n_rows if row_end is None else row_end
        h = C.c_void_p()
        self.ctx.check(self.ctx.lib.qk_weights_upload(
            self.ctx.handle, tensor_type, C.c_void_p(data.ctypes.data), data.size, n_rows, n_cols,
            row_begin, row_end, C.byref(h)))
        self.handle = h
        self.rows, self.cols = row_end - row_begin, n_cols
        t, r, c, b = C.c_int(), C.c_size_t(), C.c_size_t(), C.c_size_t()
        self.ctx.lib.qk_weights_info(h, C.byref(t), C.byref(r), C.byref(c), C.byref(b))
        self.algo_bytes = b.value

    @classmethod
    def from_gguf(cls, gguf, name: str, row_begin: int = 0, row_end: int | None = None,
                  ctx: Context | None = None) -> "DeviceWeights":
        """Rows [row_begin, row_end) of tensor `name` of an open `gguf.GgufFile`, read from the file
        through pinned staging memory (`qk_weights_upload_gguf`)."""
        self = cls.__new__(cls)
        self.ctx = ctx or default_context()
        info = gguf.info(name)
        n_rows = info.dims[0] if info.n_dims else 0
        row_end = n_rows if row_end is None else row_end
        h = C.c_void_p()
        self.ctx.check(self.ctx.lib.qk_weights_upload_gguf(self.ctx.handle, gguf.handle, name.encode(), row_begin,
                                                           row_end, C.byref(h)))
        self.handle, self.tensor_type = h, info.tensor_type
        t, r, c, b = C.c_int(), C.c_size_t(), C.c_size_t(), C.c_size_t()
        self.ctx.lib.qk_weights_info(h, C.byref(t), C.byref(r), C.byref(c), C.byref(b))
        self.rows, self.cols, self.algo_bytes = r.value, c.value, b.value
        return self

    def free(self):
        if self.handle:
            self.ctx.lib.qk_weights_free(self.ctx.handle, self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass

    @staticmethod
    def _chk(t: torch.Tensor, dtype, n: int, what: str):
        if not (t.is_cuda and t.dtype == dtype and t.is_contiguous()):
            raise TypeError(f"{what}: need a contiguous CUDA tensor of {dtype}")
        if t.numel() < n:
            raise QuantError(3, f"{what}: expected {n} elements, got {t.numel()}")

    def gemv(self, x: torch.Tensor, y: torch.Tensor, stream=None) -> None:
        """y[0:rows] = W x (overwrites)."""
        self._chk(x, torch.float32, self.cols, "input")
        self._chk(y, torch.float32, self.rows, "output")
        self.ctx.check(self.ctx.lib.qk_gemv_dev(self.ctx.handle, self.handle, C.c_void_p(x.data_ptr()),
                                                C.c_void_p(y.data_ptr()), _stream_ptr(stream)))

    def gemm(self, x: torch.Tensor, y: torch.Tensor, m: int, ldy: int | None = None,
             col_offset: int = 0, stream=None) -> None:
        """y[i, col_offset + j] = dot(W row j, x row i); y has row pitch ldy (default rows)."""
        ldy = self.rows if ldy is None else ldy
        self._chk(x, torch.float32, m * self.cols, "input")
        self._chk(y, torch.float32, (m - 1) * ldy + col_offset + self.rows if m else 0, "output")
        self.ctx.check(self.ctx.lib.qk_gemm_dev(
            self.ctx.handle, self.handle, C.c_void_p(x.data_ptr()),
            C.c_void_p(y.data_ptr() + 4 * col_offset), m, ldy, _stream_ptr(stream)))

    def dequant(self, out: torch.Tensor, stream=None) -> None:
        self._chk(out, torch.float32, self.rows * self.cols, "output")
        self.ctx.check(self.ctx.lib.qk_dequant_dev(self.ctx.handle, self.handle, C.c_void_p(out.data_ptr()),
                                                   _stream_ptr(stream)))

    def matvec_q8_fused(self, acts_q8: torch.Tensor, out: torch.Tensor, stream=None) -> None:
        bs = self.ctx.lib.qk_block_size(self.tensor_type)
        self._chk(acts_q8, torch.uint8, -(-self.cols // bs) * (bs // 32) * 34, "acts_q8")
        self._chk(out, torch.float32, self.rows, "out")
        self.ctx.check(self.ctx.lib.qk_matvec_q8_fused_dev(
            self.ctx.handle, self.handle, C.c_void_p(acts_q8.data_ptr()), C.c_void_p(out.data_ptr()),
            _stream_ptr(stream)))


def quantize_q8_0_dev(x: torch.Tensor, out: torch.Tensor, ctx: Context | None = None, stream=None) -> None:
    ctx = ctx or default_context()
    ctx.check(ctx.lib.qk_quantize_q8_0_dev(ctx.handle, C.c_void_p(x.data_ptr()), x.numel(),
                                           C.c_void_p(out.data_ptr()), _stream_ptr(stream)))


def check_device_status(ctx: Context | None = None, stream=None) -> None:
    ctx = ctx or default_context()
    ctx.check(ctx.lib.qk_check_device_status(ctx.handle, _stream_ptr(stream)))


def ffn(gate: DeviceWeights, up: DeviceWeights, down: DeviceWeights, x: torch.Tensor, y: torch.Tensor, m: int = 1,
        stream=None) -> None:
    """y[m x down.rows] = down(silu(gate x) * up x): the dense branch of the reference's
    `feed_forward` (crates/oxillama-arch/src/llama/model.rs:281-310) as one call (`qk_ffn_dev`)."""
    DeviceWeights._chk(x, torch.float32, m * gate.cols, "input")
    DeviceWeights._chk(y, torch.float32, m * down.rows, "output")
    ctx = gate.ctx
    ctx.check(ctx.lib.qk_ffn_dev(ctx.handle, gate.handle, up.handle, down.handle, C.c_void_p(x.data_ptr()),
                                 C.c_void_p(y.data_ptr()), m, _stream_ptr(stream)))
