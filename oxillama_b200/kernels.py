"""Host-side mirror of the reference's kernel interface, served by the CUDA library.

Names, argument meaning and error behaviour follow `QuantKernel`
(crates/oxillama-quant/src/traits.rs:21-183), `QuantTensor`
(crates/oxillama-quant/src/types.rs:11-49), `QuantError`
(crates/oxillama-quant/src/error.rs:10-71) and
`KernelDispatcher::get_kernel` (crates/oxillama-quant/src/dispatch.rs:141-243)
of the reference, so a test written against those reads the same here.  Slices
become numpy arrays; `output` arrays are written in place.
"""
from __future__ import annotations

import ctypes as C
import os
from dataclasses import dataclass

import numpy as np

from . import _lib
from .synth import BLOCK_BYTES, BLOCK_SIZE, IQ4_XS, NAMES, Q4_0, Q4_K, Q6_K, Q8_0  # noqa: F401

STATUS_NAMES = {
    1: "UnsupportedType", 2: "BlockSizeMismatch", 3: "DimensionMismatch", 4: "KernelError",
    5: "BlockCountMismatch", 6: "BufferTooSmall", 7: "Internal", 100: "CudaError", 101: "Timeout",
    102: "InvalidArgument",
}


class QuantError(Exception):
    """Mirror of QuantError: `.kind` is the variant name, `.code` the C status."""

    def __init__(self, code: int, detail: str = ""):
        self.code = code
        self.kind = STATUS_NAMES.get(code, f"Status{code}")
        super().__init__(f"{self.kind}{': ' + detail if detail else ''}")


@dataclass
class QuantTensor:
    """Raw GGUF block bytes plus shape and type tag (types.rs:11-18)."""
    data: np.ndarray  # uint8
    shape: tuple
    tensor_type: int

    def __post_init__(self):
        self.data = np.ascontiguousarray(self.data, dtype=np.uint8).reshape(-1)
        self.shape = tuple(int(s) for s in self.shape)
        # the bytes do not move while the tensor lives: their address is taken once, not per call
        self._addr = C.c_void_p(self.data.ctypes.data)
        self._rc = None

    def n_elements(self) -> int:
        return int(np.prod(self.shape)) if self.shape else 0

    def n_blocks(self) -> int:
        bs = BLOCK_SIZE.get(self.tensor_type, 0)
        return 0 if bs == 0 else -(-self.n_elements() // bs)

    def expected_data_size(self) -> int:
        return self.n_blocks() * BLOCK_BYTES.get(self.tensor_type, 0)

    def rows_cols(self):
        if self._rc is None:
            n_rows = self.shape[0]
            n_cols = self.shape[1] if len(self.shape) > 1 else (self.n_elements() // n_rows if n_rows else 0)
            self._rc = (n_rows, n_cols)
        return self._rc


class Context:
    """One GPU.  Stands where `KernelDispatcher::new()` stands in the reference."""

    def __init__(self, device: int = 0):
        self.lib = _lib.load()
        h = C.c_void_p()
        st = self.lib.qk_init(device, C.byref(h))
        if st != 0:
            raise QuantError(st, f"qk_init(device={device}) failed: no usable sm_100 CUDA device")
        self.handle = h
        self.device = device

    def close(self):
        if self.handle:
            self.lib.qk_shutdown(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def last_error(self) -> str:
        buf = C.create_string_buffer(512)
        self.lib.qk_last_error(self.handle, buf, 512)
        return buf.value.decode()

    def check(self, st: int):
        if st != 0:
            raise QuantError(st, self.last_error() if st >= 100 else "")


_default_ctx = None


def default_context() -> Context:
    """The process-wide context: on the GPU named by LOCAL_RANK (one process per GPU), else GPU 0."""
    global _default_ctx
    if _default_ctx is None:
        _default_ctx = Context(int(os.environ.get("LOCAL_RANK", "0")))
    return _default_ctx


def _ptr(a: np.ndarray):
    """Address of an array's first byte.  `ndarray.ctypes` builds a helper object per access
    (about a microsecond); the buffer protocol gives the same address in less than half."""
    try:
        return C.c_void_p(C.addressof(C.c_char.from_buffer(a))) if a.size else C.c_void_p(a.ctypes.data)
    except (TypeError, ValueError, BufferError):  # read-only or exotic buffers
        return C.c_void_p(a.ctypes.data)


def _u8(a):
    return np.ascontiguousarray(a, dtype=np.uint8).reshape(-1)


def _f32_in(a):
    if isinstance(a, np.ndarray) and a.dtype == np.float32 and a.flags.c_contiguous:
        return a  # only its address and its size are used
    return np.ascontiguousarray(a, dtype=np.float32).reshape(-1)


def _f32_out(a: np.ndarray):
    if not (isinstance(a, np.ndarray) and a.dtype == np.float32 and a.flags.c_contiguous and a.flags.writeable):
        raise TypeError("output must be a writable C-contiguous float32 ndarray")
    return a


class CudaQuantKernel:
    """`dyn QuantKernel` for one tensor type, computed on the GPU."""

    def __init__(self, tensor_type: int, ctx: Context | None = None):
        self.tensor_type = tensor_type
        self.ctx = ctx or default_context()
        self._lib = self.ctx.lib

    # -- getters (traits.rs:175-182)
    def block_size(self) -> int:
        return self._lib.qk_block_size(self.tensor_type)

    def block_bytes(self) -> int:
        return self._lib.qk_block_bytes(self.tensor_type)

    def name(self) -> str:
        return self._lib.qk_name(self.tensor_type).decode()

    # -- dequant_block (traits.rs:28)
    def dequant_block(self, block, output: np.ndarray) -> None:
        b, o = _u8(block), _f32_out(output)
        self.ctx.check(self._lib.qk_dequant_block(self.ctx.handle, self.tensor_type, _ptr(b), b.size,
                                                  _ptr(o), o.size))

    def dequant_matrix(self, quant_matrix: QuantTensor, output: np.ndarray) -> None:
        n_rows, n_cols = quant_matrix.rows_cols()
        o = _f32_out(output)
        self.ctx.check(self._lib.qk_dequant_matrix(self.ctx.handle, self.tensor_type, _ptr(quant_matrix.data),
                                                   quant_matrix.data.size, n_rows, n_cols, _ptr(o), o.size))

    # -- gemv (traits.rs:40-45): output overwritten
    def gemv(self, quant_matrix: QuantTensor, input, output: np.ndarray) -> None:
        n_rows, n_cols = quant_matrix.rows_cols()
        x, y = _f32_in(input), _f32_out(output)
        self.ctx.check(self._lib.qk_gemv(self.ctx.handle, self.tensor_type, quant_matrix._addr,
                                         quant_matrix.data.size, n_rows, n_cols, _ptr(x), x.size, _ptr(y), y.size))

    # -- gemm (traits.rs:59-67): input [m x k], output [m x n]
    def gemm(self, quant_matrix: QuantTensor, input, output: np.ndarray, m: int, n: int, k: int) -> None:
        x, y = _f32_in(input), _f32_out(output)
        self.ctx.check(self._lib.qk_gemm(self.ctx.handle, self.tensor_type, quant_matrix._addr,
                                         quant_matrix.data.size, _ptr(x), x.size, _ptr(y), y.size, m, n, k))

    # -- matvec_q8_fused (traits.rs:89-173): out accumulated
    def matvec_q8_fused(self, weights, acts_q8, out: np.ndarray, n_rows: int, n_cols: int) -> None:
        w, a, o = _u8(weights), _u8(acts_q8), _f32_out(out)
        self.ctx.check(self._lib.qk_matvec_q8_fused(self.ctx.handle, self.tensor_type, _ptr(w), w.size,
                                                    _ptr(a), a.size, _ptr(o), o.size, n_rows, n_cols))


class KernelDispatcher:
    """`KernelDispatcher::get_kernel(GgufTensorType)` (dispatch.rs:141-243), CUDA arm only."""

    def __init__(self, ctx: Context | None = None):
        self.ctx = ctx or default_context()

    def get_kernel(self, tensor_type: int) -> CudaQuantKernel:
        if self.ctx.lib.qk_block_size(tensor_type) == 0:
            raise QuantError(1, f"type id {tensor_type}")
        return CudaQuantKernel(tensor_type, self.ctx)


def quantize_f32_to_q8_0(data, ctx: Context | None = None) -> np.ndarray:
    """quantize.rs:58-75: f32 -> Q8_0 blocks; length must be a multiple of 32."""
    ctx = ctx or default_context()
    x = _f32_in(data)
    out = np.empty(x.size // 32 * 34, np.uint8)
    ctx.check(ctx.lib.qk_quantize_q8_0(ctx.handle, _ptr(x), x.size, _ptr(out), out.size))
    return out
