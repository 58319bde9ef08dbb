"""GGUF files as the device loader sees them: header and tensor registry parsed natively
(`qk_gguf_open`), tensor bytes read straight into pinned staging memory on upload.

Mirrors what the reference's loader exposes for this path: `GgufFile::parse`
(crates/oxillama-gguf/src/parser.rs:34-60), `TensorInfo` (tensor_info.rs:25-57) and
`tensor_data(name)` (parser.rs:62-76), whose bytes `load_quant_linear`
(crates/oxillama-arch/src/llama/model.rs:805-822) turns into a layer's weights.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

from . import _lib
from .kernels import QuantError


@dataclass
class TensorInfo:
    name: str
    n_dims: int
    dims: tuple          # in file order; dims[0] is read as the row count (out_features)
    tensor_type: int     # GGUF type id
    file_offset: int     # absolute
    nbytes: int          # TensorInfo::data_size; 0 for a type this backend does not serve


class GgufFile:
    def __init__(self, path: str):
        self.lib = _lib.load()
        h = C.c_void_p()
        st = self.lib.qk_gguf_open(str(path).encode(), C.byref(h))
        self.handle = h
        if st != 0:
            msg = self.last_error()
            self.close()
            raise QuantError(st, msg)

    def last_error(self) -> str:
        buf = C.create_string_buffer(512)
        self.lib.qk_gguf_last_error(self.handle, buf, 512)
        return buf.value.decode()

    def names(self) -> list:
        n = C.c_size_t()
        self.lib.qk_gguf_tensor_count(self.handle, C.byref(n))
        out = []
        for i in range(n.value):
            buf = C.create_string_buffer(512)
            self.lib.qk_gguf_tensor_name(self.handle, i, buf, 512)
            out.append(buf.value.decode())
        return out

    def info(self, name: str) -> TensorInfo:
        t, nd, off, nb = C.c_int(), C.c_size_t(), C.c_uint64(), C.c_uint64()
        dims = (C.c_uint64 * 4)()
        st = self.lib.qk_gguf_tensor_info(self.handle, name.encode(), C.byref(t), C.byref(nd), C.byref(dims),
                                          C.byref(off), C.byref(nb))
        if st != 0:
            raise KeyError(name)
        return TensorInfo(name, nd.value, tuple(int(d) for d in dims[: nd.value]), t.value, off.value, nb.value)

    def close(self):
        if self.handle:
            self.lib.qk_gguf_close(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
