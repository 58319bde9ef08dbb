"""ctypes binding to libqk_cuda.so (the C ABI declared in include/qk_cuda.h).

There is no fallback: if the shared library is missing or no CUDA device can be
opened, the error is raised to the caller.
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("QK_CUDA_LIB") or os.path.join(_HERE, "libqk_cuda.so")

u8p = C.POINTER(C.c_uint8)
f32p = C.POINTER(C.c_float)
vp = C.c_void_p
sz = C.c_size_t

# every symbol include/qk_cuda.h declares, with its signature
SIGNATURES = {
    "qk_init": (C.c_int, [C.c_int, C.POINTER(vp)]),
    "qk_shutdown": (C.c_int, [vp]),
    "qk_last_error": (C.c_int, [vp, C.c_char_p, sz]),
    "qk_block_size": (sz, [C.c_int]),
    "qk_block_bytes": (sz, [C.c_int]),
    "qk_name": (C.c_char_p, [C.c_int]),
    "qk_dequant_block": (C.c_int, [vp, C.c_int, vp, sz, vp, sz]),
    "qk_dequant_matrix": (C.c_int, [vp, C.c_int, vp, sz, sz, sz, vp, sz]),
    "qk_gemv": (C.c_int, [vp, C.c_int, vp, sz, sz, sz, vp, sz, vp, sz]),
    "qk_gemm": (C.c_int, [vp, C.c_int, vp, sz, vp, sz, vp, sz, sz, sz, sz]),
    "qk_matvec_q8_fused": (C.c_int, [vp, C.c_int, vp, sz, vp, sz, vp, sz, sz, sz]),
    "qk_quantize_q8_0": (C.c_int, [vp, vp, sz, vp, sz]),
    "qk_gpu_gemv": (C.c_int, [vp, C.c_int, vp, sz, vp, sz, vp, sz, sz, sz]),
    "qk_gpu_gemv_batched": (C.c_int, [vp, C.c_int, vp, sz, vp, sz, vp, sz, sz, sz, sz]),
    "qk_weights_cache_evict": (C.c_int, [vp, vp]),
    "qk_weights_upload": (C.c_int, [vp, C.c_int, vp, sz, sz, sz, sz, sz, C.POINTER(vp)]),
    "qk_weights_free": (C.c_int, [vp, vp]),
    "qk_gguf_open": (C.c_int, [C.c_char_p, C.POINTER(vp)]),
    "qk_gguf_close": (C.c_int, [vp]),
    "qk_gguf_last_error": (C.c_int, [vp, C.c_char_p, sz]),
    "qk_gguf_tensor_count": (C.c_int, [vp, C.POINTER(sz)]),
    "qk_gguf_tensor_name": (C.c_int, [vp, sz, C.c_char_p, sz]),
    "qk_gguf_tensor_info": (C.c_int, [vp, C.c_char_p, C.POINTER(C.c_int), C.POINTER(sz), C.POINTER(C.c_uint64 * 4),
                                      C.POINTER(C.c_uint64), C.POINTER(C.c_uint64)]),
    "qk_weights_upload_gguf": (C.c_int, [vp, vp, C.c_char_p, sz, sz, C.POINTER(vp)]),
    "qk_weights_info": (C.c_int, [vp, C.POINTER(C.c_int), C.POINTER(sz), C.POINTER(sz), C.POINTER(sz)]),
    "qk_gemv_dev": (C.c_int, [vp, vp, vp, vp, vp]),
    "qk_gemm_dev": (C.c_int, [vp, vp, vp, vp, sz, sz, vp]),
    "qk_ffn_dev": (C.c_int, [vp, vp, vp, vp, vp, vp, sz, vp]),
    "qk_dequant_dev": (C.c_int, [vp, vp, vp, vp]),
    "qk_matvec_q8_fused_dev": (C.c_int, [vp, vp, vp, vp, vp]),
    "qk_quantize_q8_0_dev": (C.c_int, [vp, vp, sz, vp, vp]),
    "qk_gemm_dev_noalloc": (C.c_int, [vp, vp, vp, vp, sz, sz, vp]),
    "qk_gather_create": (C.c_int, [vp, sz, sz, C.c_int, C.c_int, vp]),
    "qk_gather_export": (C.c_int, [vp, vp, vp, sz]),
    "qk_gather_import": (C.c_int, [vp, vp, C.c_int, vp, sz]),
    "qk_gather_import_local": (C.c_int, [vp, vp, C.c_int, vp]),
    "qk_gather_ready": (C.c_int, [vp, vp]),
    "qk_gather_close_peers": (C.c_int, [vp, vp]),
    "qk_gather_destroy": (C.c_int, [vp, vp]),
    "qk_gather_buffer": (vp, [vp]),
    "qk_gemm_gather_dev": (C.c_int, [vp, vp, vp, sz, vp, vp]),
    "qk_gemm_gather_after_dev": (C.c_int, [vp, vp, vp, sz, vp, vp, vp]),
    "qk_gemm_gather_unpack_dev": (C.c_int, [vp, vp, vp, sz, vp, vp, vp, vp]),
    "qk_gather_wait_dev": (C.c_int, [vp, vp, vp]),
    "qk_moe_route_dev": (C.c_int, [vp, vp, sz, sz, sz, vp, vp, vp]),
    "qk_moe_take_rows_dev": (C.c_int, [vp, vp, vp, sz, sz, vp, vp]),
    "qk_moe_sum_rows_dev": (C.c_int, [vp, vp, vp, sz, sz, sz, vp, vp]),
    "qk_moe_ffn_dev": (C.c_int, [vp, vp, vp, vp, sz, sz, sz, vp, vp, vp, sz, sz, vp]),
    "qk_check_device_status": (C.c_int, [vp, vp]),
}

_lib = None


def load() -> C.CDLL:
    """Loads the library and types every entry point.  Raises if it is not built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise OSError(f"{LIB_PATH} is not built: run `python -m oxillama_b200.build`")
        lib = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name)  # AttributeError if the symbol is missing
            fn.restype = res
            fn.argtypes = args
        _lib = lib
    return _lib
