"""ctypes binding to the CPU oracle (oracle/qk_oracle.c).  Test-side only."""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
_ORACLE_DIR = os.path.join(_ROOT, "oracle")
_SO = os.path.join(_ORACLE_DIR, "_build", "libqk_oracle.so")

_u8p = C.POINTER(C.c_uint8)
_f32p = C.POINTER(C.c_float)
_i32p = C.POINTER(C.c_int32)


def _build():
    subprocess.check_call(["make", "-s", "-C", _ORACLE_DIR, "_build/libqk_oracle.so"])


def load():
    src = os.path.join(_ORACLE_DIR, "qk_oracle.c")
    if not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(src):
        _build()
    lib = C.CDLL(_SO)
    lib.qk_oracle_f16_to_f32.restype = C.c_float
    lib.qk_oracle_f16_to_f32.argtypes = [C.c_uint16]
    lib.qk_oracle_f32_to_f16.restype = C.c_uint16
    lib.qk_oracle_f32_to_f16.argtypes = [C.c_float]
    lib.qk_oracle_block_size.restype = C.c_size_t
    lib.qk_oracle_block_bytes.restype = C.c_size_t
    return lib


_lib = None


def lib():
    global _lib
    if _lib is None:
        _lib = load()
    return _lib


def _u8(a):
    a = np.ascontiguousarray(a, dtype=np.uint8)
    return a, a.ctypes.data_as(_u8p)


def _f32(a):
    a = np.ascontiguousarray(a, dtype=np.float32)
    return a, a.ctypes.data_as(_f32p)


def dequant_block(qtype, block, out_len=None):
    b, bp = _u8(block)
    n = out_len if out_len is not None else lib().qk_oracle_block_size(C.c_int(qtype))
    out = np.zeros(max(n, 1), np.float32)
    st = lib().qk_oracle_dequant_block(C.c_int(qtype), bp, C.c_size_t(b.size),
                                       out.ctypes.data_as(_f32p), C.c_size_t(n))
    return st, out[:n]


def dequant_matrix(qtype, w, n_rows, n_cols):
    wb, wp = _u8(w)
    out = np.empty((n_rows, n_cols), np.float32)
    st = lib().qk_oracle_dequant_matrix(C.c_int(qtype), wp, C.c_size_t(wb.size), C.c_size_t(n_rows),
                                        C.c_size_t(n_cols), out.ctypes.data_as(_f32p))
    assert st == 0, st
    return out


def gemv(qtype, w, n_rows, n_cols, x, y_len=None, wide=False):
    wb, wp = _u8(w)
    xb, xp = _f32(x)
    yl = n_rows if y_len is None else y_len
    y = np.zeros(max(yl, 1), np.float32)
    fn = lib().qk_oracle_gemv_f64 if wide else lib().qk_oracle_gemv
    st = fn(C.c_int(qtype), wp, C.c_size_t(wb.size), C.c_size_t(n_rows), C.c_size_t(n_cols),
            xp, C.c_size_t(xb.size), y.ctypes.data_as(_f32p), C.c_size_t(yl))
    return st, y[:yl]


def gemm(qtype, w, x, m, n, k, wide=False):
    wb, wp = _u8(w)
    xb, xp = _f32(x)
    y = np.zeros((m, n), np.float32)
    fn = lib().qk_oracle_gemm_f64 if wide else lib().qk_oracle_gemm
    st = fn(C.c_int(qtype), wp, C.c_size_t(wb.size), xp, y.ctypes.data_as(_f32p),
            C.c_size_t(m), C.c_size_t(n), C.c_size_t(k))
    return st, y


def matvec_q8_fused(qtype, w, acts, out, n_rows, n_cols):
    wb, wp = _u8(w)
    ab, ap = _u8(acts)
    o = np.ascontiguousarray(out, dtype=np.float32).copy()
    st = lib().qk_oracle_matvec_q8_fused(C.c_int(qtype), wp, C.c_size_t(wb.size), ap,
                                         C.c_size_t(ab.size), o.ctypes.data_as(_f32p),
                                         C.c_size_t(o.size), C.c_size_t(n_rows), C.c_size_t(n_cols))
    return st, o


def quantize_q8_0(x):
    xb, xp = _f32(x)
    out = np.zeros((xb.size // 32) * 34 + 34, np.uint8)
    st = lib().qk_oracle_quantize_q8_0(xp, C.c_size_t(xb.size), out.ctypes.data_as(_u8p))
    return st, out[: (xb.size // 32) * 34]


def moe_route(logits, top_k):
    lb, lp = _f32(logits)
    tokens, n_exp = lb.shape
    ids = np.zeros((tokens, top_k), np.int32)
    wts = np.zeros((tokens, top_k), np.float32)
    lib().qk_oracle_moe_route(lp, C.c_size_t(tokens), C.c_size_t(n_exp), C.c_size_t(top_k),
                              ids.ctypes.data_as(_i32p), wts.ctypes.data_as(_f32p))
    return ids, wts


def moe_ffn_f32(gate, up, down, logits, x, top_k, token_begin=0, token_end=None):
    gb, gp = _f32(gate)
    ub, up_ = _f32(up)
    db, dp = _f32(down)
    lb, lp = _f32(logits)
    xb, xp = _f32(x)
    n_exp, inter, hidden = gb.shape
    tokens = xb.shape[0]
    y = np.zeros((tokens, hidden), np.float32)
    te = tokens if token_end is None else token_end
    st = lib().qk_oracle_moe_ffn_f32(gp, up_, dp, lp, xp, y.ctypes.data_as(_f32p), C.c_size_t(tokens),
                                     C.c_size_t(n_exp), C.c_size_t(top_k), C.c_size_t(hidden),
                                     C.c_size_t(inter), C.c_size_t(token_begin), C.c_size_t(te))
    assert st == 0
    return y


def ffn(type_gu, gate, up, type_d, down, x, m, hidden, inter, out_rows):
    """down(silu(gate x) * up x) for m rows of x (feed_forward's dense branch with swiglu_inplace)."""
    gb, gp = _u8(gate)
    ub, up_ = _u8(up)
    db, dp = _u8(down)
    xb, xp = _f32(x)
    y = np.zeros((m, out_rows), np.float32)
    scratch = np.zeros(2 * inter, np.float32)
    st = lib().qk_oracle_ffn(C.c_int(type_gu), gp, up_, C.c_size_t(gb.size), C.c_int(type_d), dp, C.c_size_t(db.size),
                             xp, y.ctypes.data_as(_f32p), C.c_size_t(m), C.c_size_t(hidden), C.c_size_t(inter),
                             C.c_size_t(out_rows), scratch.ctypes.data_as(_f32p))
    return st, y


def f16_bits(x: float) -> int:
    return int(lib().qk_oracle_f32_to_f16(C.c_float(x)))
