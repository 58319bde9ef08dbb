"""Pins the CPU oracle against the known-answer tests the reference holds for this path.

Each case is re-typed from a unit test of the reference (cited by
crates/oxillama-quant/src/<file>:<line>); blocks are built the way the
reference's `make_*_block` helpers build them.  Further down, two independent
second opinions: a numpy restatement of every dequant formula, and gguf-py's
dequantiser for the three layouts that are canonical GGUF.
"""
import numpy as np
import pytest

import oracle_lib as O
from oxillama_b200 import synth as S

OK, UNSUPPORTED, DIM, BUF = 0, 1, 3, 6


def f16b(x):
    return np.array([x], np.float32).astype(np.float16).view(np.uint8)


def q4_0_block(scale, nibbles):
    return np.concatenate([f16b(scale), np.asarray(nibbles, np.uint8)])


def q8_0_block(scale, vals):
    return np.concatenate([f16b(scale), np.asarray(vals, np.int8).view(np.uint8)])


def q4_k_block(d, dmin, scales, qs):
    return np.concatenate([f16b(d), f16b(dmin), np.asarray(scales, np.uint8), np.asarray(qs, np.uint8)])


def iq4_xs_block(scale, sub_scales, nibbles):
    sh = 0
    sl = np.zeros(4, np.uint8)
    for i, v in enumerate(sub_scales):
        v &= 0x3F
        sl[i // 2] |= (v & 0xF) << (4 * (i & 1))
        sh |= ((v >> 4) & 3) << (2 * i)
    return np.concatenate([f16b(scale), np.array([sh & 0xFF, sh >> 8], np.uint8), sl,
                           np.asarray(nibbles, np.uint8)])


Q8_VALS_A = [1, -2, 3, -4, 5, -6, 7, -8, 9, -10, 11, -12, 13, -14, 15, -16,
             -1, 2, -3, 4, -5, 6, -7, 8, -9, 10, -11, 12, -13, 14, -15, 16]


def q5_k_block(d, dmin, scales, qh, qs):
    return np.concatenate([f16b(d), f16b(dmin), np.asarray(scales, np.uint8), np.asarray(qh, np.uint8),
                           np.asarray(qs, np.uint8)])


# ------------------------------------------------------------------ Q5_K (a "next" format: generic kernels)
Q5_SC1 = [1, 1, 1, 1, 0, 0, 0, 0, 1, 1, 1, 1]


def test_q5_k_dequant():  # reference/q5_k.rs:376-440
    st, out = O.dequant_block(S.Q5_K, q5_k_block(0.0, 0.0, [0] * 12, [0] * 32, [0] * 128))
    assert st == OK and np.all(out == 0.0)
    st, out = O.dequant_block(S.Q5_K, q5_k_block(1.0, 0.0, Q5_SC1, [0] * 32, [0x88] * 128))
    assert st == OK and np.all(out == 8.0)
    st, out = O.dequant_block(S.Q5_K, q5_k_block(1.0, 0.0, Q5_SC1, [0xFF] * 32, [0] * 128))
    assert st == OK and np.all(out == 16.0)   # the fifth bit alone


def test_q5_k_high_bit_positions():  # reference/q5_k.rs:87-101: bit g for low nibbles of group g, bit g + 4 for high
    for bit in range(8):
        st, out = O.dequant_block(S.Q5_K, q5_k_block(1.0, 0.0, Q5_SC1, [1 << bit] * 32, [0] * 128))
        g, hi = bit % 4, bit // 4
        want = np.zeros(256, np.float32)
        want[64 * g + 32 * hi: 64 * g + 32 * hi + 32] = 16.0
        assert st == OK and np.array_equal(out, want), bit


def test_q5_k_gemv_matches_dequant_dot():  # reference/q5_k.rs:442-475
    scales = [(i * 17 + 3) & 0xFF for i in range(12)]
    qh = [(i * 13 + 7) & 0xFF for i in range(32)]
    qs = [(i * 5 + 11) & 0xFF for i in range(128)]
    blk = q5_k_block(0.5, 0.25, scales, qh, qs)
    st, dq = O.dequant_block(S.Q5_K, blk)
    x = (np.arange(256, dtype=np.float32) * np.float32(0.01)) - np.float32(1.28)
    st, y = O.gemv(S.Q5_K, blk, 1, 256, x)
    assert st == OK and abs(float(y[0]) - float((dq * x).sum())) < 0.1


def test_q5_k_fused_matches_unfused():  # reference/q5_k.rs:236-347 vs :137-189
    w = S.gen_weight(S.Q5_K, 3, 512, seed=12)
    x = S.gen_acts(1, 512, seed=12)[0]
    st, a = O.quantize_q8_0(x)
    st, out = O.matvec_q8_fused(S.Q5_K, w, a, np.zeros(3, np.float32), 3, 512)
    st2, y = O.gemv(S.Q5_K, w, 3, 512, x)
    assert st == OK and st2 == OK
    assert np.abs(out - y).max() / np.abs(y).max() < 2e-2   # activations rounded to 8 bits


# ------------------------------------------------------------------ Q2_K, Q3_K, Q8_K ("next" formats: generic kernels)
def q2_k_block(d, dmin, scales, qs):   # reference/q2_k.rs:323-330
    return np.concatenate([np.asarray(scales, np.uint8), np.asarray(qs, np.uint8), f16b(d), f16b(dmin)])


def q3_k_block(d, scales, hmask, qs):   # reference/q3_k.rs:357-364
    return np.concatenate([np.asarray(hmask, np.uint8), np.asarray(qs, np.uint8), np.asarray(scales, np.uint8), f16b(d)])


def q8_k_block(d, qs):   # reference/q8_k.rs:138-147
    return np.concatenate([np.array([d], np.float32).view(np.uint8), np.asarray(qs, np.int8).view(np.uint8),
                           np.zeros(32, np.uint8)])


RAMP = (np.arange(256, dtype=np.float32) * np.float32(0.01)) - np.float32(1.28)
Q3_SC1 = [0xA1] * 8 + [0x11] * 4   # all sixteen scales decode to +1 (raw 33), reference/q3_k.rs:405-421


def test_q2_k_dequant():  # reference/q2_k.rs:333-380
    st, out = O.dequant_block(S.Q2_K, q2_k_block(0.0, 0.0, [0] * 16, [0] * 64))
    assert st == OK and np.all(out == 0.0)
    st, out = O.dequant_block(S.Q2_K, q2_k_block(1.0, 0.0, [0x01] * 16, [0xFF] * 64))
    assert st == OK and np.all(out == 3.0)
    st, out = O.dequant_block(S.Q2_K, q2_k_block(2.0, 1.0, [0x11] * 16, [0x00] * 64))
    assert st == OK and np.all(out == -1.0)


def test_q2_k_element_order():  # reference/q2_k.rs:50-79: byte l of a 32-byte half holds weights l, 32 + l, 64 + l, 96 + l
    for byte in (0, 17, 40, 63):
        for shift in range(4):
            qs = [0] * 64
            qs[byte] = 3 << (2 * shift)
            st, out = O.dequant_block(S.Q2_K, q2_k_block(1.0, 0.0, [0x01] * 16, qs))
            want = np.zeros(256, np.float32)
            want[128 * (byte // 32) + 32 * shift + byte % 32] = 3.0
            assert st == OK and np.array_equal(out, want), (byte, shift)


def test_q2_k_gemv_matches_dequant_dot():  # reference/q2_k.rs:382-414
    blk = q2_k_block(0.5, 0.25, [0x21 + i for i in range(16)], [(i * 3 + 7) & 0xFF for i in range(64)])
    st, dq = O.dequant_block(S.Q2_K, blk)
    st, y = O.gemv(S.Q2_K, blk, 1, 256, RAMP)
    assert st == OK and abs(float(y[0]) - float((dq * RAMP).sum())) < 0.1


def test_q3_k_dequant():  # reference/q3_k.rs:366-458
    st, out = O.dequant_block(S.Q3_K, q3_k_block(0.0, [0] * 12, [0] * 32, [0] * 64))
    assert st == OK and np.all(out == 0.0)
    st, out = O.dequant_block(S.Q3_K, q3_k_block(1.0, [0x21] * 8 + [0] * 4, [0xFF] * 32, [0] * 64))
    assert st == OK and np.all(np.abs(out) < 0.01)
    st, out = O.dequant_block(S.Q3_K, q3_k_block(1.0, Q3_SC1, [0x00] * 32, [0x00] * 64))
    assert st == OK and np.all(out == -4.0)
    st, out = O.dequant_block(S.Q3_K, q3_k_block(1.0, Q3_SC1, [0xFF] * 32, [0xFF] * 64))
    assert st == OK and np.all(out == 3.0)


def test_q3_k_mask_bit_and_scale_positions():  # reference/q3_k.rs:29-59, :100-117
    # bit b of hmask byte k covers weight 32 b + k
    for bit in range(8):
        st, out = O.dequant_block(S.Q3_K, q3_k_block(1.0, Q3_SC1, [1 << bit] * 32, [0] * 64))
        want = np.full(256, -4.0, np.float32)
        want[32 * bit: 32 * bit + 32] = 0.0
        assert st == OK and np.array_equal(out, want), bit
    # sub-block i of 16 weights takes scale i: raw value 32 + (i + 1) packed per the 12-byte layout
    raw = [33 + i for i in range(16)]
    r = [0] * 12
    for j in range(4):
        r[j] = (raw[j] & 0x3F) | ((raw[8 + j] >> 4) << 6)
        r[4 + j] = (raw[4 + j] & 0x3F) | ((raw[12 + j] >> 4) << 6)
        r[8 + j] = (raw[8 + j] & 0x0F) | ((raw[12 + j] & 0x0F) << 4)
    st, out = O.dequant_block(S.Q3_K, q3_k_block(1.0, r, [0xFF] * 32, [0x55] * 64))   # every quant = 1
    assert st == OK and np.array_equal(out, np.repeat(np.arange(1, 17, dtype=np.float32), 16))


def test_q3_k_gemv_matches_dequant_dot():  # reference/q3_k.rs:460-501
    blk = q3_k_block(0.5, Q3_SC1, [(i * 7 + 3) & 0xFF for i in range(32)], [(i * 11 + 5) & 0xFF for i in range(64)])
    st, dq = O.dequant_block(S.Q3_K, blk)
    st, y = O.gemv(S.Q3_K, blk, 1, 256, RAMP)
    assert st == OK and abs(float(y[0]) - float((dq * RAMP).sum())) < 0.1


def test_q8_k_dequant_and_gemv():  # reference/q8_k.rs:150-217
    st, out = O.dequant_block(S.Q8_K, q8_k_block(0.0, [0] * 256))
    assert st == OK and np.all(out == 0.0)
    st, out = O.dequant_block(S.Q8_K, q8_k_block(0.25, [40] * 256))
    assert st == OK and np.all(out == 10.0)
    st, out = O.dequant_block(S.Q8_K, q8_k_block(1.0, [-100] * 256))
    assert st == OK and np.all(out == -100.0)
    blk = q8_k_block(0.25, [max(-128, min(127, i * 3 - 128)) for i in range(256)])
    st, dq = O.dequant_block(S.Q8_K, blk)
    st, y = O.gemv(S.Q8_K, blk, 1, 256, RAMP)
    assert st == OK and abs(float(y[0]) - float((dq * RAMP).sum())) < 0.1


@pytest.mark.parametrize("t", [S.Q2_K, S.Q3_K, S.Q8_K])
def test_next_formats_fused_matches_unfused(t):  # reference/q2_k.rs:187-297, q3_k.rs:217-336 against their gemv
    w = S.gen_weight(t, 3, 512, seed=13)
    x = S.gen_acts(1, 512, seed=13)[0]
    st, a = O.quantize_q8_0(x)
    st, out = O.matvec_q8_fused(t, w, a, np.zeros(3, np.float32), 3, 512)
    st2, y = O.gemv(t, w, 3, 512, x)
    assert st == OK and st2 == OK
    assert np.abs(out - y).max() / np.abs(y).max() < 3e-2   # activations rounded to 8 bits


@pytest.mark.parametrize("t", [S.Q2_K, S.Q3_K, S.Q8_K])
def test_next_formats_row_dot_against_numpy(t):
    """gemv against an independent numpy product of the oracle's own dequantised blocks (f64),
    full and ragged column counts."""
    for rows, cols in ((4, 768), (3, 256 + 100)):
        w = S.gen_weight(t, rows, cols, seed=14)
        x = S.gen_acts(1, cols, seed=14)[0]
        bpr = S.blocks_per_row(t, cols)
        dq = np.stack([np.concatenate([O.dequant_block(t, w[(r * bpr + b) * S.BLOCK_BYTES[t]:(r * bpr + b + 1) * S.BLOCK_BYTES[t]])[1]
                                       for b in range(bpr)])[:cols] for r in range(rows)])
        st, y = O.gemv(t, w, rows, cols, x)
        ref = dq.astype(np.float64) @ x.astype(np.float64)
        assert st == OK and np.abs(y - ref).max() / np.abs(ref).max() < 1e-5


# ------------------------------------------------------------------ Q4_0
def test_q4_0_dequant_zeros():  # reference/q4_0.rs:246-256
    st, out = O.dequant_block(S.Q4_0, q4_0_block(1.0, [0x88] * 16))
    assert st == OK and np.all(out == 0.0)


def test_q4_0_dequant_pins_interleave():  # reference/q4_0.rs:258-270
    nib = [0x88] * 16
    nib[0] = 0xF0
    st, out = O.dequant_block(S.Q4_0, q4_0_block(0.5, nib))
    assert st == OK
    assert out[0] == -4.0 and out[1] == 3.5  # low nibble -> element 0, high -> element 1
    assert np.all(out[2:] == 0.0)


def test_q4_0_gemv_gemm_zero():  # reference/q4_0.rs:272-308
    blk = q4_0_block(1.0, [0x88] * 16)
    st, y = O.gemv(S.Q4_0, blk, 1, 32, np.ones(32, np.float32))
    assert st == OK and y[0] == 0.0
    st, y = O.gemm(S.Q4_0, np.concatenate([blk, blk]), np.ones(64, np.float32), 2, 2, 32)
    assert st == OK and np.all(y == 0.0)


def test_q4_0_error_paths():  # reference/q4_0.rs:310-366
    blk = q4_0_block(1.0, [0x88] * 16)
    assert O.gemv(S.Q4_0, blk, 1, 32, np.zeros(4, np.float32))[0] == DIM
    assert O.gemv(S.Q4_0, np.concatenate([blk, blk]), 2, 32, np.zeros(32, np.float32), y_len=1)[0] == DIM
    assert O.dequant_block(S.Q4_0, np.zeros(4, np.uint8))[0] == BUF
    assert O.dequant_block(S.Q4_0, blk, out_len=1)[0] == BUF
    assert O.lib().qk_oracle_block_size(S.Q4_0) == 32 and O.lib().qk_oracle_block_bytes(S.Q4_0) == 18


def test_q4_0_fused_zero_and_accumulate():  # reference/q4_0.rs:381-420
    st, o = O.matvec_q8_fused(S.Q4_0, q4_0_block(1.0, [0x5A] * 16), q8_0_block(1.0, [0] * 32), [0.0], 1, 32)
    assert st == OK and o[0] == 0.0
    st, o = O.matvec_q8_fused(S.Q4_0, q4_0_block(1.0, [0x88] * 16), q8_0_block(1.0, [127] * 32), [0.0], 1, 32)
    assert st == OK and o[0] == 0.0
    st, o = O.matvec_q8_fused(S.Q4_0, q4_0_block(1.0, [0x88] * 16), q8_0_block(1.0, [0] * 32), [42.0], 1, 32)
    assert st == OK and o[0] == 42.0


def test_q4_0_fused_matches_unfused():  # reference/q4_0.rs:422-464
    nib = [0x5A, 0xF0, 0x13, 0x7E, 0xC2, 0x48, 0x9D, 0x6B, 0xA3, 0x2F, 0x71, 0xE4, 0x0C, 0x58, 0xB6, 0xD9]
    w = q4_0_block(0.25, nib)
    a = q8_0_block(0.5, Q8_VALS_A)
    x = np.array(Q8_VALS_A, np.float32) * 0.5
    _, yu = O.gemv(S.Q4_0, w, 1, 32, x)
    _, yf = O.matvec_q8_fused(S.Q4_0, w, a, [0.0], 1, 32)
    assert abs(yf[0] - yu[0]) < 1e-3
    # all operands are small dyadic rationals: both paths are exact
    ref = sum(((((b >> (4 * (i & 1))) & 15) - 8) * 0.25) * x[i] for i, b in
              ((i, nib[i // 2]) for i in range(32)))
    assert yu[0] == np.float32(ref) and yf[0] == np.float32(ref)


def test_q4_0_fused_multi_row():  # reference/q4_0.rs:466-537
    nib = [0x13, 0x57, 0x9B, 0xDF, 0x24, 0x68, 0xAC, 0xE0, 0x5F, 0x3A, 0x72, 0x8D, 0xC6, 0x4E, 0x91, 0xB7]
    q8 = [2, 4, -6, 8, -10, 12, -14, 16, 1, -3, 5, -7, 9, -11, 13, -15,
          0, 1, -2, 3, -4, 5, -6, 7, -8, 9, -10, 11, -12, 13, -14, 15]
    w = np.concatenate([q4_0_block(s, nib) for s in (0.1, 0.25, 0.5, 1.0) for _ in range(2)])
    a = np.concatenate([q8_0_block(0.125, q8)] * 2)
    x = np.array(q8 + q8, np.float32) * 0.125
    _, yu = O.gemv(S.Q4_0, w, 4, 64, x)
    _, yf = O.matvec_q8_fused(S.Q4_0, w, a, np.zeros(4), 4, 64)
    assert np.all(np.abs(yf - yu) < 1e-3)


# ------------------------------------------------------------------ Q8_0
def test_q8_0_dequant():  # reference/q8_0.rs:147-172
    st, out = O.dequant_block(S.Q8_0, q8_0_block(1.0, [0] * 32))
    assert st == OK and np.all(out == 0.0)
    v = [0] * 32
    v[0], v[1], v[31] = 10, -5, 127
    _, out = O.dequant_block(S.Q8_0, q8_0_block(0.5, v))
    assert out[0] == 5.0 and out[1] == -2.5 and out[31] == 63.5


def test_q8_0_gemv_gemm():  # reference/q8_0.rs:174-232
    v = [0] * 32
    v[0] = 1
    x = np.zeros(32, np.float32)
    x[0] = 3.0
    _, y = O.gemv(S.Q8_0, q8_0_block(2.0, v), 1, 32, x)
    assert y[0] == 6.0
    v[0] = 4
    _, y = O.gemm(S.Q8_0, q8_0_block(0.5, v), x, 1, 1, 32)
    assert y[0, 0] == 6.0
    z = q8_0_block(1.0, [0] * 32)
    _, y = O.gemm(S.Q8_0, np.concatenate([z, z]), np.ones(64, np.float32), 2, 2, 32)
    assert np.all(y == 0.0)
    assert O.gemv(S.Q8_0, z, 1, 32, np.zeros(4, np.float32))[0] == DIM


def test_q8_0_fused_default_matches_gemv():  # traits.rs:89-173
    w = S.gen_weight(S.Q8_0, 3, 96, seed=1)
    x = S.gen_acts(1, 96, seed=1)[0]
    _, a = O.quantize_q8_0(x)
    xa = np.concatenate([O.dequant_block(S.Q8_0, a[i * 34:(i + 1) * 34])[1] for i in range(3)])
    _, yu = O.gemv(S.Q8_0, w, 3, 96, xa)
    _, yf = O.matvec_q8_fused(S.Q8_0, w, a, np.full(3, 7.0), 3, 96)
    assert np.all(np.abs(yf - 7.0 - yu) < 1e-3)


# ------------------------------------------------------------------ Q4_K
SC1 = [1, 1, 1, 1, 0, 0, 0, 0, 1, 1, 1, 1]


def test_q4_k_dequant():  # reference/q4_k.rs:368-408
    st, out = O.dequant_block(S.Q4_K, q4_k_block(0.0, 0.0, [0] * 12, [0] * 128))
    assert st == OK and np.all(out == 0.0)
    _, out = O.dequant_block(S.Q4_K, q4_k_block(1.0, 0.0, SC1, [0x88] * 128))
    assert np.all(out == 8.0)


def test_q4_k_gemv():  # reference/q4_k.rs:410-436
    _, y = O.gemv(S.Q4_K, q4_k_block(1.0, 0.0, SC1, [0x11] * 128), 1, 256, np.ones(256, np.float32))
    assert y[0] == 256.0


def test_q4_k_fused_zero_and_accumulate():  # reference/q4_k.rs:450-493
    acts0 = np.concatenate([q8_0_block(1.0, [0] * 32)] * 8)
    _, o = O.matvec_q8_fused(S.Q4_K, q4_k_block(1.0, 0.0, SC1, [0x88] * 128), acts0, [0.0], 1, 256)
    assert o[0] == 0.0
    _, o = O.matvec_q8_fused(S.Q4_K, q4_k_block(0.0, 0.0, [0] * 12, [0] * 128), acts0, [42.0], 1, 256)
    assert o[0] == 42.0


def test_q4_k_fused_matches_unfused():  # reference/q4_k.rs:495-559
    sc = [5, 3, 7, 2, 4, 6, 1, 3, 9, 11, 13, 15]
    w = q4_k_block(0.5, 0.1, sc, [0xA5] * 128)
    a = np.concatenate([q8_0_block(0.25, Q8_VALS_A)] * 8)
    x = np.tile(np.array(Q8_VALS_A, np.float32) * 0.25, 8)
    _, yu = O.gemv(S.Q4_K, w, 1, 256, x)
    _, yf = O.matvec_q8_fused(S.Q4_K, w, a, [0.0], 1, 256)
    assert abs(yf[0] - yu[0]) < 1e-3
    # the six-bit fields this packing decodes to (reference/q4_k.rs:27-49)
    _, dq = O.dequant_block(S.Q4_K, w)
    d, dmin = np.float32(0.5), np.float32(np.float16(0.1))
    exp_sc = [5, 3, 7, 2, 9, 11, 13, 15]
    exp_mn = [4, 6, 1, 3, 0, 0, 0, 0]
    for s in range(8):
        q = np.float32(5.0 if s % 2 == 0 else 10.0)
        want = np.float32(np.float32(d * np.float32(exp_sc[s])) * q) - np.float32(dmin * np.float32(exp_mn[s]))
        assert np.all(dq[32 * s:32 * s + 32] == want), s


def test_q4_k_fused_multi_row():  # reference/q4_k.rs:561-625
    q8 = [2, -1, 4, -3, 6, -5, 8, -7, 1, -2, 3, -4, 5, -6, 7, -8,
          -2, 1, -4, 3, -6, 5, -8, 7, -1, 2, -3, 4, -5, 6, -7, 8]
    w = np.concatenate([q4_k_block(s, 0.0, SC1, [0x55] * 128) for s in (0.5, 1.0, 0.25, 0.1)])
    a = np.concatenate([q8_0_block(0.5, q8)] * 8)
    x = np.tile(np.array(q8, np.float32) * 0.5, 8)
    _, yu = O.gemv(S.Q4_K, w, 4, 256, x)
    _, yf = O.matvec_q8_fused(S.Q4_K, w, a, np.zeros(4), 4, 256)
    assert np.all(np.abs(yf - yu) < 1e-3)


# ------------------------------------------------------------------ Q6_K
def test_q6_k_dequant_zero():  # reference/q6_k.rs:368-414
    _, out = O.dequant_block(S.Q6_K, np.zeros(210, np.uint8))
    assert np.all(out == 0.0)
    b = np.zeros(210, np.uint8)
    b[128:192] = 0xAA
    b[192:208] = 1
    b[208:210] = f16b(1.0)
    _, out = O.dequant_block(S.Q6_K, b)
    assert np.all(out == 0.0)


def _q6_k_pattern_block():
    b = np.zeros(210, np.uint8)
    b[0:128] = [(i * 7 + 3) & 0xFF for i in range(128)]
    b[128:192] = [(i * 13 + 5) & 0xFF for i in range(64)]
    b[192:208] = np.array([i * 3 - 8 for i in range(16)], np.int8).view(np.uint8)
    b[208:210] = f16b(0.5)
    return b


def test_q6_k_gemv_matches_dequant_dot():  # reference/q6_k.rs:416-460
    b = _q6_k_pattern_block()
    _, dq = O.dequant_block(S.Q6_K, b)
    x = (np.arange(256, dtype=np.float32) * np.float32(0.01)) - np.float32(1.28)
    expected = np.float32(0)
    for w, v in zip(dq, x):
        expected = np.float32(expected + np.float32(w * v))
    _, y = O.gemv(S.Q6_K, b, 1, 256, x)
    assert abs(y[0] - expected) < 0.1


def test_q6_k_fused_matches_unfused():  # reference/q6_k.rs:212-354 vs :77-172
    w = S.gen_weight(S.Q6_K, 2, 512, seed=3)
    x = S.gen_acts(1, 512, seed=3)[0]
    _, a = O.quantize_q8_0(x)
    xa = np.concatenate([O.dequant_block(S.Q8_0, a[i * 34:(i + 1) * 34])[1] for i in range(16)])
    _, yu = O.gemv(S.Q6_K, w, 2, 512, xa)
    _, yf = O.matvec_q8_fused(S.Q6_K, w, a, np.zeros(2), 2, 512)
    assert np.all(np.abs(yf - yu) < 1e-3)


# ------------------------------------------------------------------ IQ4_XS
def test_iq4_xs_dequant():  # reference/iq4_xs.rs:251-285
    _, out = O.dequant_block(S.IQ4_XS, iq4_xs_block(1.0, [32] * 8, [0xAA] * 128))
    assert np.all(out == 0.0)
    ss = [32] * 8
    ss[0] = 33
    _, out = O.dequant_block(S.IQ4_XS, iq4_xs_block(1.0, ss, [0x88] * 128))
    assert np.all(out[:32] == 1.0) and np.all(out[32:] == 0.0)


def test_iq4_xs_errors_and_meta():  # reference/iq4_xs.rs:287-301,356-361
    assert O.dequant_block(S.IQ4_XS, np.zeros(50, np.uint8))[0] == BUF
    assert O.dequant_block(S.IQ4_XS, iq4_xs_block(1.0, [32] * 8, [0] * 128), out_len=100)[0] == BUF
    assert O.lib().qk_oracle_block_size(S.IQ4_XS) == 256 and O.lib().qk_oracle_block_bytes(S.IQ4_XS) == 136


def test_iq4_xs_gemv():  # reference/iq4_xs.rs:303-354
    b1 = iq4_xs_block(1.0, [33] * 8, [0x88] * 128)
    _, y = O.gemv(S.IQ4_XS, b1, 1, 256, np.ones(256, np.float32))
    assert y[0] == 256.0
    b0 = iq4_xs_block(1.0, [32] * 8, [0x88] * 128)
    _, y = O.gemv(S.IQ4_XS, np.concatenate([b0, b1]), 2, 256, np.ones(256, np.float32))
    assert y[0] == 0.0 and y[1] == 256.0


def test_iq4_xs_sub_scale_roundtrip():  # reference/iq4_xs.rs:363-380
    ss = [32, 0, 63, 1, 31, 33, 16, 48]
    # nibble 8 -> table value 1, d = 1: the weight equals the signed sub-scale
    _, out = O.dequant_block(S.IQ4_XS, iq4_xs_block(1.0, ss, [0x88] * 128))
    for i, v in enumerate(ss):
        assert np.all(out[32 * i:32 * i + 32] == float(v - 32))


def test_iq4_xs_table_and_interleave():  # reference/iq_shared.rs:16-18, iq4_xs.rs:87-93
    K = [-127, -104, -83, -65, -49, -35, -22, -10, 1, 13, 25, 38, 53, 69, 89, 113]
    nib = [(i % 16) | (((15 - i) % 16) << 4) for i in range(128)]
    _, out = O.dequant_block(S.IQ4_XS, iq4_xs_block(1.0, [33] * 8, nib))
    for i in range(128):
        assert out[2 * i] == K[i % 16] and out[2 * i + 1] == K[(15 - i) % 16]


# ------------------------------------------------------------------ unsupported / shapes
def test_unsupported_type():
    assert O.dequant_block(3, np.zeros(64, np.uint8), out_len=32)[0] == UNSUPPORTED
    assert O.gemv(16, np.zeros(84, np.uint8), 1, 256, np.zeros(256, np.float32))[0] == UNSUPPORTED   # IQ2_XXS


@pytest.mark.parametrize("qtype", S.ALL_TYPES)
def test_partial_last_block_guards_columns(qtype):
    """Columns past n_cols inside the last block contribute nothing (e.g. q4_k.rs:161,168)."""
    bs = S.BLOCK_SIZE[qtype]
    n_cols = bs + bs // 2 + 3
    w = S.gen_weight(qtype, 3, n_cols, seed=5)
    x = S.gen_acts(1, 2 * bs, seed=5)[0]
    _, y = O.gemv(qtype, w, 3, n_cols, x)
    dq = O.dequant_matrix(qtype, w, 3, n_cols)
    want = (dq.astype(np.float64) @ x[:n_cols].astype(np.float64))
    assert np.allclose(y, want, rtol=1e-4, atol=1e-5)


# ------------------------------------------------------------------ f16 and the Q8_0 encoder
def test_f16_to_f32_exhaustive():
    bits = np.arange(65536, dtype=np.uint16)
    want = bits.view(np.float16).astype(np.float32)
    got = np.array([O.lib().qk_oracle_f16_to_f32(int(b)) for b in bits], np.float32)
    nan = np.isnan(want)
    assert np.array_equal(got[~nan].view(np.uint32), want[~nan].view(np.uint32))
    assert np.all(np.isnan(got[nan]))


def test_f32_to_f16_matches_ieee_rne():
    rng = np.random.default_rng(0)
    xs = np.concatenate([
        rng.standard_normal(20000).astype(np.float32),
        (rng.standard_normal(5000) * 1e-6).astype(np.float32),  # f16 subnormal range
        (rng.standard_normal(2000) * 7e4).astype(np.float32),   # overflow to inf
        np.array([0.0, -0.0, 65504.0, 65520.0, 65519.99, 5.9604645e-8, 2.9802322e-8, 2.98023224e-8 * 1.0001,
                  1.0 + 2 ** -11, 1.0 + 3 * 2 ** -11, 0.1, 0.01, np.inf, -np.inf], np.float32),
    ])
    with np.errstate(over="ignore"):
        want = xs.astype(np.float16).view(np.uint16)
    got = np.array([O.f16_bits(float(x)) for x in xs], np.uint16)
    assert np.array_equal(got, want)


def _np_quantize_q8_0(x):
    x = x.reshape(-1, 32).astype(np.float32)
    amax = np.abs(x).max(axis=1)
    d = (amax / np.float32(127.0)).astype(np.float32)
    with np.errstate(divide="ignore"):
        idv = np.where(d != 0, np.float32(1.0) / d, np.float32(0)).astype(np.float32)
    v = (x * idv[:, None]).astype(np.float32)
    q = np.clip(np.where(v >= 0, np.floor(v + np.float32(0.5)), np.ceil(v - np.float32(0.5))), -128, 127).astype(np.int8)
    out = np.empty((x.shape[0], 34), np.uint8)
    out[:, :2] = d.astype(np.float16).view(np.uint8).reshape(-1, 2)
    out[:, 2:] = q.view(np.uint8)
    return out.reshape(-1)


def test_quantize_q8_0():  # quantize.rs:58-75,190-210
    x = S.gen_acts(1, 4096, seed=2)[0]
    x[:32] = 0.0  # d == 0 branch
    x[32:64] = np.linspace(-1, 1, 32, dtype=np.float32) * 127 / 127  # ties at .5 multiples
    st, got = O.quantize_q8_0(x)
    assert st == OK and np.array_equal(got, _np_quantize_q8_0(x))
    assert O.quantize_q8_0(np.zeros(33, np.float32))[0] == DIM
    # the largest element always maps to +-127 and the scale is amax/127 in f16
    blk = got[34 * 5: 34 * 6]
    assert np.abs(blk[2:].view(np.int8)).max() == 127


# ------------------------------------------------------------------ second opinions
def _np_dequant(qtype, b):
    K = np.array([-127, -104, -83, -65, -49, -35, -22, -10, 1, 13, 25, 38, 53, 69, 89, 113], np.float32)
    f = np.float32
    if qtype == S.Q4_0:
        d = b[:2].view(np.float16).astype(f)[0]
        q = b[2:18]
        out = np.empty(32, f)
        out[0::2] = ((q & 15).astype(np.int32) - 8).astype(f) * d
        out[1::2] = ((q >> 4).astype(np.int32) - 8).astype(f) * d
        return out
    if qtype == S.Q8_0:
        return b[2:34].view(np.int8).astype(f) * b[:2].view(np.float16).astype(f)[0]
    if qtype == S.Q4_K:
        d, dmin = b[:4].view(np.float16).astype(f)
        s = b[4:16].astype(np.int32)
        qs = b[16:144]
        sc = [s[j] & 63 for j in range(4)] + [(s[j + 4] & 15) | ((s[j - 4] >> 6) << 4) for j in range(4, 8)]
        mn = [s[j + 4] & 63 for j in range(4)] + [(s[j + 4] >> 4) | ((s[j] >> 6) << 4) for j in range(4, 8)]
        out = np.empty(256, f)
        for g in range(4):
            q = qs[32 * g:32 * g + 32]
            out[64 * g:64 * g + 32] = f(d * f(sc[2 * g])) * (q & 15).astype(f) - f(dmin * f(mn[2 * g]))
            out[64 * g + 32:64 * g + 64] = f(d * f(sc[2 * g + 1])) * (q >> 4).astype(f) - f(dmin * f(mn[2 * g + 1]))
        return out
    if qtype == S.Q6_K:
        ql, qh, sc = b[:128].astype(np.int32), b[128:192].astype(np.int32), b[192:208].view(np.int8)
        d = b[208:210].view(np.float16).astype(f)[0]
        out = np.empty(256, f)
        for g in range(2):
            for l in range(32):
                L, L2, H = ql[64 * g + l], ql[64 * g + l + 32], qh[32 * g + l]
                q = [(L & 15) | ((H & 3) << 4), (L2 & 15) | (((H >> 2) & 3) << 4),
                     (L >> 4) | (((H >> 4) & 3) << 4), (L2 >> 4) | (((H >> 6) & 3) << 4)]
                for k in range(4):
                    out[128 * g + l + 32 * k] = f(f(d * f(sc[8 * g + l // 16 + 2 * k])) * f(q[k] - 32))
        return out
    d = b[:2].view(np.float16).astype(f)[0]
    sh = int(b[2]) | (int(b[3]) << 8)
    out = np.empty(256, f)
    for s in range(8):
        ls = ((int(b[4 + s // 2]) >> (4 * (s & 1))) & 15) | (((sh >> (2 * s)) & 3) << 4)
        scale = f(d * f(ls - 32))
        q = b[8 + 16 * s:8 + 16 * s + 16]
        out[32 * s:32 * s + 32:2] = scale * K[q & 15]
        out[32 * s + 1:32 * s + 32:2] = scale * K[q >> 4]
    return out


@pytest.mark.parametrize("qtype", S.ALL_TYPES)
def test_dequant_bit_exact_vs_numpy_restatement(qtype):
    bb = S.BLOCK_BYTES[qtype]
    blocks = S.gen_blocks(qtype, 64, seed=11).reshape(64, bb).copy()
    # include f16 subnormal, zero and negative scales
    off = 208 if qtype == S.Q6_K else 0
    blocks[0, off:off + 2] = [0x01, 0x00]
    blocks[1, off:off + 2] = [0xFF, 0x03]
    blocks[2, off:off + 2] = [0x00, 0x80]
    blocks[3, off:off + 2] = [0x00, 0xBC]
    for b in blocks:
        st, got = O.dequant_block(qtype, b)
        assert st == OK
        assert np.array_equal(got.view(np.uint32), _np_dequant(qtype, b).view(np.uint32))


def test_q2_k_against_gguf_py():
    """Q2_K is canonical GGUF in the reference: bit-identical to gguf-py."""
    gguf = pytest.importorskip("gguf")
    from gguf import quants
    for b in S.gen_blocks(S.Q2_K, 40, seed=12).reshape(40, 84):
        _, got = O.dequant_block(S.Q2_K, b)
        g = quants.dequantize(b[None, :].copy(), gguf.GGMLQuantizationType.Q2_K).reshape(-1).astype(np.float32)
        assert np.array_equal(got.view(np.uint32), g.view(np.uint32))


def test_q3_k_against_gguf_py_up_to_the_scale_packing():
    """The reference packs Q3_K's sixteen 6-bit scales differently from llama.cpp (reference/
    q3_k.rs:29-59: bytes 0-7 hold scales 0-7 in their low six bits; llama.cpp keeps the low
    four bits of scales 0-7 / 8-15 in the nibbles of bytes 0-7 and all high bit pairs in bytes
    8-11), so a block means different weights to the two.  Everything else (mask bits, 2-bit
    quants, element order, arithmetic) is the same: the same sixteen scale values packed each
    way give bit-identical weights."""
    gguf = pytest.importorskip("gguf")
    from gguf import quants
    rng = np.random.default_rng(3)
    for _ in range(20):
        raw = rng.integers(0, 64, 16)
        ref = np.zeros(12, np.uint8)
        cpp = np.zeros(12, np.uint8)
        for j in range(4):
            ref[j] = (raw[j] & 0x3F) | ((raw[8 + j] >> 4) << 6)
            ref[4 + j] = (raw[4 + j] & 0x3F) | ((raw[12 + j] >> 4) << 6)
            ref[8 + j] = (raw[8 + j] & 0x0F) | ((raw[12 + j] & 0x0F) << 4)
            cpp[j] = (raw[j] & 0x0F) | ((raw[8 + j] & 0x0F) << 4)
            cpp[4 + j] = (raw[4 + j] & 0x0F) | ((raw[12 + j] & 0x0F) << 4)
            cpp[8 + j] = (raw[j] >> 4) | ((raw[4 + j] >> 4) << 2) | ((raw[8 + j] >> 4) << 4) | ((raw[12 + j] >> 4) << 6)
        hmask, qs = rng.integers(0, 256, 32, dtype=np.uint8), rng.integers(0, 256, 64, dtype=np.uint8)
        d = f16b(float(rng.uniform(1e-3, 2e-2)))
        _, got = O.dequant_block(S.Q3_K, np.concatenate([hmask, qs, ref, d]))
        g = quants.dequantize(np.concatenate([hmask, qs, cpp, d])[None, :].copy(),
                              gguf.GGMLQuantizationType.Q3_K).reshape(-1).astype(np.float32)
        assert np.array_equal(got.view(np.uint32), g.view(np.uint32))


@pytest.mark.parametrize("qtype,gname", [(S.Q8_0, "Q8_0"), (S.Q4_K, "Q4_K"), (S.Q6_K, "Q6_K"),
                                         (S.Q4_0, "Q4_0"), (S.IQ4_XS, "IQ4_XS")])
def test_against_gguf_py(qtype, gname):
    """Q8_0 / Q4_K / Q6_K are canonical GGUF: bit-identical to gguf-py.  Q4_0 and
    IQ4_XS hold the same values in the reference's interleaved order
    (reference/q4_0.rs:40-46, iq4_xs.rs:87-93): equal after that permutation."""
    gguf = pytest.importorskip("gguf")
    from gguf import quants
    t = getattr(gguf.GGMLQuantizationType, gname)
    bb = S.BLOCK_BYTES[qtype]
    blocks = S.gen_blocks(qtype, 40, seed=12).reshape(40, bb)
    for b in blocks:
        _, got = O.dequant_block(qtype, b)
        g = quants.dequantize(b[None, :].copy(), t).reshape(-1).astype(np.float32)
        if qtype in (S.Q8_0, S.Q4_K, S.Q6_K):
            assert np.array_equal(got.view(np.uint32), g.view(np.uint32))
        else:
            # canonical: element i <- low nibble of byte i, element i+16 <- high nibble (per 32)
            perm = got.reshape(-1, 16, 2)
            canon = np.concatenate([perm[:, :, 0], perm[:, :, 1]], axis=1).reshape(-1)
            assert np.array_equal(canon.view(np.uint32), g.view(np.uint32))
            assert not np.array_equal(got, g)


# ------------------------------------------------------------------ MoE routing (moe.rs:200-248)
def test_moe_route_properties():
    logits = S.gen_acts(64, 8, seed=4)
    ids, wts = O.moe_route(logits, 2)
    assert np.allclose(wts.sum(axis=1), 1.0, atol=1e-6)
    top2 = np.argsort(-logits, axis=1, kind="stable")[:, :2]
    assert np.array_equal(ids, top2)
    p = np.exp(logits - logits.max(1, keepdims=True))
    p /= p.sum(1, keepdims=True)
    want = np.take_along_axis(p, top2, 1)
    want /= want.sum(1, keepdims=True)
    assert np.allclose(wts, want, rtol=1e-5)
    ids3, _ = O.moe_route(logits[:, :2], 2)  # top_k clamps to n_exp
    assert ids3.shape == (64, 2)


def test_moe_ffn_small_matches_float64():
    n_exp, hidden, inter, tokens = 4, 256, 512, 6
    qt = S.Q4_K
    gate = np.stack([O.dequant_matrix(qt, S.gen_weight(qt, inter, hidden, 9, e), inter, hidden) for e in range(n_exp)])
    up = np.stack([O.dequant_matrix(qt, S.gen_weight(qt, inter, hidden, 9, 10 + e), inter, hidden) for e in range(n_exp)])
    down = np.stack([O.dequant_matrix(qt, S.gen_weight(qt, hidden, inter, 9, 20 + e), hidden, inter) for e in range(n_exp)])
    x = S.gen_acts(tokens, hidden, seed=9)
    logits = S.gen_acts(tokens, n_exp, seed=9, stream=77)
    y = O.moe_ffn_f32(gate, up, down, logits, x, 2)
    ids, wts = O.moe_route(logits, 2)
    want = np.zeros((tokens, hidden))
    for t in range(tokens):
        for k in range(2):
            e = ids[t, k]
            g = gate[e].astype(np.float64) @ x[t]
            u = up[e].astype(np.float64) @ x[t]
            h = g / (1 + np.exp(-g)) * u
            want[t] += wts[t, k] * (down[e].astype(np.float64) @ h)
    assert np.allclose(y, want, rtol=2e-4, atol=2e-4 * np.abs(want).max())
