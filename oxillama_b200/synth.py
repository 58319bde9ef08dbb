"""Seeded synthetic GGUF-layout blocks and activations for the benchmark configurations.

The reference measures this path on no public suite; these draws *are* the
workload.  Every field is drawn so that the block is a legal block of its
format (finite f16 scales, 6-bit scale fields, int8 quants), using numpy's
counter-based Philox generator keyed by (seed, stream) so that any tensor can
be regenerated independently and identically on any machine.

Block layouts (bytes) follow crates/oxillama-gguf/src/types.rs:199-259 of the
reference: Q4_0 18, Q8_0 34, Q4_K 144, Q6_K 210, IQ4_XS 136.
"""
from __future__ import annotations

import numpy as np

Q4_0, Q8_0, Q4_K, Q6_K, IQ4_XS = 2, 8, 12, 14, 23
Q5_K, Q2_K, Q3_K, Q8_K = 13, 10, 11, 15  # served by the generic kernels; not among the benchmark's formats
BLOCK_SIZE = {Q4_0: 32, Q8_0: 32, Q4_K: 256, Q6_K: 256, IQ4_XS: 256, Q5_K: 256, Q2_K: 256, Q3_K: 256, Q8_K: 256}
BLOCK_BYTES = {Q4_0: 18, Q8_0: 34, Q4_K: 144, Q6_K: 210, IQ4_XS: 136, Q5_K: 176, Q2_K: 84, Q3_K: 110, Q8_K: 292}
NAMES = {Q4_0: "Q4_0", Q8_0: "Q8_0", Q4_K: "Q4_K", Q6_K: "Q6_K", IQ4_XS: "IQ4_XS", Q5_K: "Q5_K", Q2_K: "Q2_K", Q3_K: "Q3_K",
         Q8_K: "Q8_K"}
NEXT_TYPES = (Q5_K, Q2_K, Q3_K, Q8_K)
ALL_TYPES = (Q4_0, Q8_0, Q4_K, Q6_K, IQ4_XS)


def rng_for(seed: int, stream: int) -> np.random.Generator:
    return np.random.Generator(np.random.Philox(key=[seed & 0xFFFFFFFFFFFFFFFF, stream]))


def blocks_per_row(qtype: int, n_cols: int) -> int:
    bs = BLOCK_SIZE[qtype]
    return (n_cols + bs - 1) // bs


def weight_nbytes(qtype: int, n_rows: int, n_cols: int) -> int:
    return n_rows * blocks_per_row(qtype, n_cols) * BLOCK_BYTES[qtype]


def _f16_bytes(rng, lo, hi, n):
    return rng.uniform(lo, hi, n).astype(np.float16).view(np.uint8).reshape(n, 2)


def gen_blocks(qtype: int, n_blocks: int, seed: int = 0, stream: int = 0,
               d_range=(1e-3, 2e-2)) -> np.ndarray:
    """`n_blocks` random blocks of `qtype` as a flat uint8 array."""
    rng = rng_for(seed, stream)
    bb = BLOCK_BYTES[qtype]
    out = np.empty((n_blocks, bb), np.uint8)
    if qtype == Q4_0:
        out[:, 0:2] = _f16_bytes(rng, *d_range, n_blocks)
        out[:, 2:] = rng.integers(0, 256, (n_blocks, 16), dtype=np.uint8)
    elif qtype == Q8_0:
        out[:, 0:2] = _f16_bytes(rng, *d_range, n_blocks)
        out[:, 2:] = rng.integers(-127, 128, (n_blocks, 32), dtype=np.int8).view(np.uint8)
    elif qtype == Q4_K:
        out[:, 0:2] = _f16_bytes(rng, *d_range, n_blocks)
        out[:, 2:4] = _f16_bytes(rng, *d_range, n_blocks)
        # any 12 bytes are a bijective packing of sixteen uniform 6-bit fields
        out[:, 4:] = rng.integers(0, 256, (n_blocks, 140), dtype=np.uint8)
    elif qtype == Q5_K:
        out[:, 0:2] = _f16_bytes(rng, *d_range, n_blocks)
        out[:, 2:4] = _f16_bytes(rng, *d_range, n_blocks)
        out[:, 4:] = rng.integers(0, 256, (n_blocks, 172), dtype=np.uint8)
    elif qtype == Q2_K:
        out[:, 0:80] = rng.integers(0, 256, (n_blocks, 80), dtype=np.uint8)
        out[:, 80:82] = _f16_bytes(rng, *d_range, n_blocks)
        out[:, 82:84] = _f16_bytes(rng, *d_range, n_blocks)
    elif qtype == Q3_K:
        out[:, 0:108] = rng.integers(0, 256, (n_blocks, 108), dtype=np.uint8)
        out[:, 108:110] = _f16_bytes(rng, *d_range, n_blocks)
    elif qtype == Q8_K:
        lo, hi = d_range
        out[:, 0:4] = rng.uniform(lo, hi, n_blocks).astype(np.float32).view(np.uint8).reshape(n_blocks, 4)
        q = rng.integers(-128, 128, (n_blocks, 256), dtype=np.int8)
        out[:, 4:260] = q.view(np.uint8)
        # sixteen i16 sums of 16 quants each (llama.cpp's bsums; the reference never reads them)
        out[:, 260:292] = q.reshape(n_blocks, 16, 16).sum(axis=2).astype('<i2').view(np.uint8).reshape(n_blocks, 32)
    elif qtype == Q6_K:
        out[:, 0:192] = rng.integers(0, 256, (n_blocks, 192), dtype=np.uint8)
        out[:, 192:208] = rng.integers(-32, 32, (n_blocks, 16), dtype=np.int8).view(np.uint8)
        lo, hi = d_range
        out[:, 208:210] = _f16_bytes(rng, lo, min(hi, 1e-2), n_blocks)
    elif qtype == IQ4_XS:
        out[:, 0:2] = _f16_bytes(rng, *d_range, n_blocks)
        out[:, 2:] = rng.integers(0, 256, (n_blocks, 134), dtype=np.uint8)
    else:
        raise ValueError(f"unsupported type {qtype}")
    return out.reshape(-1)


def gen_weight(qtype: int, n_rows: int, n_cols: int, seed: int = 0, stream: int = 0,
               d_range=(1e-3, 2e-2)) -> np.ndarray:
    """A [n_rows x n_cols] weight matrix: rows of ceil(n_cols/block) blocks."""
    return gen_blocks(qtype, n_rows * blocks_per_row(qtype, n_cols), seed, stream, d_range)


def gen_acts(m: int, k: int, seed: int = 0, stream: int = 1000) -> np.ndarray:
    """[m x k] f32 activations ~ N(0,1)."""
    return rng_for(seed, stream).standard_normal((m, k), dtype=np.float32)
