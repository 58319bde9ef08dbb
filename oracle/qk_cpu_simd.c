/*
 * CPU baseline for the timing report.  TEST / BENCH INFRASTRUCTURE ONLY — never
 * part of the product path.
 *
 * Restates, in C intrinsics, the reference's fastest CPU tiers for the decode
 * matvec so that they can be timed on the GPU box's host cores beside the CUDA
 * kernels (the reference is Rust and cannot be built where this runs):
 *   tier 0  scalar        crates/oxillama-quant/src/reference/ (the oracle rows)
 *   tier 1  AVX2 + FMA    crates/oxillama-quant/src/simd/avx2/{q4_0,q8_0,q4_k,q6_k,iq4_xs}.rs  gemv_row_avx2
 *   tier 2  AVX-512F      crates/oxillama-quant/src/simd/avx512/{...}.rs                        gemv_row_avx512
 * wrapped in a row-parallel driver that mirrors parallel_gemv
 * (crates/oxillama-quant/src/parallel.rs:33-92; rayon's pool there, a pthread pool here).
 * The reference's own call chain is single-threaded (threads = 1); the
 * all-cores figure is what parallel_gemv would give it.
 *
 * The tiers round differently from one another and from the scalar kernels (lane-wise
 * sums, FMAs, where the scale is applied): they are held to the scalar oracle at the
 * reference's own 1e-3 (tests/test_cpu_simd.py), not bit for bit.
 */
#include <immintrin.h>
#include <pthread.h>
#include <unistd.h>

#include "qk_oracle.c"

static float hsum256(__m256 v) {
  __m128 lo = _mm256_castps256_ps128(v), hi = _mm256_extractf128_ps(v, 1);
  __m128 s = _mm_add_ps(lo, hi);
  s = _mm_add_ps(s, _mm_movehl_ps(s, s));
  s = _mm_add_ss(s, _mm_shuffle_ps(s, s, 1));
  return _mm_cvtss_f32(s);
}

/* One Q4_K row, 8 lanes: per 64-weight group the two sub-block scales and mins
 * are broadcast, nibbles widened u8 -> i32 -> f32, w = fmsub(a, q, b), and the
 * block accumulator takes fmadd(w, x); one horizontal sum per super-block. */
__attribute__((target("avx2,fma"))) static float row_q4_k_avx2(const uint8_t *row, size_t bpr,
                                                               size_t n_cols, const float *x) {
  float row_sum = 0.0f;
  const __m128i m4 = _mm_set1_epi8(0x0F);
  for (size_t blk = 0; blk < bpr; blk++) {
    const uint8_t *b = row + blk * 144;
    size_t io = blk * 256;
    size_t remaining = n_cols > io ? n_cols - io : 0;
    if (remaining >= 256) {
      float d = rd_f16(b), dmin = rd_f16(b + 2);
      uint8_t sc[8], mn[8];
      decode_scales_mins(b + 4, sc, mn);
      const uint8_t *qs = b + 16;
      __m256 acc = _mm256_setzero_ps();
      for (int g = 0; g < 4; g++) {
        __m256 va_lo = _mm256_set1_ps(d * (float)sc[2 * g]), vb_lo = _mm256_set1_ps(dmin * (float)mn[2 * g]);
        __m256 va_hi = _mm256_set1_ps(d * (float)sc[2 * g + 1]),
               vb_hi = _mm256_set1_ps(dmin * (float)mn[2 * g + 1]);
        __m128i r0 = _mm_loadu_si128((const __m128i *)(qs + 32 * g));
        __m128i r1 = _mm_loadu_si128((const __m128i *)(qs + 32 * g + 16));
        __m128i part[4] = {_mm_and_si128(r0, m4), _mm_and_si128(r1, m4),
                           _mm_and_si128(_mm_srli_epi16(r0, 4), m4),
                           _mm_and_si128(_mm_srli_epi16(r1, 4), m4)};
        const float *xp = x + io + 64 * g;
        for (int p = 0; p < 4; p++) {
          __m256 va = p < 2 ? va_lo : va_hi, vb = p < 2 ? vb_lo : vb_hi;
          const float *xq = xp + 16 * p; /* parts 0,1 -> columns 0..31; parts 2,3 -> 32..63 */
          __m256 q0 = _mm256_cvtepi32_ps(_mm256_cvtepu8_epi32(part[p]));
          __m256 q1 = _mm256_cvtepi32_ps(_mm256_cvtepu8_epi32(_mm_srli_si128(part[p], 8)));
          acc = _mm256_fmadd_ps(_mm256_fmsub_ps(va, q0, vb), _mm256_loadu_ps(xq), acc);
          acc = _mm256_fmadd_ps(_mm256_fmsub_ps(va, q1, vb), _mm256_loadu_ps(xq + 8), acc);
        }
      }
      row_sum += hsum256(acc);
    } else if (remaining > 0) {
      row_sum += row_q4_k_f32(b, 1, remaining, x + io); /* scalar tail, as the reference */
    }
  }
  return row_sum;
}

__attribute__((target("avx512f,avx2,fma"))) static float row_q4_k_avx512(const uint8_t *row, size_t bpr,
                                                                       size_t n_cols, const float *x) {
  float row_sum = 0.0f;
  const __m128i m4 = _mm_set1_epi8(0x0F);
  for (size_t blk = 0; blk < bpr; blk++) {
    const uint8_t *b = row + blk * 144;
    size_t io = blk * 256;
    size_t remaining = n_cols > io ? n_cols - io : 0;
    if (remaining >= 256) {
      float d = rd_f16(b), dmin = rd_f16(b + 2);
      uint8_t sc[8], mn[8];
      decode_scales_mins(b + 4, sc, mn);
      const uint8_t *qs = b + 16;
      __m512 acc = _mm512_setzero_ps();
      for (int g = 0; g < 4; g++) {
        __m512 va_lo = _mm512_set1_ps(d * (float)sc[2 * g]), vb_lo = _mm512_set1_ps(dmin * (float)mn[2 * g]);
        __m512 va_hi = _mm512_set1_ps(d * (float)sc[2 * g + 1]),
               vb_hi = _mm512_set1_ps(dmin * (float)mn[2 * g + 1]);
        __m128i r0 = _mm_loadu_si128((const __m128i *)(qs + 32 * g));
        __m128i r1 = _mm_loadu_si128((const __m128i *)(qs + 32 * g + 16));
        const float *xp = x + io + 64 * g;
        __m512 q;
        q = _mm512_cvtepi32_ps(_mm512_cvtepu8_epi32(_mm_and_si128(r0, m4)));
        acc = _mm512_fmadd_ps(_mm512_fmsub_ps(va_lo, q, vb_lo), _mm512_loadu_ps(xp), acc);
        q = _mm512_cvtepi32_ps(_mm512_cvtepu8_epi32(_mm_and_si128(r1, m4)));
        acc = _mm512_fmadd_ps(_mm512_fmsub_ps(va_lo, q, vb_lo), _mm512_loadu_ps(xp + 16), acc);
        q = _mm512_cvtepi32_ps(_mm512_cvtepu8_epi32(_mm_and_si128(_mm_srli_epi16(r0, 4), m4)));
        acc = _mm512_fmadd_ps(_mm512_fmsub_ps(va_hi, q, vb_hi), _mm512_loadu_ps(xp + 32), acc);
        q = _mm512_cvtepi32_ps(_mm512_cvtepu8_epi32(_mm_and_si128(_mm_srli_epi16(r1, 4), m4)));
        acc = _mm512_fmadd_ps(_mm512_fmsub_ps(va_hi, q, vb_hi), _mm512_loadu_ps(xp + 48), acc);
      }
      row_sum += _mm512_reduce_add_ps(acc);
    } else if (remaining > 0) {
      row_sum += row_q4_k_f32(b, 1, remaining, x + io);
    }
  }
  return row_sum;
}


static float hsum512(__m512 v) { return _mm512_reduce_add_ps(v); }

/* ---- Q4_0: simd/avx2/q4_0.rs:386-470, simd/avx512/q4_0.rs:205-283.  Nibbles are
 * re-interleaved (unpacklo/hi of the low and high nibbles) into element order, 8 is
 * subtracted as integers, the block's products are summed in lanes (first group a plain
 * multiply, the rest FMAs), one horizontal sum per block, times d. */
static float q4_0_tail(const uint8_t *b, size_t io, size_t n_cols, const float *x) {
  float partial = 0.0f;
  for (size_t i = 0; i < 16; i++) {
    int lo = (int)(b[2 + i] & 0x0F) - 8, hi = (int)((b[2 + i] >> 4) & 0x0F) - 8;
    size_t idx = io + i * 2;
    if (idx + 1 < n_cols) {
      partial += (float)lo * x[idx];
      partial += (float)hi * x[idx + 1];
    } else if (idx < n_cols) {
      partial += (float)lo * x[idx];
    }
  }
  return partial;
}

__attribute__((target("avx2,fma"))) static float row_q4_0_avx2(const uint8_t *row, size_t bpr, size_t n_cols,
                                                               const float *x) {
  float row_sum = 0.0f;
  const __m256i eight = _mm256_set1_epi32(8);
  const __m128i m4 = _mm_set1_epi8(0x0F);
  for (size_t blk = 0; blk < bpr; blk++) {
    const uint8_t *b = row + blk * 18;
    size_t io = blk * 32, remaining = n_cols > io ? n_cols - io : 0;
    float d = rd_f16(b);
    __m128i raw = _mm_loadu_si128((const __m128i *)(b + 2));
    __m128i lo = _mm_and_si128(raw, m4), hi = _mm_and_si128(_mm_srli_epi16(raw, 4), m4);
    __m128i first16 = _mm_unpacklo_epi8(lo, hi), last16 = _mm_unpackhi_epi8(lo, hi);
    if (remaining >= 32) {
      const float *xp = x + io;
      __m256 acc = _mm256_mul_ps(_mm256_cvtepi32_ps(_mm256_sub_epi32(_mm256_cvtepu8_epi32(first16), eight)),
                                 _mm256_loadu_ps(xp));
      acc = _mm256_fmadd_ps(
          _mm256_cvtepi32_ps(_mm256_sub_epi32(_mm256_cvtepu8_epi32(_mm_srli_si128(first16, 8)), eight)),
          _mm256_loadu_ps(xp + 8), acc);
      acc = _mm256_fmadd_ps(_mm256_cvtepi32_ps(_mm256_sub_epi32(_mm256_cvtepu8_epi32(last16), eight)),
                            _mm256_loadu_ps(xp + 16), acc);
      acc = _mm256_fmadd_ps(
          _mm256_cvtepi32_ps(_mm256_sub_epi32(_mm256_cvtepu8_epi32(_mm_srli_si128(last16, 8)), eight)),
          _mm256_loadu_ps(xp + 24), acc);
      row_sum += hsum256(acc) * d;
    } else if (remaining > 0) {
      row_sum += q4_0_tail(b, io, n_cols, x) * d;
    }
  }
  return row_sum;
}

__attribute__((target("avx512f,avx2,fma"))) static float row_q4_0_avx512(const uint8_t *row, size_t bpr,
                                                                       size_t n_cols, const float *x) {
  float row_sum = 0.0f;
  const __m512i eight = _mm512_set1_epi32(8);
  const __m128i m4 = _mm_set1_epi8(0x0F);
  for (size_t blk = 0; blk < bpr; blk++) {
    const uint8_t *b = row + blk * 18;
    size_t io = blk * 32, remaining = n_cols > io ? n_cols - io : 0;
    float d = rd_f16(b);
    __m128i raw = _mm_loadu_si128((const __m128i *)(b + 2));
    __m128i lo = _mm_and_si128(raw, m4), hi = _mm_and_si128(_mm_srli_epi16(raw, 4), m4);
    __m128i first16 = _mm_unpacklo_epi8(lo, hi), last16 = _mm_unpackhi_epi8(lo, hi);
    if (remaining >= 32) {
      const float *xp = x + io;
      __m512 acc = _mm512_mul_ps(_mm512_cvtepi32_ps(_mm512_sub_epi32(_mm512_cvtepu8_epi32(first16), eight)),
                                 _mm512_loadu_ps(xp));
      acc = _mm512_fmadd_ps(_mm512_cvtepi32_ps(_mm512_sub_epi32(_mm512_cvtepu8_epi32(last16), eight)),
                            _mm512_loadu_ps(xp + 16), acc);
      row_sum += hsum512(acc) * d;
    } else if (remaining > 0) {
      row_sum += q4_0_tail(b, io, n_cols, x) * d;
    }
  }
  return row_sum;
}

/* ---- Q8_0: simd/avx2/q8_0.rs:335-400 (block sum, then times d) and
 * simd/avx512/q8_0.rs:183-240 (every weight times d first): the two tiers round differently,
 * as they do in the reference. */
static float q8_0_tail(const uint8_t *b, size_t io, size_t remaining, const float *x) {
  float partial = 0.0f;
  for (size_t i = 0; i < remaining; i++) partial += (float)(int8_t)b[2 + i] * x[io + i];
  return partial;
}

__attribute__((target("avx2,fma"))) static float row_q8_0_avx2(const uint8_t *row, size_t bpr, size_t n_cols,
                                                               const float *x) {
  float row_sum = 0.0f;
  for (size_t blk = 0; blk < bpr; blk++) {
    const uint8_t *b = row + blk * 34;
    size_t io = blk * 32, remaining = n_cols > io ? n_cols - io : 0;
    float d = rd_f16(b);
    if (remaining >= 32) {
      __m256i raw = _mm256_loadu_si256((const __m256i *)(b + 2));
      __m128i lo = _mm256_castsi256_si128(raw), hi = _mm256_extracti128_si256(raw, 1);
      const float *xp = x + io;
      __m256 acc = _mm256_mul_ps(_mm256_cvtepi32_ps(_mm256_cvtepi8_epi32(lo)), _mm256_loadu_ps(xp));
      acc = _mm256_fmadd_ps(_mm256_cvtepi32_ps(_mm256_cvtepi8_epi32(_mm_srli_si128(lo, 8))), _mm256_loadu_ps(xp + 8), acc);
      acc = _mm256_fmadd_ps(_mm256_cvtepi32_ps(_mm256_cvtepi8_epi32(hi)), _mm256_loadu_ps(xp + 16), acc);
      acc = _mm256_fmadd_ps(_mm256_cvtepi32_ps(_mm256_cvtepi8_epi32(_mm_srli_si128(hi, 8))), _mm256_loadu_ps(xp + 24), acc);
      row_sum += hsum256(acc) * d;
    } else if (remaining > 0) {
      row_sum += q8_0_tail(b, io, remaining, x) * d;
    }
  }
  return row_sum;
}

__attribute__((target("avx512f,avx2,fma"))) static float row_q8_0_avx512(const uint8_t *row, size_t bpr,
                                                                       size_t n_cols, const float *x) {
  float row_sum = 0.0f;
  for (size_t blk = 0; blk < bpr; blk++) {
    const uint8_t *b = row + blk * 34;
    size_t io = blk * 32, remaining = n_cols > io ? n_cols - io : 0;
    float d = rd_f16(b);
    if (remaining >= 32) {
      __m128i q1 = _mm_loadu_si128((const __m128i *)(b + 2)), q2 = _mm_loadu_si128((const __m128i *)(b + 18));
      __m512 vd = _mm512_set1_ps(d);
      const float *xp = x + io;
      __m512 w1 = _mm512_mul_ps(_mm512_cvtepi32_ps(_mm512_cvtepi8_epi32(q1)), vd);
      __m512 acc = _mm512_mul_ps(w1, _mm512_loadu_ps(xp));
      __m512 w2 = _mm512_mul_ps(_mm512_cvtepi32_ps(_mm512_cvtepi8_epi32(q2)), vd);
      acc = _mm512_fmadd_ps(w2, _mm512_loadu_ps(xp + 16), acc);
      row_sum += hsum512(acc);
    } else if (remaining > 0) {
      row_sum += q8_0_tail(b, io, remaining, x) * d;
    }
  }
  return row_sum;
}

/* ---- Q6_K: simd/avx2/q6_k.rs:497-742 with decode_q6_group (:307-355), simd/avx512/q6_k.rs:337-470.
 * Per half of a super-block the four 6-bit streams are assembled from ql / qh sixteen bytes at
 * a time, 32 is subtracted as integers, each 16-column strip is scaled by d * scale (one
 * rounded product per weight) and FMA'd into the block accumulator; one horizontal sum per
 * super-block.  A partial last super-block goes to the scalar row. */
static inline void q6_group(const uint8_t *ql, const uint8_t *qh, __m128i q[4]) {
  const __m128i m4 = _mm_set1_epi8(0x0F), m2 = _mm_set1_epi8(0x03);
  __m128i ql0 = _mm_loadu_si128((const __m128i *)ql), ql1 = _mm_loadu_si128((const __m128i *)(ql + 32));
  __m128i h = _mm_loadu_si128((const __m128i *)qh);
  q[0] = _mm_or_si128(_mm_and_si128(ql0, m4), _mm_slli_epi16(_mm_and_si128(h, m2), 4));
  q[1] = _mm_or_si128(_mm_and_si128(ql1, m4), _mm_slli_epi16(_mm_and_si128(_mm_srli_epi16(h, 2), m2), 4));
  q[2] = _mm_or_si128(_mm_and_si128(_mm_srli_epi16(ql0, 4), m4), _mm_slli_epi16(_mm_and_si128(_mm_srli_epi16(h, 4), m2), 4));
  q[3] = _mm_or_si128(_mm_and_si128(_mm_srli_epi16(ql1, 4), m4), _mm_slli_epi16(_mm_and_si128(_mm_srli_epi16(h, 6), m2), 4));
}

__attribute__((target("avx2,fma"))) static float row_q6_k_avx2(const uint8_t *row, size_t bpr, size_t n_cols,
                                                               const float *x) {
  float row_sum = 0.0f;
  const __m256i off32 = _mm256_set1_epi32(32);
  for (size_t blk = 0; blk < bpr; blk++) {
    const uint8_t *b = row + blk * 210;
    size_t io = blk * 256, remaining = n_cols > io ? n_cols - io : 0;
    if (remaining >= 256) {
      const uint8_t *ql = b, *qh = b + 128;
      const int8_t *sc = (const int8_t *)(b + 192);
      float d = rd_f16(b + 208);
      __m256 acc = _mm256_setzero_ps();
      for (int g = 0; g < 2; g++) {
        __m128i qa[4], qb[4];
        q6_group(ql + 64 * g, qh + 32 * g, qa);            /* positions 0..15 of every stream */
        q6_group(ql + 64 * g + 16, qh + 32 * g + 16, qb);  /* positions 16..31 */
        for (int k = 0; k < 4; k++) {
          __m256 va = _mm256_set1_ps(d * (float)sc[8 * g + 2 * k]), vb = _mm256_set1_ps(d * (float)sc[8 * g + 2 * k + 1]);
          const float *xp = x + io + 128 * g + 32 * k;
          __m256 w;
          w = _mm256_cvtepi32_ps(_mm256_sub_epi32(_mm256_cvtepu8_epi32(qa[k]), off32));
          acc = _mm256_fmadd_ps(_mm256_mul_ps(va, w), _mm256_loadu_ps(xp), acc);
          w = _mm256_cvtepi32_ps(_mm256_sub_epi32(_mm256_cvtepu8_epi32(_mm_srli_si128(qa[k], 8)), off32));
          acc = _mm256_fmadd_ps(_mm256_mul_ps(va, w), _mm256_loadu_ps(xp + 8), acc);
          w = _mm256_cvtepi32_ps(_mm256_sub_epi32(_mm256_cvtepu8_epi32(qb[k]), off32));
          acc = _mm256_fmadd_ps(_mm256_mul_ps(vb, w), _mm256_loadu_ps(xp + 16), acc);
          w = _mm256_cvtepi32_ps(_mm256_sub_epi32(_mm256_cvtepu8_epi32(_mm_srli_si128(qb[k], 8)), off32));
          acc = _mm256_fmadd_ps(_mm256_mul_ps(vb, w), _mm256_loadu_ps(xp + 24), acc);
        }
      }
      row_sum += hsum256(acc);
    } else if (remaining > 0) {
      row_sum += row_q6_k_f32(b, 1, remaining, x + io);
    }
  }
  return row_sum;
}

__attribute__((target("avx512f,avx2,fma"))) static float row_q6_k_avx512(const uint8_t *row, size_t bpr,
                                                                       size_t n_cols, const float *x) {
  float row_sum = 0.0f;
  const __m512i off32 = _mm512_set1_epi32(32);
  for (size_t blk = 0; blk < bpr; blk++) {
    const uint8_t *b = row + blk * 210;
    size_t io = blk * 256, remaining = n_cols > io ? n_cols - io : 0;
    if (remaining >= 256) {
      const uint8_t *ql = b, *qh = b + 128;
      const int8_t *sc = (const int8_t *)(b + 192);
      float d = rd_f16(b + 208);
      __m512 acc = _mm512_setzero_ps();
      for (int g = 0; g < 2; g++) {
        __m128i qa[4], qb[4];
        q6_group(ql + 64 * g, qh + 32 * g, qa);
        q6_group(ql + 64 * g + 16, qh + 32 * g + 16, qb);
        for (int k = 0; k < 4; k++) {
          __m512 va = _mm512_set1_ps(d * (float)sc[8 * g + 2 * k]), vb = _mm512_set1_ps(d * (float)sc[8 * g + 2 * k + 1]);
          const float *xp = x + io + 128 * g + 32 * k;
          __m512 w = _mm512_cvtepi32_ps(_mm512_sub_epi32(_mm512_cvtepu8_epi32(qa[k]), off32));
          acc = _mm512_fmadd_ps(_mm512_mul_ps(va, w), _mm512_loadu_ps(xp), acc);
          w = _mm512_cvtepi32_ps(_mm512_sub_epi32(_mm512_cvtepu8_epi32(qb[k]), off32));
          acc = _mm512_fmadd_ps(_mm512_mul_ps(vb, w), _mm512_loadu_ps(xp + 16), acc);
        }
      }
      row_sum += hsum512(acc);
    } else if (remaining > 0) {
      row_sum += row_q6_k_f32(b, 1, remaining, x + io);
    }
  }
  return row_sum;
}

/* ---- IQ4_XS: simd/avx2/iq4_xs.rs:217-283, simd/avx512/iq4_xs.rs:277-335.  The table lookup is
 * scalar (a small f32 array per 8 or 16 weights), then (scale * w) FMA'd with x into one
 * accumulator for the whole row; chunks that straddle n_cols are summed in scalar. */
__attribute__((target("avx2,fma"))) static float row_iq4_xs_avx2(const uint8_t *row, size_t bpr, size_t n_cols,
                                                                 const float *x) {
  __m256 acc = _mm256_setzero_ps();
  float scalar_rem = 0.0f;
  size_t col = 0;
  for (size_t blk = 0; blk < bpr; blk++, col += 256) {
    const uint8_t *b = row + blk * 136;
    float d = rd_f16(b);
    uint16_t sh = (uint16_t)(b[2] | (b[3] << 8));
    const uint8_t *nib = b + 8;
    for (int sub = 0; sub < 8; sub++) {
      float scale = d * (float)unpack_sub_scale(sh, b + 4, sub);
      __m256 sv = _mm256_set1_ps(scale);
      for (int chunk = 0; chunk < 4; chunk++) {
        float w8[8];
        for (int i = 0; i < 4; i++) {
          uint8_t byte = nib[16 * sub + 4 * chunk + i];
          w8[2 * i] = (float)KVALUES_IQ4NL[byte & 0x0F];
          w8[2 * i + 1] = (float)KVALUES_IQ4NL[byte >> 4];
        }
        size_t c = col + 32 * (size_t)sub + 8 * (size_t)chunk;
        if (c + 8 <= n_cols) {
          acc = _mm256_fmadd_ps(_mm256_mul_ps(sv, _mm256_loadu_ps(w8)), _mm256_loadu_ps(x + c), acc);
        } else {
          for (int j = 0; j < 8; j++)
            if (c + (size_t)j < n_cols) scalar_rem += scale * w8[j] * x[c + j];
        }
      }
    }
  }
  return hsum256(acc) + scalar_rem;
}

__attribute__((target("avx512f,avx2,fma"))) static float row_iq4_xs_avx512(const uint8_t *row, size_t bpr,
                                                                         size_t n_cols, const float *x) {
  __m512 acc = _mm512_setzero_ps();
  float scalar_rem = 0.0f;
  size_t col = 0;
  for (size_t blk = 0; blk < bpr; blk++, col += 256) {
    const uint8_t *b = row + blk * 136;
    float d = rd_f16(b);
    uint16_t sh = (uint16_t)(b[2] | (b[3] << 8));
    const uint8_t *nib = b + 8;
    for (int sub = 0; sub < 8; sub++) {
      float scale = d * (float)unpack_sub_scale(sh, b + 4, sub);
      __m512 sv = _mm512_set1_ps(scale);
      for (int chunk = 0; chunk < 2; chunk++) {
        float w16[16];
        for (int i = 0; i < 8; i++) {
          uint8_t byte = nib[16 * sub + 8 * chunk + i];
          w16[2 * i] = (float)KVALUES_IQ4NL[byte & 0x0F];
          w16[2 * i + 1] = (float)KVALUES_IQ4NL[byte >> 4];
        }
        size_t c = col + 32 * (size_t)sub + 16 * (size_t)chunk;
        if (c + 16 <= n_cols) {
          acc = _mm512_fmadd_ps(_mm512_mul_ps(sv, _mm512_loadu_ps(w16)), _mm512_loadu_ps(x + c), acc);
        } else {
          for (int j = 0; j < 16; j++)
            if (c + (size_t)j < n_cols) scalar_rem += scale * w16[j] * x[c + j];
        }
      }
    }
  }
  return hsum512(acc) + scalar_rem;
}

/* Highest tier this CPU can run: 2 = AVX-512F, 1 = AVX2+FMA, 0 = scalar. */
int qk_cpu_best_tier(void) {
  __builtin_cpu_init();
  if (__builtin_cpu_supports("avx512f")) return 2;
  if (__builtin_cpu_supports("avx2") && __builtin_cpu_supports("fma")) return 1;
  return 0;
}

int qk_cpu_max_threads(void) {
  long n = sysconf(_SC_NPROCESSORS_ONLN);
  return n < 1 ? 1 : (int)n;
}

/* The row kernel of (type, tier), NULL where the reference has none (then the tier below runs). */
static row_fn simd_row(int type, int tier) {
  switch (type) {
    case T_Q4_0:
      return tier == 2 ? row_q4_0_avx512 : tier == 1 ? row_q4_0_avx2 : NULL;
    case T_Q8_0:
      return tier == 2 ? row_q8_0_avx512 : tier == 1 ? row_q8_0_avx2 : NULL;
    case T_Q4_K:
      return tier == 2 ? row_q4_k_avx512 : tier == 1 ? row_q4_k_avx2 : NULL;
    case T_Q6_K:
      return tier == 2 ? row_q6_k_avx512 : tier == 1 ? row_q6_k_avx2 : NULL;
    case T_IQ4_XS:
      return tier == 2 ? row_iq4_xs_avx512 : tier == 1 ? row_iq4_xs_avx2 : NULL;
    default:
      return NULL;
  }
}

/* ---- a persistent pool of workers (the reference's parallel_gemv runs on rayon's pool,
 * crates/oxillama-quant/src/parallel.rs:33-92; spawning threads per matvec would charge the
 * CPU arm a cost the reference does not pay) ---- */
typedef struct {
  row_fn f;
  const uint8_t *w;
  const float *x;
  float *y;
  size_t n_rows, bpr, row_bytes, n_cols;
  int threads;
} job_t;

#define POOL_MAX 256
static pthread_t pool_tid[POOL_MAX];
static int pool_size = 0;
static pthread_mutex_t pool_mu = PTHREAD_MUTEX_INITIALIZER;
static pthread_cond_t pool_go = PTHREAD_COND_INITIALIZER, pool_done = PTHREAD_COND_INITIALIZER;
static job_t pool_job;
static unsigned long pool_epoch = 0;
static int pool_pending = 0;

static void run_rows(const job_t *j, int t) {
  size_t r0 = j->n_rows * (size_t)t / (size_t)j->threads, r1 = j->n_rows * (size_t)(t + 1) / (size_t)j->threads;
  for (size_t r = r0; r < r1; r++) j->y[r] = j->f(j->w + r * j->row_bytes, j->bpr, j->n_cols, j->x);
}

static void *pool_worker(void *arg) {
  const int id = (int)(size_t)arg; /* workers are 1 .. pool_size; the caller is thread 0 */
  unsigned long seen = 0;
  for (;;) {
    pthread_mutex_lock(&pool_mu);
    while (pool_epoch == seen) pthread_cond_wait(&pool_go, &pool_mu);
    seen = pool_epoch;
    job_t j = pool_job;
    pthread_mutex_unlock(&pool_mu);
    if (id < j.threads) run_rows(&j, id);
    pthread_mutex_lock(&pool_mu);
    if (--pool_pending == 0) pthread_cond_signal(&pool_done);
    pthread_mutex_unlock(&pool_mu);
  }
  return NULL;
}

/* y = W x over `threads` cores, contiguous row spans.  *tier_used reports the tier that ran
 * (the highest one <= `tier` that both the CPU and the format have). */
int qk_cpu_gemv(int type, int tier, int threads, const uint8_t *w, size_t n_rows, size_t n_cols,
                const float *x, float *y, int *tier_used) {
  size_t bs = qk_oracle_block_size(type), bb = qk_oracle_block_bytes(type);
  if (bs == 0) return QK_UNSUPPORTED_TYPE;
  size_t bpr = (n_cols + bs - 1) / bs, row_bytes = bpr * bb;
  row_fn f = pick_row(type, 0);
  int used = 0, best = qk_cpu_best_tier();
  for (int t = tier < best ? tier : best; t >= 1; t--)
    if (simd_row(type, t)) {
      f = simd_row(type, t);
      used = t;
      break;
    }
  if (tier_used) *tier_used = used;
  if (threads < 1) threads = 1;
  if (threads > POOL_MAX) threads = POOL_MAX;
  if ((size_t)threads > n_rows) threads = n_rows ? (int)n_rows : 1;
  job_t j = {f, w, x, y, n_rows, bpr, row_bytes, n_cols, threads};
  if (threads == 1) {
    run_rows(&j, 0);
    return QK_OK;
  }
  pthread_mutex_lock(&pool_mu);
  while (pool_size < threads - 1) { /* grow the pool to threads - 1 workers */
    pool_size++;
    if (pthread_create(&pool_tid[pool_size], NULL, pool_worker, (void *)(size_t)pool_size) != 0) {
      pool_size--;
      pthread_mutex_unlock(&pool_mu);
      return QK_KERNEL_ERROR;
    }
  }
  pool_job = j;
  pool_pending = pool_size; /* every worker wakes and checks whether it has a span */
  pool_epoch++;
  pthread_cond_broadcast(&pool_go);
  pthread_mutex_unlock(&pool_mu);
  run_rows(&j, 0);
  pthread_mutex_lock(&pool_mu);
  while (pool_pending) pthread_cond_wait(&pool_done, &pool_mu);
  pthread_mutex_unlock(&pool_mu);
  return QK_OK;
}
