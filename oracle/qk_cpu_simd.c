/*
 * CPU baseline for the timing report.  TEST / BENCH INFRASTRUCTURE ONLY — never
 * part of the product path.
 *
 * Restates, in C intrinsics, the reference's fastest CPU tiers for the decode
 * matvec so that they can be timed on the GPU box's host cores beside the CUDA
 * kernels (the reference is Rust and cannot be built where this runs):
 *   tier 0  scalar        crates/oxillama-quant/src/reference/ (the oracle rows)
 *   tier 1  AVX2 + FMA    crates/oxillama-quant/src/simd/avx2/q4_k.rs:589-742   (Q4_K)
 *   tier 2  AVX-512F      crates/oxillama-quant/src/simd/avx512/q4_k.rs:279-410 (Q4_K)
 * wrapped in a row-parallel driver that mirrors parallel_gemv
 * (crates/oxillama-quant/src/parallel.rs:33-92; rayon there, pthreads here).
 * The reference's own call chain is single-threaded (threads = 1); the
 * all-cores figure is what parallel_gemv would give it.
 *
 * Formats without a SIMD restatement here run their scalar rows under the
 * same driver, and the caller is told which tier actually ran.
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

typedef struct {
  row_fn f;
  const uint8_t *w;
  const float *x;
  float *y;
  size_t r0, r1, bpr, row_bytes, n_cols;
} span_t;

static void *run_span(void *p) {
  span_t *s = (span_t *)p;
  for (size_t r = s->r0; r < s->r1; r++) s->y[r] = s->f(s->w + r * s->row_bytes, s->bpr, s->n_cols, s->x);
  return NULL;
}

/* y = W x over `threads` cores, contiguous row spans.  *tier_used reports the
 * tier that ran (a format without a SIMD restatement runs tier 0). */
int qk_cpu_gemv(int type, int tier, int threads, const uint8_t *w, size_t n_rows, size_t n_cols,
                const float *x, float *y, int *tier_used) {
  size_t bs = qk_oracle_block_size(type), bb = qk_oracle_block_bytes(type);
  if (bs == 0) return QK_UNSUPPORTED_TYPE;
  size_t bpr = (n_cols + bs - 1) / bs, row_bytes = bpr * bb;
  row_fn f = pick_row(type, 0);
  int used = 0;
  if (type == T_Q4_K && tier >= 2 && qk_cpu_best_tier() >= 2) {
    f = row_q4_k_avx512;
    used = 2;
  } else if (type == T_Q4_K && tier >= 1 && qk_cpu_best_tier() >= 1) {
    f = row_q4_k_avx2;
    used = 1;
  }
  if (tier_used) *tier_used = used;
  if (threads < 1) threads = 1;
  if (threads > 256) threads = 256;
  if ((size_t)threads > n_rows) threads = n_rows ? (int)n_rows : 1;
  span_t spans[256];
  pthread_t tids[256];
  for (int t = 0; t < threads; t++) {
    span_t s = {f, w, x, y, n_rows * t / threads, n_rows * (t + 1) / threads, bpr, row_bytes, n_cols};
    spans[t] = s;
  }
  for (int t = 1; t < threads; t++) pthread_create(&tids[t], NULL, run_span, &spans[t]);
  run_span(&spans[0]);
  for (int t = 1; t < threads; t++) pthread_join(tids[t], NULL);
  return QK_OK;
}
