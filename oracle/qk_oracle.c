/*
 * CPU oracle for the quantized dequant-dot path.  TEST INFRASTRUCTURE ONLY.
 *
 * This file is a plain-C restatement, statement for statement, of the scalar
 * kernels of cool-japan/oxillama's `oxillama-quant` crate.  It exists so that
 * the CUDA path can be checked against the reference's arithmetic; it is never
 * linked into, loaded by, or called from the product library.  Only tests, the
 * smoke check and the CPU-baseline leg of the benchmark may use it.
 *
 * Parity status: pinned against the known-answer tests the reference's own
 * unit tests hold for these formats (re-typed in tests/test_oracle_kat.py) and
 * cross-checked against gguf-py for the three canonical layouts (Q8_0, Q4_K,
 * Q6_K).  The reference itself is Rust and cannot be compiled where this was
 * written, so no output of the reference binary pins it; the subnormal and
 * rounding-tie behaviour of the f16 conversions rests on IEEE-754 semantics
 * (the `half` crate, version 2.7.1, implements exactly those).
 *
 * Build with -ffp-contract=off and without -ffast-math: Rust never contracts
 * a*b+c into an FMA and never reassociates, and neither may this file.
 *
 * Every function cites the reference source it follows as
 * crates/oxillama-quant/src/<file>:<lines>.
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define QK_OK 0
#define QK_UNSUPPORTED_TYPE 1
#define QK_DIMENSION_MISMATCH 3
#define QK_KERNEL_ERROR 4
#define QK_BUFFER_TOO_SMALL 6

#define T_Q4_0 2
#define T_Q8_0 8
#define T_Q4_K 12
#define T_Q6_K 14
#define T_IQ4_XS 23
#define T_Q5_K 13
#define T_Q2_K 10
#define T_Q3_K 11
#define T_Q8_K 15

#define Q8_0_BLOCK_BYTES 34

/* ---- f16 <-> f32, IEEE-754 binary16, as half::f16::{to_f32,from_f32} ---- */

/* Exact widening, subnormals included (reference/q4_k.rs:351-353). */
float qk_oracle_f16_to_f32(uint16_t h) {
  uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
  uint32_t exp = (h >> 10) & 0x1Fu;
  uint32_t man = h & 0x3FFu;
  uint32_t bits;
  if (exp == 0) {
    if (man == 0) {
      bits = sign;
    } else { /* subnormal: normalise */
      int e = -1;
      do {
        man <<= 1;
        e++;
      } while ((man & 0x400u) == 0);
      man &= 0x3FFu;
      bits = sign | ((uint32_t)(127 - 15 - e) << 23) | (man << 13);
    }
  } else if (exp == 31) {
    bits = sign | 0x7F800000u | (man << 13);
  } else {
    bits = sign | ((exp + 127 - 15) << 23) | (man << 13);
  }
  float f;
  memcpy(&f, &bits, 4);
  return f;
}

/* Round-to-nearest-even narrowing (quantize.rs:201, f16::from_f32). */
uint16_t qk_oracle_f32_to_f16(float f) {
  uint32_t x;
  memcpy(&x, &f, 4);
  uint32_t sign = (x >> 16) & 0x8000u;
  uint32_t exp = (x >> 23) & 0xFFu;
  uint32_t man = x & 0x7FFFFFu;
  if (exp == 255) { /* inf / nan */
    return (uint16_t)(sign | 0x7C00u | (man ? (0x200u | (man >> 13)) : 0));
  }
  int e = (int)exp - 127 + 15;
  if (e >= 31) return (uint16_t)(sign | 0x7C00u); /* overflow -> inf */
  if (e <= 0) {                                   /* subnormal or zero */
    if (e < -10) return (uint16_t)sign;
    man |= 0x800000u;
    int shift = 14 - e; /* 14..24 */
    uint32_t half_man = man >> shift;
    uint32_t rem = man & ((1u << shift) - 1);
    uint32_t halfway = 1u << (shift - 1);
    if (rem > halfway || (rem == halfway && (half_man & 1))) half_man++;
    return (uint16_t)(sign | half_man);
  }
  uint32_t half_man = man >> 13;
  uint32_t rem = man & 0x1FFFu;
  uint16_t out = (uint16_t)(sign | ((uint32_t)e << 10) | half_man);
  if (rem > 0x1000u || (rem == 0x1000u && (half_man & 1))) out++; /* may carry into exp: correct */
  return out;
}

static inline float rd_f16(const uint8_t *p) {
  return qk_oracle_f16_to_f32((uint16_t)(p[0] | (p[1] << 8)));
}

/* reference/iq_shared.rs:16-18 */
static const int8_t KVALUES_IQ4NL[16] = {-127, -104, -83, -65, -49, -35, -22, -10,
                                         1,    13,   25,  38,  53,  69,  89,  113};

size_t qk_oracle_block_size(int type) {
  switch (type) {
    case T_Q4_0:
    case T_Q8_0:
      return 32;
    case T_Q2_K:
    case T_Q3_K:
    case T_Q4_K:
    case T_Q5_K:
    case T_Q6_K:
    case T_Q8_K:
    case T_IQ4_XS:
      return 256;
    default:
      return 0;
  }
}

size_t qk_oracle_block_bytes(int type) {
  switch (type) {
    case T_Q4_0:
      return 18;
    case T_Q8_0:
      return 34;
    case T_Q4_K:
      return 144;
    case T_Q5_K:
      return 176;
    case T_Q2_K:
      return 84;
    case T_Q3_K:
      return 110;
    case T_Q8_K:
      return 292;
    case T_Q6_K:
      return 210;
    case T_IQ4_XS:
      return 136;
    default:
      return 0;
  }
}

/* reference/q4_k.rs:27-49 */
static void decode_scales_mins(const uint8_t *s, uint8_t sc[8], uint8_t mn[8]) {
  for (int j = 0; j < 4; j++) {
    sc[j] = s[j] & 0x3F;
    mn[j] = s[j + 4] & 0x3F;
  }
  for (int j = 4; j < 8; j++) {
    uint8_t lo_sc = s[j + 4] & 0x0F;
    uint8_t hi_sc = (s[j - 4] >> 6) & 0x03;
    sc[j] = (uint8_t)(lo_sc | (hi_sc << 4));
    uint8_t lo_mn = (s[j + 4] >> 4) & 0x0F;
    uint8_t hi_mn = (s[j] >> 6) & 0x03;
    mn[j] = (uint8_t)(lo_mn | (hi_mn << 4));
  }
}

/* reference/iq4_xs.rs:47-53 */
static int unpack_sub_scale(uint16_t scales_h, const uint8_t *scales_l, int i) {
  uint8_t ls_low = (uint8_t)((scales_l[i / 2] >> (4 * (i & 1))) & 0x0F);
  uint8_t ls_high = (uint8_t)((uint8_t)(scales_h >> (2 * i)) & 0x03);
  uint8_t ls = (uint8_t)(ls_low | (ls_high << 4));
  return (int)ls - 32;
}

/* ------------------------------ dequant_block ------------------------------ */

/* reference/q4_0.rs:22-49 — low nibble of byte i -> element 2i, high -> 2i+1. */
static void dq_q4_0(const uint8_t *b, float *out) {
  float d = rd_f16(b);
  for (int i = 0; i < 16; i++) {
    uint8_t byte = b[2 + i];
    int lo = (int)(byte & 0x0F) - 8;
    int hi = (int)((byte >> 4) & 0x0F) - 8;
    out[i * 2] = (float)lo * d;
    out[i * 2 + 1] = (float)hi * d;
  }
}

/* reference/q8_0.rs:22-44 */
static void dq_q8_0(const uint8_t *b, float *out) {
  float d = rd_f16(b);
  for (int i = 0; i < 32; i++) out[i] = (float)(int8_t)b[2 + i] * d;
}

/* reference/q4_k.rs:52-102 */
static void dq_q4_k(const uint8_t *b, float *out) {
  float d = rd_f16(b), dmin = rd_f16(b + 2);
  const uint8_t *qs = b + 16;
  uint8_t sc[8], mn[8];
  decode_scales_mins(b + 4, sc, mn);
  int is = 0, qo = 0, oo = 0;
  for (int g = 0; g < 4; g++) {
    float d1 = d * (float)sc[is];
    float m1 = dmin * (float)mn[is];
    float d2 = d * (float)sc[is + 1];
    float m2 = dmin * (float)mn[is + 1];
    for (int l = 0; l < 32; l++) {
      float q = (float)(qs[qo + l] & 0x0F);
      float t = d1 * q; /* separately rounded product, then subtraction */
      out[oo + l] = t - m1;
    }
    for (int l = 0; l < 32; l++) {
      float q = (float)((qs[qo + l] >> 4) & 0x0F);
      float t = d2 * q;
      out[oo + 32 + l] = t - m2;
    }
    is += 2;
    qo += 32;
    oo += 64;
  }
}

/* reference/q5_k.rs:53-111: d @0, dmin @2, 12 bytes of 6-bit scales / mins @4 (same packing as
 * Q4_K, q5_k.rs:27-50), qh @16 (32 bytes: bit g of byte l is the fifth bit of the low-nibble
 * quant of group g, bit g + 4 that of the high-nibble quant), qs @48 (128 bytes). */
static void dq_q5_k(const uint8_t *b, float *out) {
  float d = rd_f16(b), dmin = rd_f16(b + 2);
  const uint8_t *qh = b + 16, *qs = b + 48;
  uint8_t sc[8], mn[8];
  decode_scales_mins(b + 4, sc, mn);
  int is = 0, qo = 0, oo = 0;
  for (int g = 0; g < 4; g++) {
    float d1 = d * (float)sc[is];
    float m1 = dmin * (float)mn[is];
    float d2 = d * (float)sc[is + 1];
    float m2 = dmin * (float)mn[is + 1];
    for (int l = 0; l < 32; l++) {
      uint8_t hb = (uint8_t)((qh[l] >> g) & 1);
      float q = (float)(uint8_t)((qs[qo + l] & 0x0F) | (hb << 4));
      float t = d1 * q;
      out[oo + l] = t - m1;
    }
    for (int l = 0; l < 32; l++) {
      uint8_t hb = (uint8_t)((qh[l] >> (g + 4)) & 1);
      float q = (float)(uint8_t)(((qs[qo + l] >> 4) & 0x0F) | (hb << 4));
      float t = d2 * q;
      out[oo + 32 + l] = t - m2;
    }
    is += 2;
    qo += 32;
    oo += 64;
  }
}

/* reference/q2_k.rs:27-82: scales @0 (16 bytes: low nibble = scale, high nibble = min of a
 * 16-weight sub-block), qs @16 (64 bytes, four 2-bit quants per byte), d @80, dmin @82. */
static void dq_q2_k(const uint8_t *b, float *out) {
  const uint8_t *scales = b, *qs = b + 16;
  float d = rd_f16(b + 80), dmin = rd_f16(b + 82);
  int is = 0;
  size_t qo = 0, oo = 0;
  for (int n = 0; n < 2; n++) {
    for (int shift = 0; shift < 8; shift += 2) {
      for (int h = 0; h < 2; h++) {
        uint8_t sb = scales[is++];
        float dl = d * (float)(sb & 0x0F);
        float ml = dmin * (float)(sb >> 4);
        for (int l = 0; l < 16; l++) {
          uint8_t q = (uint8_t)((qs[qo + 16 * h + l] >> shift) & 3);
          float t = dl * (float)q;
          out[oo + l] = t - ml;
        }
        oo += 16;
      }
    }
    qo += 32;
  }
}

/* reference/q3_k.rs:29-59: sixteen 6-bit scales from 12 bytes, then -32. */
static void decode_scales_q3_k(const uint8_t *r, float *sc) {
  uint32_t u[16];
  for (int j = 0; j < 4; j++) u[j] = r[j] & 0x3Fu;
  for (int j = 0; j < 4; j++) u[4 + j] = r[4 + j] & 0x3Fu;
  for (int j = 0; j < 4; j++) u[8 + j] = (uint32_t)(r[8 + j] & 0x0F) | (((uint32_t)(r[j] >> 6) & 3u) << 4);
  for (int j = 0; j < 4; j++) u[12 + j] = (uint32_t)((r[8 + j] >> 4) & 0x0F) | (((uint32_t)(r[4 + j] >> 6) & 3u) << 4);
  for (int i = 0; i < 16; i++) sc[i] = (float)((int32_t)u[i] - 32);
}

/* reference/q3_k.rs:61-121: hmask @0 (32 bytes; bit set: subtract 0, clear: subtract 4), qs @32
 * (64 bytes, low two bits of each quant), scales @96, d @108. */
static void dq_q3_k(const uint8_t *b, float *out) {
  const uint8_t *hmask = b, *qs = b + 32;
  float d = rd_f16(b + 108);
  float sc[16];
  decode_scales_q3_k(b + 96, sc);
  int is = 0;
  size_t oo = 0;
  uint8_t m = 1;
  for (int group = 0; group < 2; group++) {
    size_t qs_base = (size_t)group * 32;
    for (int shift = 0; shift < 8; shift += 2) {
      for (int n = 0; n < 2; n++) {
        float dl = d * sc[is++];
        for (int l = 0; l < 16; l++) {
          int q_lo = (qs[qs_base + (size_t)n * 16 + l] >> shift) & 3;
          int sub = (hmask[n * 16 + l] & m) ? 0 : 4;
          out[oo + l] = dl * (float)(q_lo - sub);
        }
        oo += 16;
      }
      m = (uint8_t)(m << 1);
    }
  }
}

/* reference/q8_k.rs:26-50: d (f32) @0, 256 int8 quants @4, sixteen i16 block sums @260 (unused). */
static float rd_f32(const uint8_t *p) {
  uint32_t u = (uint32_t)p[0] | ((uint32_t)p[1] << 8) | ((uint32_t)p[2] << 16) | ((uint32_t)p[3] << 24);
  float f;
  memcpy(&f, &u, 4);
  return f;
}
static void dq_q8_k(const uint8_t *b, float *out) {
  float d = rd_f32(b);
  for (int i = 0; i < 256; i++) out[i] = d * (float)(int8_t)b[4 + i];
}

/* reference/q6_k.rs:25-75 */
static void dq_q6_k(const uint8_t *b, float *out) {
  const uint8_t *ql = b, *qh = b + 128, *scales = b + 192;
  float d = rd_f16(b + 208);
  for (int g = 0; g < 2; g++) {
    int ql_off = g * 64, qh_off = g * 32, sc_off = g * 8, out_off = g * 128;
    for (int l = 0; l < 32; l++) {
      int is = l / 16;
      int q1 = (int)(uint8_t)((ql[ql_off + l] & 0x0F) | ((qh[qh_off + l] & 3) << 4)) - 32;
      int q2 = (int)(uint8_t)((ql[ql_off + l + 32] & 0x0F) | (((qh[qh_off + l] >> 2) & 3) << 4)) - 32;
      int q3 = (int)(uint8_t)((ql[ql_off + l] >> 4) | (((qh[qh_off + l] >> 4) & 3) << 4)) - 32;
      int q4 = (int)(uint8_t)((ql[ql_off + l + 32] >> 4) | (((qh[qh_off + l] >> 6) & 3) << 4)) - 32;
      float s0 = (float)(int8_t)scales[sc_off + is];
      float s1 = (float)(int8_t)scales[sc_off + is + 2];
      float s2 = (float)(int8_t)scales[sc_off + is + 4];
      float s3 = (float)(int8_t)scales[sc_off + is + 6];
      float t0 = d * s0, t1 = d * s1, t2 = d * s2, t3 = d * s3;
      out[out_off + l] = t0 * (float)q1;
      out[out_off + l + 32] = t1 * (float)q2;
      out[out_off + l + 64] = t2 * (float)q3;
      out[out_off + l + 96] = t3 * (float)q4;
    }
  }
}

/* reference/iq4_xs.rs:59-97 */
static void dq_iq4_xs(const uint8_t *b, float *out) {
  float d = rd_f16(b);
  uint16_t sh = (uint16_t)(b[2] | (b[3] << 8));
  const uint8_t *sl = b + 4, *nib = b + 8;
  for (int sub = 0; sub < 8; sub++) {
    int ls = unpack_sub_scale(sh, sl, sub);
    float scale = d * (float)ls;
    for (int i = 0; i < 16; i++) {
      uint8_t byte = nib[sub * 16 + i];
      out[sub * 32 + i * 2] = scale * (float)KVALUES_IQ4NL[byte & 0x0F];
      out[sub * 32 + i * 2 + 1] = scale * (float)KVALUES_IQ4NL[(byte >> 4) & 0x0F];
    }
  }
}

int qk_oracle_dequant_block(int type, const uint8_t *block, size_t block_len, float *out,
                            size_t out_len) {
  size_t bs = qk_oracle_block_size(type), bb = qk_oracle_block_bytes(type);
  if (bs == 0) return QK_UNSUPPORTED_TYPE;
  if (block_len < bb) return QK_BUFFER_TOO_SMALL;
  if (out_len < bs) return QK_BUFFER_TOO_SMALL;
  switch (type) {
    case T_Q4_0:
      dq_q4_0(block, out);
      break;
    case T_Q8_0:
      dq_q8_0(block, out);
      break;
    case T_Q4_K:
      dq_q4_k(block, out);
      break;
    case T_Q2_K:
      dq_q2_k(block, out);
      break;
    case T_Q3_K:
      dq_q3_k(block, out);
      break;
    case T_Q8_K:
      dq_q8_k(block, out);
      break;
    case T_Q5_K:
      dq_q5_k(block, out);
      break;
    case T_Q6_K:
      dq_q6_k(block, out);
      break;
    case T_IQ4_XS:
      dq_iq4_xs(block, out);
      break;
  }
  return QK_OK;
}

/* Dequantise a whole [n_rows x n_cols] matrix to f32, block by block, in
 * order, dropping the padding columns of a partial last block — what the MoE
 * loader does (crates/oxillama-arch/src/llama/model.rs:843-886). */
int qk_oracle_dequant_matrix(int type, const uint8_t *w, size_t w_len, size_t n_rows,
                             size_t n_cols, float *out) {
  size_t bs = qk_oracle_block_size(type), bb = qk_oracle_block_bytes(type);
  if (bs == 0) return QK_UNSUPPORTED_TYPE;
  size_t bpr = (n_cols + bs - 1) / bs;
  if (w_len < n_rows * bpr * bb) return QK_BUFFER_TOO_SMALL;
  float tmp[256];
  for (size_t r = 0; r < n_rows; r++)
    for (size_t b = 0; b < bpr; b++) {
      qk_oracle_dequant_block(type, w + (r * bpr + b) * bb, bb, tmp, 256);
      size_t valid = n_cols - b * bs < bs ? n_cols - b * bs : bs;
      memcpy(out + r * n_cols + b * bs, tmp, valid * sizeof(float));
    }
  return QK_OK;
}

/* ---------------------------------- gemv ---------------------------------- */
/* Each row: `sum` starts at 0.0f32 and is updated sequentially in the
 * reference's column order with separately rounded f32 multiplies and adds.
 * ACC is float for the bit-level oracle and double for the error-budget
 * variant (same products, wider running sum). */

#define DEFINE_ROW_DOTS(SUFFIX, ACC)                                                           \
  /* reference/q4_0.rs:80-104 */                                                               \
  static float row_q4_0##SUFFIX(const uint8_t *row, size_t bpr, size_t n_cols, const float *x) { \
    ACC sum = 0;                                                                               \
    for (size_t blk = 0; blk < bpr; blk++) {                                                   \
      const uint8_t *b = row + blk * 18;                                                       \
      float d = rd_f16(b);                                                                     \
      size_t io = blk * 32;                                                                    \
      for (int i = 0; i < 16; i++) {                                                           \
        uint8_t byte = b[2 + i];                                                               \
        int lo = (int)(byte & 0x0F) - 8, hi = (int)((byte >> 4) & 0x0F) - 8;                   \
        size_t idx = io + (size_t)i * 2;                                                       \
        if (idx + 1 < n_cols) {                                                                \
          float w0 = (float)lo * d, w1 = (float)hi * d;                                        \
          float p0 = w0 * x[idx], p1 = w1 * x[idx + 1];                                        \
          sum += p0;                                                                           \
          sum += p1;                                                                           \
        } else if (idx < n_cols) {                                                             \
          float w0 = (float)lo * d;                                                            \
          float p0 = w0 * x[idx];                                                              \
          sum += p0;                                                                           \
        }                                                                                      \
      }                                                                                        \
    }                                                                                          \
    return (float)sum;                                                                         \
  }                                                                                            \
  /* reference/q8_0.rs:75-94 */                                                                \
  static float row_q8_0##SUFFIX(const uint8_t *row, size_t bpr, size_t n_cols, const float *x) { \
    ACC sum = 0;                                                                               \
    for (size_t blk = 0; blk < bpr; blk++) {                                                   \
      const uint8_t *b = row + blk * 34;                                                       \
      float d = rd_f16(b);                                                                     \
      size_t io = blk * 32;                                                                    \
      for (int i = 0; i < 32; i++) {                                                           \
        size_t idx = io + (size_t)i;                                                           \
        if (idx < n_cols) {                                                                    \
          float w = (float)(int8_t)b[2 + i] * d;                                               \
          float p = w * x[idx];                                                                \
          sum += p;                                                                            \
        }                                                                                      \
      }                                                                                        \
    }                                                                                          \
    return (float)sum;                                                                         \
  }                                                                                            \
  /* reference/q4_k.rs:133-181 */                                                              \
  static float row_q4_k##SUFFIX(const uint8_t *row, size_t bpr, size_t n_cols, const float *x) { \
    ACC sum = 0;                                                                               \
    for (size_t blk = 0; blk < bpr; blk++) {                                                   \
      const uint8_t *b = row + blk * 144;                                                      \
      float d = rd_f16(b), dmin = rd_f16(b + 2);                                               \
      const uint8_t *qs = b + 16;                                                              \
      uint8_t sc[8], mn[8];                                                                    \
      decode_scales_mins(b + 4, sc, mn);                                                       \
      int is = 0;                                                                              \
      size_t qo = 0, wo = blk * 256;                                                           \
      for (int g = 0; g < 4; g++) {                                                            \
        float d1 = d * (float)sc[is], m1 = dmin * (float)mn[is];                               \
        float d2 = d * (float)sc[is + 1], m2 = dmin * (float)mn[is + 1];                       \
        for (int l = 0; l < 32; l++) {                                                         \
          size_t idx = wo + (size_t)l;                                                         \
          if (idx < n_cols) {                                                                  \
            float q = (float)(qs[qo + l] & 0x0F);                                              \
            float t = d1 * q;                                                                  \
            float w = t - m1;                                                                  \
            float p = w * x[idx];                                                              \
            sum += p;                                                                          \
          }                                                                                    \
        }                                                                                      \
        for (int l = 0; l < 32; l++) {                                                         \
          size_t idx = wo + 32 + (size_t)l;                                                    \
          if (idx < n_cols) {                                                                  \
            float q = (float)((qs[qo + l] >> 4) & 0x0F);                                       \
            float t = d2 * q;                                                                  \
            float w = t - m2;                                                                  \
            float p = w * x[idx];                                                              \
            sum += p;                                                                          \
          }                                                                                    \
        }                                                                                      \
        is += 2;                                                                               \
        qo += 32;                                                                              \
        wo += 64;                                                                              \
      }                                                                                        \
    }                                                                                          \
    return (float)sum;                                                                         \
  }                                                                                            \
  /* reference/q2_k.rs:84-166 */                                                               \
  static float row_q2_k##SUFFIX(const uint8_t *row, size_t bpr, size_t n_cols, const float *x) {\
    ACC sum = 0;                                                                               \
    for (size_t blk = 0; blk < bpr; blk++) {                                                   \
      const uint8_t *b = row + blk * 84;                                                       \
      const uint8_t *scales = b, *qs = b + 16;                                                 \
      float d = rd_f16(b + 80), dmin = rd_f16(b + 82);                                         \
      int is = 0;                                                                              \
      size_t qo = 0, wo = blk * 256;                                                           \
      for (int n = 0; n < 2; n++) {                                                            \
        for (int shift = 0; shift < 8; shift += 2) {                                           \
          for (int h = 0; h < 2; h++) {                                                        \
            uint8_t sb = scales[is++];                                                         \
            float dl = d * (float)(sb & 0x0F);                                                 \
            float ml = dmin * (float)(sb >> 4);                                                \
            for (int l = 0; l < 16; l++) {                                                     \
              size_t idx = wo + (size_t)l;                                                     \
              if (idx < n_cols) {                                                              \
                uint8_t q = (uint8_t)((qs[qo + 16 * h + l] >> shift) & 3);                     \
                float t = dl * (float)q;                                                       \
                float w = t - ml;                                                              \
                float p = w * x[idx];                                                          \
                sum += p;                                                                      \
              }                                                                                \
            }                                                                                  \
            wo += 16;                                                                          \
          }                                                                                    \
        }                                                                                      \
        qo += 32;                                                                              \
      }                                                                                        \
    }                                                                                          \
    return (float)sum;                                                                         \
  }                                                                                            \
  /* reference/q3_k.rs:123-199 */                                                              \
  static float row_q3_k##SUFFIX(const uint8_t *row, size_t bpr, size_t n_cols, const float *x) {\
    ACC sum = 0;                                                                               \
    for (size_t blk = 0; blk < bpr; blk++) {                                                   \
      const uint8_t *b = row + blk * 110;                                                      \
      const uint8_t *hmask = b, *qs = b + 32;                                                  \
      float d = rd_f16(b + 108);                                                               \
      float sc[16];                                                                            \
      decode_scales_q3_k(b + 96, sc);                                                          \
      int is = 0;                                                                              \
      size_t wo = blk * 256;                                                                   \
      uint8_t m = 1;                                                                           \
      for (int group = 0; group < 2; group++) {                                                \
        size_t qs_base = (size_t)group * 32;                                                   \
        for (int shift = 0; shift < 8; shift += 2) {                                           \
          for (int n = 0; n < 2; n++) {                                                        \
            float dl = d * sc[is++];                                                           \
            for (int l = 0; l < 16; l++) {                                                     \
              size_t idx = wo + (size_t)l;                                                     \
              if (idx < n_cols) {                                                              \
                int q_lo = (qs[qs_base + (size_t)n * 16 + l] >> shift) & 3;                    \
                int sub = (hmask[n * 16 + l] & m) ? 0 : 4;                                     \
                float w = dl * (float)(q_lo - sub);                                            \
                float p = w * x[idx];                                                          \
                sum += p;                                                                      \
              }                                                                                \
            }                                                                                  \
            wo += 16;                                                                          \
          }                                                                                    \
          m = (uint8_t)(m << 1);                                                               \
        }                                                                                      \
      }                                                                                        \
    }                                                                                          \
    return (float)sum;                                                                         \
  }                                                                                            \
  /* reference/q8_k.rs:52-101: the quants of a block are summed against x first, the block     \
   * scale applied once.  (The reference walks all 256 quants of every block; it is defined    \
   * only when n_cols is a multiple of 256, and columns beyond n_cols are skipped here.) */    \
  static float row_q8_k##SUFFIX(const uint8_t *row, size_t bpr, size_t n_cols, const float *x) {\
    ACC sum = 0;                                                                               \
    for (size_t blk = 0; blk < bpr; blk++) {                                                   \
      const uint8_t *b = row + blk * 292;                                                      \
      float d = rd_f32(b);                                                                     \
      ACC block_sum = 0;                                                                       \
      for (int i = 0; i < 256; i++) {                                                          \
        size_t idx = blk * 256 + (size_t)i;                                                    \
        if (idx < n_cols) {                                                                    \
          float p = (float)(int8_t)b[4 + i] * x[idx];                                          \
          block_sum += p;                                                                      \
        }                                                                                      \
      }                                                                                        \
      sum += (ACC)((ACC)d * block_sum);                                                        \
    }                                                                                          \
    return (float)sum;                                                                         \
  }                                                                                            \
  /* reference/q5_k.rs:137-189 */                                                              \
  static float row_q5_k##SUFFIX(const uint8_t *row, size_t bpr, size_t n_cols, const float *x) {\
    ACC sum = 0;                                                                               \
    for (size_t blk = 0; blk < bpr; blk++) {                                                   \
      const uint8_t *b = row + blk * 176;                                                      \
      float d = rd_f16(b), dmin = rd_f16(b + 2);                                               \
      const uint8_t *qh = b + 16, *qs = b + 48;                                                \
      uint8_t sc[8], mn[8];                                                                    \
      decode_scales_mins(b + 4, sc, mn);                                                       \
      int is = 0;                                                                              \
      size_t qo = 0, wo = blk * 256;                                                           \
      for (int g = 0; g < 4; g++) {                                                            \
        float d1 = d * (float)sc[is], m1 = dmin * (float)mn[is];                               \
        float d2 = d * (float)sc[is + 1], m2 = dmin * (float)mn[is + 1];                       \
        for (int l = 0; l < 32; l++) {                                                         \
          size_t idx = wo + (size_t)l;                                                         \
          if (idx < n_cols) {                                                                  \
            uint8_t hb = (uint8_t)((qh[l] >> g) & 1);                                          \
            float q = (float)(uint8_t)((qs[qo + l] & 0x0F) | (hb << 4));                       \
            float t = d1 * q;                                                                  \
            float w = t - m1;                                                                  \
            float p = w * x[idx];                                                              \
            sum += p;                                                                          \
          }                                                                                    \
        }                                                                                      \
        for (int l = 0; l < 32; l++) {                                                         \
          size_t idx = wo + 32 + (size_t)l;                                                    \
          if (idx < n_cols) {                                                                  \
            uint8_t hb = (uint8_t)((qh[l] >> (g + 4)) & 1);                                    \
            float q = (float)(uint8_t)(((qs[qo + l] >> 4) & 0x0F) | (hb << 4));                \
            float t = d2 * q;                                                                  \
            float w = t - m2;                                                                  \
            float p = w * x[idx];                                                              \
            sum += p;                                                                          \
          }                                                                                    \
        }                                                                                      \
        is += 2;                                                                               \
        qo += 32;                                                                              \
        wo += 64;                                                                              \
      }                                                                                        \
    }                                                                                          \
    return (float)sum;                                                                         \
  }                                                                                            \
  /* reference/q6_k.rs:106-169 */                                                              \
  static float row_q6_k##SUFFIX(const uint8_t *row, size_t bpr, size_t n_cols, const float *x) { \
    ACC sum = 0;                                                                               \
    for (size_t blk = 0; blk < bpr; blk++) {                                                   \
      const uint8_t *b = row + blk * 210;                                                      \
      const uint8_t *ql = b, *qh = b + 128, *scales = b + 192;                                 \
      float d = rd_f16(b + 208);                                                               \
      const float *inp = x + blk * 256;                                                        \
      size_t cib = n_cols - blk * 256 < 256 ? n_cols - blk * 256 : 256;                        \
      for (int g = 0; g < 2; g++) {                                                            \
        int ql_off = g * 64, qh_off = g * 32, sc_off = g * 8;                                  \
        size_t in_off = (size_t)g * 128;                                                       \
        for (int l = 0; l < 32; l++) {                                                         \
          int is = l / 16;                                                                     \
          int q1 = (int)(uint8_t)((ql[ql_off + l] & 0x0F) | ((qh[qh_off + l] & 3) << 4)) - 32; \
          int q2 = (int)(uint8_t)((ql[ql_off + l + 32] & 0x0F) |                               \
                                  (((qh[qh_off + l] >> 2) & 3) << 4)) - 32;                    \
          int q3 = (int)(uint8_t)((ql[ql_off + l] >> 4) | (((qh[qh_off + l] >> 4) & 3) << 4)) - 32; \
          int q4 = (int)(uint8_t)((ql[ql_off + l + 32] >> 4) |                                 \
                                  (((qh[qh_off + l] >> 6) & 3) << 4)) - 32;                    \
          float s0 = d * (float)(int8_t)scales[sc_off + is];                                   \
          float s1 = d * (float)(int8_t)scales[sc_off + is + 2];                               \
          float s2 = d * (float)(int8_t)scales[sc_off + is + 4];                               \
          float s3 = d * (float)(int8_t)scales[sc_off + is + 6];                               \
          size_t c0 = in_off + (size_t)l, c1 = c0 + 32, c2 = c0 + 64, c3 = c0 + 96;            \
          if (c0 < cib) {                                                                      \
            float w = s0 * (float)q1;                                                          \
            float p = w * inp[c0];                                                             \
            sum += p;                                                                          \
          }                                                                                    \
          if (c1 < cib) {                                                                      \
            float w = s1 * (float)q2;                                                          \
            float p = w * inp[c1];                                                             \
            sum += p;                                                                          \
          }                                                                                    \
          if (c2 < cib) {                                                                      \
            float w = s2 * (float)q3;                                                          \
            float p = w * inp[c2];                                                             \
            sum += p;                                                                          \
          }                                                                                    \
          if (c3 < cib) {                                                                      \
            float w = s3 * (float)q4;                                                          \
            float p = w * inp[c3];                                                             \
            sum += p;                                                                          \
          }                                                                                    \
        }                                                                                      \
      }                                                                                        \
    }                                                                                          \
    return (float)sum;                                                                         \
  }                                                                                            \
  /* reference/iq4_xs.rs:128-165 — note the order (K * scale) * x. */                          \
  static float row_iq4_xs##SUFFIX(const uint8_t *row, size_t bpr, size_t n_cols,               \
                                  const float *x) {                                            \
    ACC sum = 0;                                                                               \
    for (size_t blk = 0; blk < bpr; blk++) {                                                   \
      const uint8_t *b = row + blk * 136;                                                      \
      float d = rd_f16(b);                                                                     \
      uint16_t sh = (uint16_t)(b[2] | (b[3] << 8));                                            \
      const uint8_t *sl = b + 4, *nib = b + 8;                                                 \
      for (int sub = 0; sub < 8; sub++) {                                                      \
        float scale = d * (float)unpack_sub_scale(sh, sl, sub);                                \
        size_t co = blk * 256 + (size_t)sub * 32;                                              \
        for (int i = 0; i < 16; i++) {                                                         \
          uint8_t byte = nib[sub * 16 + i];                                                    \
          size_t idx = co + (size_t)i * 2;                                                     \
          if (idx + 1 < n_cols) {                                                              \
            float w0 = (float)KVALUES_IQ4NL[byte & 0x0F] * scale;                              \
            float w1 = (float)KVALUES_IQ4NL[(byte >> 4) & 0x0F] * scale;                       \
            float p0 = w0 * x[idx], p1 = w1 * x[idx + 1];                                      \
            sum += p0;                                                                         \
            sum += p1;                                                                         \
          } else if (idx < n_cols) {                                                           \
            float w0 = (float)KVALUES_IQ4NL[byte & 0x0F] * scale;                              \
            float p0 = w0 * x[idx];                                                            \
            sum += p0;                                                                         \
          }                                                                                    \
        }                                                                                      \
      }                                                                                        \
    }                                                                                          \
    return (float)sum;                                                                         \
  }

DEFINE_ROW_DOTS(_f32, float)
DEFINE_ROW_DOTS(_f64, double)

typedef float (*row_fn)(const uint8_t *, size_t, size_t, const float *);

static row_fn pick_row(int type, int wide) {
  switch (type) {
    case T_Q4_0:
      return wide ? row_q4_0_f64 : row_q4_0_f32;
    case T_Q8_0:
      return wide ? row_q8_0_f64 : row_q8_0_f32;
    case T_Q4_K:
      return wide ? row_q4_k_f64 : row_q4_k_f32;
    case T_Q5_K:
      return wide ? row_q5_k_f64 : row_q5_k_f32;
    case T_Q2_K:
      return wide ? row_q2_k_f64 : row_q2_k_f32;
    case T_Q3_K:
      return wide ? row_q3_k_f64 : row_q3_k_f32;
    case T_Q8_K:
      return wide ? row_q8_k_f64 : row_q8_k_f32;
    case T_Q6_K:
      return wide ? row_q6_k_f64 : row_q6_k_f32;
    case T_IQ4_XS:
      return wide ? row_iq4_xs_f64 : row_iq4_xs_f32;
    default:
      return NULL;
  }
}

static int gemv_impl(int type, int wide, const uint8_t *w, size_t w_len, size_t n_rows,
                     size_t n_cols, const float *x, size_t x_len, float *y, size_t y_len) {
  row_fn f = pick_row(type, wide);
  if (!f) return QK_UNSUPPORTED_TYPE;
  if (x_len < n_cols) return QK_DIMENSION_MISMATCH;
  if (y_len < n_rows) return QK_DIMENSION_MISMATCH;
  size_t bs = qk_oracle_block_size(type), bb = qk_oracle_block_bytes(type);
  size_t bpr = (n_cols + bs - 1) / bs, row_bytes = bpr * bb;
  if (w_len < n_rows * row_bytes) return QK_BUFFER_TOO_SMALL;
  for (size_t r = 0; r < n_rows; r++) y[r] = f(w + r * row_bytes, bpr, n_cols, x);
  return QK_OK;
}

/* `gemv`: output is overwritten (reference/q4_k.rs:104-184 and siblings). */
int qk_oracle_gemv(int type, const uint8_t *w, size_t w_len, size_t n_rows, size_t n_cols,
                   const float *x, size_t x_len, float *y, size_t y_len) {
  return gemv_impl(type, 0, w, w_len, n_rows, n_cols, x, x_len, y, y_len);
}

/* Same products, running sum held in f64: the error-budget companion. */
int qk_oracle_gemv_f64(int type, const uint8_t *w, size_t w_len, size_t n_rows, size_t n_cols,
                       const float *x, size_t x_len, float *y, size_t y_len) {
  return gemv_impl(type, 1, w, w_len, n_rows, n_cols, x, x_len, y, y_len);
}

/* `gemm` = M independent GEMVs; input [m x k], output [m x n], row-major
 * (reference/q4_k.rs:186-201, identical in every format). */
int qk_oracle_gemm(int type, const uint8_t *w, size_t w_len, const float *x, float *y, size_t m,
                   size_t n, size_t k) {
  for (size_t r = 0; r < m; r++) {
    int st = gemv_impl(type, 0, w, w_len, n, k, x + r * k, k, y + r * n, n);
    if (st) return st;
  }
  return QK_OK;
}

int qk_oracle_gemm_f64(int type, const uint8_t *w, size_t w_len, const float *x, float *y,
                       size_t m, size_t n, size_t k) {
  for (size_t r = 0; r < m; r++) {
    int st = gemv_impl(type, 1, w, w_len, n, k, x + r * k, k, y + r * n, n);
    if (st) return st;
  }
  return QK_OK;
}

/* ----------------------------- matvec_q8_fused ----------------------------- */
/* All variants ACCUMULATE into out (traits.rs:89-173). */

/* reference/q4_0.rs:159-232 (free function matvec_q8_fused_reference):
 * sum += (((q * d_w) * a) * d_a), left to right. */
static float fused_row_q4_0(const uint8_t *row, size_t bpr, size_t n_cols, const uint8_t *acts) {
  float sum = 0.0f;
  for (size_t blk = 0; blk < bpr; blk++) {
    const uint8_t *wb = row + blk * 18;
    float d_w = rd_f16(wb);
    const uint8_t *ab = acts + blk * Q8_0_BLOCK_BYTES;
    float d_a = rd_f16(ab);
    const uint8_t *q8 = ab + 2;
    size_t wo = blk * 32;
    size_t valid = n_cols - wo < 32 ? n_cols - wo : 32;
    for (size_t i = 0; i < valid / 2; i++) {
      uint8_t byte = wb[2 + i];
      int q_lo = (int)(byte & 0x0F) - 8, q_hi = (int)((byte >> 4) & 0x0F) - 8;
      float a_lo = (float)(int8_t)q8[i * 2], a_hi = (float)(int8_t)q8[i * 2 + 1];
      float t0 = (float)q_lo * d_w;
      t0 = t0 * a_lo;
      t0 = t0 * d_a;
      sum += t0;
      float t1 = (float)q_hi * d_w;
      t1 = t1 * a_hi;
      t1 = t1 * d_a;
      sum += t1;
    }
    if (valid % 2 == 1) {
      size_t i = valid / 2;
      uint8_t byte = wb[2 + i];
      int q_lo = (int)(byte & 0x0F) - 8;
      float a_lo = (float)(int8_t)q8[i * 2];
      float t0 = (float)q_lo * d_w;
      t0 = t0 * a_lo;
      t0 = t0 * d_a;
      sum += t0;
    }
  }
  return sum;
}

/* traits.rs:89-173, the trait default, which Q8_0Ref inherits: dequantise the
 * weight block and the activation block to f32 scratch, then dot. */
static float fused_row_default32(int type, const uint8_t *row, size_t bpr, size_t n_cols,
                                 const uint8_t *acts) {
  size_t bb = qk_oracle_block_bytes(type);
  float sum = 0.0f, ws[32], as[32];
  for (size_t blk = 0; blk < bpr; blk++) {
    qk_oracle_dequant_block(type, row + blk * bb, bb, ws, 32);
    const uint8_t *ab = acts + blk * Q8_0_BLOCK_BYTES;
    float d_a = rd_f16(ab);
    size_t ws0 = blk * 32;
    size_t we = ws0 + 32 < n_cols ? ws0 + 32 : n_cols;
    size_t valid = we - ws0;
    for (size_t i = 0; i < valid; i++) as[i] = (float)(int8_t)ab[2 + i] * d_a;
    for (size_t i = 0; i < valid; i++) {
      float p = ws[i] * as[i];
      sum += p;
    }
  }
  return sum;
}

/* reference/q4_k.rs:218-333 */
static float fused_row_q4_k(const uint8_t *row, size_t bpr, size_t n_cols, const uint8_t *acts) {
  float sum = 0.0f;
  for (size_t blk = 0; blk < bpr; blk++) {
    const uint8_t *b = row + blk * 144;
    float d = rd_f16(b), dmin = rd_f16(b + 2);
    uint8_t sc[8], mn[8];
    decode_scales_mins(b + 4, sc, mn);
    const uint8_t *qs = b + 16;
    size_t is = 0, qo = 0, wo = blk * 256;
    for (int g = 0; g < 4; g++) {
      const uint8_t *alo = acts + (blk * 8 + is) * Q8_0_BLOCK_BYTES;
      float d_a_lo = rd_f16(alo);
      float da_lo = d * (float)sc[is], m_lo = dmin * (float)mn[is];
      const uint8_t *ahi = acts + (blk * 8 + is + 1) * Q8_0_BLOCK_BYTES;
      float d_a_hi = rd_f16(ahi);
      float da_hi = d * (float)sc[is + 1], m_hi = dmin * (float)mn[is + 1];
      float dot_lo = 0.0f, sum_a_lo = 0.0f;
      for (int l = 0; l < 32; l++) {
        if (wo + (size_t)l < n_cols) {
          float q_w = (float)(qs[qo + l] & 0x0F), q_a = (float)(int8_t)alo[2 + l];
          float p = q_w * q_a;
          dot_lo += p;
          sum_a_lo += q_a;
        }
      }
      {
        float a = da_lo * dot_lo, c = m_lo * sum_a_lo;
        float t = a - c;
        t = t * d_a_lo;
        sum += t;
      }
      float dot_hi = 0.0f, sum_a_hi = 0.0f;
      for (int l = 0; l < 32; l++) {
        if (wo + 32 + (size_t)l < n_cols) {
          float q_w = (float)((qs[qo + l] >> 4) & 0x0F), q_a = (float)(int8_t)ahi[2 + l];
          float p = q_w * q_a;
          dot_hi += p;
          sum_a_hi += q_a;
        }
      }
      {
        float a = da_hi * dot_hi, c = m_hi * sum_a_hi;
        float t = a - c;
        t = t * d_a_hi;
        sum += t;
      }
      is += 2;
      qo += 32;
      wo += 64;
    }
  }
  return sum;
}

/* reference/q2_k.rs:187-297: per 16-weight sub-block (dl * dot - ml * sum_a) * d_a, sums in f32. */
static float fused_row_q2_k(const uint8_t *row, size_t bpr, size_t n_cols, const uint8_t *acts) {
  float sum = 0.0f;
  for (size_t blk = 0; blk < bpr; blk++) {
    const uint8_t *b = row + blk * 84;
    const uint8_t *scales = b, *qs = b + 16;
    float d = rd_f16(b + 80), dmin = rd_f16(b + 82);
    size_t left = n_cols > blk * 256 ? n_cols - blk * 256 : 0;  /* n_cols.saturating_sub(blk * 256) */
    int is = 0;
    size_t qo = 0, col_off = 0;
    for (int group = 0; group < 2; group++) {
      for (int shift = 0; shift < 8; shift += 2) {
        for (int h = 0; h < 2; h++) {
          uint8_t sb = scales[is++];
          float dl = d * (float)(sb & 0x0F);
          float ml = dmin * (float)(sb >> 4);
          const uint8_t *a = acts + (blk * 8 + col_off / 32) * Q8_0_BLOCK_BYTES;
          size_t lane = col_off % 32;
          float d_a = rd_f16(a);
          float dot = 0.0f, sum_a = 0.0f;
          for (int l = 0; l < 16; l++) {
            if (col_off + (size_t)l < left) {
              float q2 = (float)(uint8_t)((qs[qo + 16 * h + l] >> shift) & 3);
              float q_a = (float)(int8_t)a[2 + lane + l];
              float p = q2 * q_a;
              dot += p;
              sum_a += q_a;
            }
          }
          float t1 = dl * dot, t2 = ml * sum_a;
          float t = t1 - t2;
          t = t * d_a;
          sum += t;
          col_off += 16;
        }
      }
      qo += 32;
    }
  }
  return sum;
}

/* reference/q3_k.rs:217-336: per 16-weight sub-block dl * dot * d_a, sums in f32. */
static float fused_row_q3_k(const uint8_t *row, size_t bpr, size_t n_cols, const uint8_t *acts) {
  float sum = 0.0f;
  for (size_t blk = 0; blk < bpr; blk++) {
    const uint8_t *b = row + blk * 110;
    const uint8_t *hmask = b, *qs = b + 32;
    float d = rd_f16(b + 108);
    float sc[16];
    decode_scales_q3_k(b + 96, sc);
    size_t left = n_cols > blk * 256 ? n_cols - blk * 256 : 0;
    if (left > 256) left = 256;
    int is = 0;
    size_t col_off = 0;
    uint8_t m = 1;
    for (int group = 0; group < 2; group++) {
      size_t qs_base = (size_t)group * 32;
      for (int shift = 0; shift < 8; shift += 2) {
        for (int n = 0; n < 2; n++) {
          float dl = d * sc[is++];
          const uint8_t *a = acts + (blk * 8 + col_off / 32) * Q8_0_BLOCK_BYTES;
          size_t lane = col_off % 32;
          float d_a = rd_f16(a);
          float dot = 0.0f;
          for (int l = 0; l < 16; l++) {
            if (col_off + (size_t)l < left) {
              int q_lo = (qs[qs_base + (size_t)n * 16 + l] >> shift) & 3;
              int sub = (hmask[n * 16 + l] & m) ? 0 : 4;
              float q3 = (float)(q_lo - sub);
              float q_a = (float)(int8_t)a[2 + lane + l];
              float p = q3 * q_a;
              dot += p;
            }
          }
          float t = dl * dot;
          t = t * d_a;
          sum += t;
          col_off += 16;
        }
        m = (uint8_t)(m << 1);
      }
    }
  }
  return sum;
}

/* Q8_K has no override of matvec_q8_fused, and the trait default (traits.rs:89-173) pairs one
 * weight block with one 32-value activation block, which for a 256-weight block reads past
 * that block (a panic in the reference): undefined there, PARITY UNPINNED.  Here, by analogy
 * with the default's arithmetic: eight activation blocks per weight block, the dequantised
 * weight times the dequantised activation (q_a * d_a), summed in f32 in column order. */
static float fused_row_q8_k(const uint8_t *row, size_t bpr, size_t n_cols, const uint8_t *acts) {
  float sum = 0.0f;
  float w[256];
  for (size_t blk = 0; blk < bpr; blk++) {
    dq_q8_k(row + blk * 292, w);
    for (int i = 0; i < 256; i++) {
      size_t idx = blk * 256 + (size_t)i;
      if (idx < n_cols) {
        const uint8_t *a = acts + (idx / 32) * Q8_0_BLOCK_BYTES;
        float av = (float)(int8_t)a[2 + idx % 32] * rd_f16(a);
        float p = w[i] * av;
        sum += p;
      }
    }
  }
  return sum;
}

/* reference/q5_k.rs:236-347: per sub-block (da * dot - m * sum_a) * d_a, sums in f32. */
static float fused_row_q5_k(const uint8_t *row, size_t bpr, size_t n_cols, const uint8_t *acts) {
  float sum = 0.0f;
  for (size_t blk = 0; blk < bpr; blk++) {
    const uint8_t *b = row + blk * 176;
    float d = rd_f16(b), dmin = rd_f16(b + 2);
    uint8_t sc[8], mn[8];
    decode_scales_mins(b + 4, sc, mn);
    const uint8_t *qh = b + 16, *qs = b + 48;
    size_t is = 0, qo = 0, wo = blk * 256;
    for (int g = 0; g < 4; g++) {
      const uint8_t *alo = acts + (blk * 8 + is) * Q8_0_BLOCK_BYTES;
      float d_a_lo = rd_f16(alo);
      float da_lo = d * (float)sc[is], m_lo = dmin * (float)mn[is];
      const uint8_t *ahi = acts + (blk * 8 + is + 1) * Q8_0_BLOCK_BYTES;
      float d_a_hi = rd_f16(ahi);
      float da_hi = d * (float)sc[is + 1], m_hi = dmin * (float)mn[is + 1];
      float dot_lo = 0.0f, sum_a_lo = 0.0f;
      for (int l = 0; l < 32; l++) {
        if (wo + (size_t)l < n_cols) {
          uint8_t hb = (uint8_t)((qh[l] >> g) & 1);
          float q_w = (float)(uint8_t)((qs[qo + l] & 0x0F) | (hb << 4)), q_a = (float)(int8_t)alo[2 + l];
          float p = q_w * q_a;
          dot_lo += p;
          sum_a_lo += q_a;
        }
      }
      {
        float a = da_lo * dot_lo, c = m_lo * sum_a_lo;
        float t = a - c;
        t = t * d_a_lo;
        sum += t;
      }
      float dot_hi = 0.0f, sum_a_hi = 0.0f;
      for (int l = 0; l < 32; l++) {
        if (wo + 32 + (size_t)l < n_cols) {
          uint8_t hb = (uint8_t)((qh[l] >> (g + 4)) & 1);
          float q_w = (float)(uint8_t)(((qs[qo + l] >> 4) & 0x0F) | (hb << 4)), q_a = (float)(int8_t)ahi[2 + l];
          float p = q_w * q_a;
          dot_hi += p;
          sum_a_hi += q_a;
        }
      }
      {
        float a = da_hi * dot_hi, c = m_hi * sum_a_hi;
        float t = a - c;
        t = t * d_a_hi;
        sum += t;
      }
      is += 2;
      qo += 32;
      wo += 64;
    }
  }
  return sum;
}

/* reference/q6_k.rs:212-354: sum += (s * q) * (d_a * q_a). */
static float fused_row_q6_k(const uint8_t *row, size_t bpr, size_t n_cols, const uint8_t *acts) {
  float sum = 0.0f;
  for (size_t blk = 0; blk < bpr; blk++) {
    const uint8_t *b = row + blk * 210;
    const uint8_t *ql = b, *qh = b + 128, *scales = b + 192;
    float d = rd_f16(b + 208);
    size_t io = blk * 256;
    size_t cib = n_cols - io < 256 ? n_cols - io : 256;
    for (int g = 0; g < 2; g++) {
      int ql_off = g * 64, qh_off = g * 32, sc_off = g * 8;
      size_t in_off = (size_t)g * 128;
      for (int l = 0; l < 32; l++) {
        int is = l / 16;
        int q[4];
        q[0] = (int)(uint8_t)((ql[ql_off + l] & 0x0F) | ((qh[qh_off + l] & 3) << 4)) - 32;
        q[1] = (int)(uint8_t)((ql[ql_off + l + 32] & 0x0F) | (((qh[qh_off + l] >> 2) & 3) << 4)) - 32;
        q[2] = (int)(uint8_t)((ql[ql_off + l] >> 4) | (((qh[qh_off + l] >> 4) & 3) << 4)) - 32;
        q[3] = (int)(uint8_t)((ql[ql_off + l + 32] >> 4) | (((qh[qh_off + l] >> 6) & 3) << 4)) - 32;
        for (int k = 0; k < 4; k++) {
          float s = d * (float)(int8_t)scales[sc_off + is + 2 * k];
          size_t col = in_off + (size_t)l + 32 * (size_t)k;
          if (col < cib) {
            const uint8_t *ab = acts + (blk * 8 + col / 32) * Q8_0_BLOCK_BYTES;
            float d_a = rd_f16(ab);
            float q_a = (float)(int8_t)ab[2 + col % 32];
            float a = d_a * q_a;
            float w = s * (float)q[k];
            float p = w * a;
            sum += p;
          }
        }
      }
    }
  }
  return sum;
}

/* No tier of the reference defines IQ4_XS x Q8_0 (the trait default would
 * overrun its 32-float scratch with a 256-element block).  Defined here by
 * analogy with Q4_K: one super-block pairs with 8 Q8_0 blocks and the dot is
 * taken over dequantised f32 values in column order.  PARITY UNPINNED. */
static float fused_row_iq4_xs(const uint8_t *row, size_t bpr, size_t n_cols,
                              const uint8_t *acts) {
  float sum = 0.0f, ws[256];
  for (size_t blk = 0; blk < bpr; blk++) {
    dq_iq4_xs(row + blk * 136, ws);
    size_t io = blk * 256;
    size_t cib = n_cols - io < 256 ? n_cols - io : 256;
    for (size_t c = 0; c < cib; c++) {
      const uint8_t *ab = acts + (blk * 8 + c / 32) * Q8_0_BLOCK_BYTES;
      float a = (float)(int8_t)ab[2 + c % 32] * rd_f16(ab);
      float p = ws[c] * a;
      sum += p;
    }
  }
  return sum;
}

int qk_oracle_matvec_q8_fused(int type, const uint8_t *w, size_t w_len, const uint8_t *acts,
                              size_t acts_len, float *out, size_t out_len, size_t n_rows,
                              size_t n_cols) {
  size_t bs = qk_oracle_block_size(type), bb = qk_oracle_block_bytes(type);
  if (bs == 0) return QK_UNSUPPORTED_TYPE;
  if (out_len < n_rows) return QK_DIMENSION_MISMATCH;
  size_t bpr = (n_cols + bs - 1) / bs, row_bytes = bpr * bb;
  size_t acts_needed = bpr * (bs / 32) * Q8_0_BLOCK_BYTES;
  if (w_len < n_rows * row_bytes) return QK_BUFFER_TOO_SMALL;
  if (acts_len < acts_needed) return QK_BUFFER_TOO_SMALL;
  for (size_t r = 0; r < n_rows; r++) {
    const uint8_t *row = w + r * row_bytes;
    float s;
    switch (type) {
      case T_Q4_0:
        s = fused_row_q4_0(row, bpr, n_cols, acts);
        break;
      case T_Q8_0:
        s = fused_row_default32(type, row, bpr, n_cols, acts);
        break;
      case T_Q4_K:
        s = fused_row_q4_k(row, bpr, n_cols, acts);
        break;
      case T_Q5_K:
        s = fused_row_q5_k(row, bpr, n_cols, acts);
        break;
      case T_Q2_K:
        s = fused_row_q2_k(row, bpr, n_cols, acts);
        break;
      case T_Q3_K:
        s = fused_row_q3_k(row, bpr, n_cols, acts);
        break;
      case T_Q8_K:
        s = fused_row_q8_k(row, bpr, n_cols, acts);
        break;
      case T_Q6_K:
        s = fused_row_q6_k(row, bpr, n_cols, acts);
        break;
      default:
        s = fused_row_iq4_xs(row, bpr, n_cols, acts);
        break;
    }
    out[r] += s;
  }
  return QK_OK;
}

/* ------------------------------ dense feed-forward block ------------------------------ */
/* swiglu_inplace, crates/oxillama-arch/src/common/swiglu.rs:15-21 */
void qk_oracle_swiglu_inplace(float *gate, const float *up, size_t n) {
  for (size_t i = 0; i < n; i++) {
    float e = expf(-gate[i]);
    float den = 1.0f + e;
    float sigmoid = 1.0f / den;
    float t = gate[i] * sigmoid;
    gate[i] = t * up[i];
  }
}

/* feed_forward, dense branch (crates/oxillama-arch/src/llama/model.rs:281-310), for m rows of x:
 * gate = gate_proj(x); up = up_proj(x); swiglu_inplace(gate, up); y = down_proj(gate). */
int qk_oracle_ffn(int type_gu, const uint8_t *gate, const uint8_t *up, size_t gu_len, int type_d,
                  const uint8_t *down, size_t d_len, const float *x, float *y, size_t m, size_t hidden,
                  size_t inter, size_t out_rows, float *scratch /* 2 * inter floats */) {
  for (size_t i = 0; i < m; i++) {
    int st = qk_oracle_gemv(type_gu, gate, gu_len, inter, hidden, x + i * hidden, hidden, scratch, inter);
    if (st) return st;
    st = qk_oracle_gemv(type_gu, up, gu_len, inter, hidden, x + i * hidden, hidden, scratch + inter, inter);
    if (st) return st;
    qk_oracle_swiglu_inplace(scratch, scratch + inter, inter);
    st = qk_oracle_gemv(type_d, down, d_len, out_rows, inter, scratch, inter, y + i * out_rows, out_rows);
    if (st) return st;
  }
  return QK_OK;
}

/* ---------------------------- Q8_0 activation encoder ---------------------------- */
/* quantize.rs:58-75,190-210.  `q` uses the f32 scale; the stored scale is its
 * f16 rounding.  Rust's f32::round is round-half-away-from-zero (roundf); the
 * `as i32` cast saturates and maps NaN to 0. */
int qk_oracle_quantize_q8_0(const float *x, size_t n, uint8_t *out) {
  if (n % 32 != 0) return QK_DIMENSION_MISMATCH;
  for (size_t b = 0; b < n / 32; b++) {
    const float *v = x + b * 32;
    float amax = 0.0f;
    for (int i = 0; i < 32; i++) {
      float a = fabsf(v[i]);
      /* f32::max: returns the non-NaN operand */
      if (a > amax || amax != amax) amax = a;
    }
    float d = amax / 127.0f;
    float id = d != 0.0f ? 1.0f / d : 0.0f;
    uint16_t h = qk_oracle_f32_to_f16(d);
    uint8_t *o = out + b * 34;
    o[0] = (uint8_t)(h & 0xFF);
    o[1] = (uint8_t)(h >> 8);
    for (int i = 0; i < 32; i++) {
      float r = roundf(v[i] * id);
      int q;
      if (r != r)
        q = 0;
      else if (r >= 2147483648.0f)
        q = 2147483647;
      else if (r <= -2147483648.0f)
        q = -2147483647 - 1;
      else
        q = (int)r;
      if (q < -128) q = -128;
      if (q > 127) q = 127;
      o[2 + i] = (uint8_t)(int8_t)q;
    }
  }
  return QK_OK;
}

/* ------------------------------------ MoE ------------------------------------ */
/* crates/oxillama-arch/src/common/moe.rs:75-126 (Expert::forward) and
 * :184-258 (MoeFfn::forward), on f32 expert weights obtained by the bit-exact
 * block dequant above.  Dots are sequential f32 sums of separately rounded
 * products (`iter().map(|(w,x)| w*x).sum::<f32>()`).  expf stands in for
 * Rust's f32::exp; both are libm-grade, not bit-pinned.
 *
 * The router is given as precomputed logits [tokens x n_exp] (the benchmark
 * configuration draws them directly); everything from the softmax on follows
 * the reference.  Ties in the descending sort keep the lower index first. */

static float dot_seq(const float *a, const float *b, size_t n) {
  float s = 0.0f;
  for (size_t i = 0; i < n; i++) {
    float p = a[i] * b[i];
    s += p;
  }
  return s;
}

/* Routing only: top_k expert ids and renormalised weights per token. */
void qk_oracle_moe_route(const float *logits, size_t tokens, size_t n_exp, size_t top_k,
                         int32_t *ids, float *wts) {
  size_t ek = top_k < n_exp ? top_k : n_exp;
  float *ev = (float *)malloc(n_exp * sizeof(float));
  size_t *idx = (size_t *)malloc(n_exp * sizeof(size_t));
  for (size_t t = 0; t < tokens; t++) {
    const float *l = logits + t * n_exp;
    float mx = -INFINITY;
    for (size_t i = 0; i < n_exp; i++) mx = fmaxf(mx, l[i]);
    float es = 0.0f;
    for (size_t i = 0; i < n_exp; i++) {
      ev[i] = expf(l[i] - mx);
      es += ev[i];
    }
    if (es > 0.0f) {
      for (size_t i = 0; i < n_exp; i++) ev[i] /= es;
    } else {
      for (size_t i = 0; i < n_exp; i++) ev[i] = 1.0f / (float)n_exp;
    }
    for (size_t i = 0; i < n_exp; i++) idx[i] = i;
    for (size_t i = 1; i < n_exp; i++) { /* stable insertion sort, descending */
      size_t v = idx[i], j = i;
      while (j > 0 && ev[idx[j - 1]] < ev[v]) {
        idx[j] = idx[j - 1];
        j--;
      }
      idx[j] = v;
    }
    float ssum = 0.0f;
    for (size_t k = 0; k < ek; k++) ssum += ev[idx[k]];
    for (size_t k = 0; k < ek; k++) {
      ids[t * top_k + k] = (int32_t)idx[k];
      wts[t * top_k + k] = ssum > 1e-9f ? ev[idx[k]] / ssum : 1.0f / (float)ek;
    }
  }
  free(ev);
  free(idx);
}

/* gate/up: [n_exp][inter x hidden] f32, down: [n_exp][hidden x inter] f32.
 * token_begin/token_end select a token range so a caller can bound the work. */
int qk_oracle_moe_ffn_f32(const float *gate, const float *up, const float *down,
                          const float *logits, const float *x, float *y, size_t tokens,
                          size_t n_exp, size_t top_k, size_t hidden, size_t inter,
                          size_t token_begin, size_t token_end) {
  size_t ek = top_k < n_exp ? top_k : n_exp;
  int32_t *ids = (int32_t *)malloc(tokens * top_k * sizeof(int32_t));
  float *wts = (float *)malloc(tokens * top_k * sizeof(float));
  float *gv = (float *)malloc(inter * sizeof(float));
  float *uv = (float *)malloc(inter * sizeof(float));
  float *eo = (float *)malloc(hidden * sizeof(float));
  qk_oracle_moe_route(logits, tokens, n_exp, top_k, ids, wts);
  for (size_t t = token_begin; t < token_end && t < tokens; t++) {
    const float *in = x + t * hidden;
    float *out = y + t * hidden;
    for (size_t i = 0; i < hidden; i++) out[i] = 0.0f;
    for (size_t k = 0; k < ek; k++) {
      size_t e = (size_t)ids[t * top_k + k];
      float wgt = wts[t * top_k + k];
      const float *G = gate + e * inter * hidden, *U = up + e * inter * hidden;
      const float *D = down + e * hidden * inter;
      for (size_t i = 0; i < inter; i++) gv[i] = dot_seq(G + i * hidden, in, hidden);
      for (size_t i = 0; i < inter; i++) {
        float sig = 1.0f / (1.0f + expf(-gv[i]));
        gv[i] *= sig;
      }
      for (size_t i = 0; i < inter; i++) uv[i] = dot_seq(U + i * hidden, in, hidden);
      for (size_t i = 0; i < inter; i++) uv[i] *= gv[i];
      for (size_t i = 0; i < hidden; i++) eo[i] = dot_seq(D + i * inter, uv, inter);
      for (size_t i = 0; i < hidden; i++) {
        float p = wgt * eo[i];
        out[i] += p;
      }
    }
  }
  free(ids);
  free(wts);
  free(gv);
  free(uv);
  free(eo);
  return QK_OK;
}
