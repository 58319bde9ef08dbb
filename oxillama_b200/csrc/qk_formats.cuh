// Per-format element decode, bit-exact to the scalar reference kernels.
//
// Every product and difference is formed with an explicit round-to-nearest
// intrinsic (__fmul_rn / __fsub_rn) so that the compiler can never contract
// a*b-c into one FMA: the reference's Rust rounds the product first
// (e.g. reference/q4_k.rs:79-93: `d1 * q - m1` is two roundings).
#pragma once
#include "qk_layout.cuh"

__device__ __forceinline__ float qk_h2f(const uint8_t *p) {
  return __half2float(__ushort_as_half(*reinterpret_cast<const unsigned short *>(p)));
}

// reference/iq_shared.rs:16-18
static __device__ __constant__ int8_t QK_KVALUES_IQ4NL[16] = {-127, -104, -83, -65, -49, -35, -22, -10,
                                                       1,    13,   25,  38,  53,  69,  89,  113};

// reference/q4_k.rs:27-49: 6-bit scale and min of sub-block j from the 12 packed bytes.
__device__ __forceinline__ void qk_q4k_scale_min(const uint8_t *s, int j, int &sc, int &mn) {
  if (j < 4) {
    sc = s[j] & 0x3F;
    mn = s[j + 4] & 0x3F;
  } else {
    sc = (s[j + 4] & 0x0F) | ((s[j - 4] >> 6) << 4);
    mn = (s[j + 4] >> 4) | ((s[j] >> 6) << 4);
  }
}

// Weight (row, col) of a tiled matrix as the reference's dequant_block gives it.
// `base` is the tiled buffer; col < blocks_per_row * block_size.
__device__ __forceinline__ float qk_dequant_elem(const QkLayout &L, const uint8_t *base,
                                                 uint32_t row, uint32_t col) {
  uint32_t blk = col / L.bs, i = col % L.bs;
  auto at = [&](int p, uint32_t o) { return base + qk_byte_offset(L, row, blk, p, o); };
  switch (L.type) {
    case QK_T_Q4_0: {  // reference/q4_0.rs:36-46
      float d = qk_h2f(at(1, 0));
      uint8_t byte = *at(0, i >> 1);
      int q = (int)((i & 1) ? (byte >> 4) : (byte & 0x0F)) - 8;
      return __fmul_rn((float)q, d);
    }
    case QK_T_Q8_0: {  // reference/q8_0.rs:36-41
      float d = qk_h2f(at(1, 0));
      return __fmul_rn((float)(int8_t)*at(0, i), d);
    }
    case QK_T_Q4_K: {  // reference/q4_k.rs:66-99
      const uint8_t *h = at(0, 0);
      float d = qk_h2f(h), dmin = qk_h2f(h + 2);
      int sub = i >> 5, g = i >> 6, l = i & 31;
      uint8_t byte = *at(1, 32 * g + l);
      int q = (sub & 1) ? (byte >> 4) : (byte & 0x0F);
      int sc, mn;
      qk_q4k_scale_min(h + 4, sub, sc, mn);
      float d1 = __fmul_rn(d, (float)sc), m1 = __fmul_rn(dmin, (float)mn);
      return __fsub_rn(__fmul_rn(d1, (float)q), m1);
    }
    case QK_T_Q5_K: {  // reference/q5_k.rs:66-108: Q4_K plus a fifth bit from qh (bit g for the low-nibble
                       // quant of group g, bit g + 4 for the high-nibble one)
      const uint8_t *h = at(0, 0);
      float d = qk_h2f(h), dmin = qk_h2f(h + 2);
      int sub = i >> 5, g = i >> 6, l = i & 31;
      uint8_t byte = *at(2, 32 * g + l), hb = *at(1, l);
      int q = (sub & 1) ? ((byte >> 4) | (((hb >> (g + 4)) & 1) << 4)) : ((byte & 0x0F) | (((hb >> g) & 1) << 4));
      int sc, mn;
      qk_q4k_scale_min(h + 4, sub, sc, mn);
      float d1 = __fmul_rn(d, (float)sc), m1 = __fmul_rn(dmin, (float)mn);
      return __fsub_rn(__fmul_rn(d1, (float)q), m1);
    }
    case QK_T_Q2_K: {  // reference/q2_k.rs:42-79: sub-block is = 8 n + 2 j + h of 16 weights, shift 2 j
      const uint8_t *dm = at(2, 0);
      float d = qk_h2f(dm), dmin = qk_h2f(dm + 2);
      int n = i >> 7, r = i & 127, j = r >> 5, h = (r >> 4) & 1, l = r & 15;
      uint8_t sb = *at(0, 8 * n + 2 * j + h);
      int q = (*at(1, 32 * n + 16 * h + l) >> (2 * j)) & 3;
      float dl = __fmul_rn(d, (float)(sb & 0x0F)), ml = __fmul_rn(dmin, (float)(sb >> 4));
      return __fsub_rn(__fmul_rn(dl, (float)q), ml);
    }
    case QK_T_Q3_K: {  // reference/q3_k.rs:29-59 (scales), :79-118 (weights)
      float d = qk_h2f(at(3, 0));
      int grp = i >> 7, r = i & 127, j = r >> 5, n = (r >> 4) & 1, l = r & 15, is = 8 * grp + 2 * j + n;
      int raw;
      if (is < 8) {
        raw = *at(2, is) & 0x3F;
      } else if (is < 12) {
        raw = (*at(2, is) & 0x0F) | (((*at(2, is - 8) >> 6) & 3) << 4);
      } else {
        raw = ((*at(2, is - 4) >> 4) & 0x0F) | (((*at(2, is - 8) >> 6) & 3) << 4);
      }
      int q_lo = (*at(1, 32 * grp + 16 * n + l) >> (2 * j)) & 3;
      int sub = ((*at(0, 16 * n + l) >> (4 * grp + j)) & 1) ? 0 : 4;
      float dl = __fmul_rn(d, (float)(raw - 32));
      return __fmul_rn(dl, (float)(q_lo - sub));
    }
    case QK_T_Q8_K: {  // reference/q8_k.rs:40-47
      float d = *reinterpret_cast<const float *>(at(0, 0));
      return __fmul_rn(d, (float)(int8_t)*at(1, i));
    }
    case QK_T_Q6_K: {  // reference/q6_k.rs:39-71
      const uint8_t *sc = at(1, 0);
      float d = qk_h2f(at(2, 0));
      int g = i >> 7, rem = i & 127, k = rem >> 5, l = rem & 31, is = l >> 4;
      uint8_t qlb = *at(0, 64 * g + l + ((k & 1) ? 32 : 0));
      uint8_t qhb = *at(0, 128 + 32 * g + l);
      int nib = (k & 2) ? (qlb >> 4) : (qlb & 0x0F);
      int q = (nib | (((qhb >> (2 * k)) & 3) << 4)) - 32;
      float s = (float)(int8_t)sc[8 * g + is + 2 * k];
      return __fmul_rn(__fmul_rn(d, s), (float)q);
    }
    default: {  // IQ4_XS, reference/iq4_xs.rs:73-93
      const uint8_t *h = at(1, 0);
      float d = qk_h2f(h);
      uint32_t sh = h[2] | (h[3] << 8);
      int sub = i >> 5, j = i & 31;
      int ls = ((h[4 + (sub >> 1)] >> (4 * (sub & 1))) & 0x0F) | (((sh >> (2 * sub)) & 3) << 4);
      uint8_t byte = *at(0, 16 * sub + (j >> 1));
      int n = (j & 1) ? (byte >> 4) : (byte & 0x0F);
      float scale = __fmul_rn(d, (float)(ls - 32));
      return __fmul_rn(scale, (float)QK_KVALUES_IQ4NL[n]);
    }
  }
}
