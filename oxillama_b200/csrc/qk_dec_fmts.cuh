// Q8_0, Q4_0, IQ4_XS and Q6_K policies of the decode kernel (qk_gemv_skel.cuh).
//
// All four use the MMA the way the Q4_K policy does: k = 32 of one
// mma.sync.m16n8k32 is one group of 32 weights that share a scale, the even B columns
// carry the three activation digits of one group and the odd columns those of a second
// group, and every lane of an MMA quad (g = lane / 4 = weight row, tig = lane % 4 = digit)
// keeps fixed registers.  They differ in what the two groups of an MMA are:
//
//   Q8_0, Q4_0, IQ4_XS   A rows 0-7 = the eight weight rows of 32-weight block (sub-block)
//                        2p, A rows 8-15 = the same rows of block 2p + 1; wanted are
//                        C[r][2j] (block 2p, digit j) and C[8 + r][2j + 1] (block 2p + 1).
//   Q6_K                 its scales cover 16 columns, so the two groups are the two
//                        16-column strips of one 32-column block: k-slots 0-15 hold strip
//                        0, slots 16-31 strip 1, the even B columns are zero in slots
//                        16-31 and the odd ones zero in slots 0-15; A rows 8-15 are zero.
//                        Wanted are C[r][2j] (strip 0) and C[r][2j + 1] (strip 1).
//
// Zero points (Q4_0: q - 8, Q6_K: q - 32) are not subtracted from the weights: the
// unsigned fields go into the MMA and  zero * scale * (sum of x over the group)  comes off
// once per group, from the block sums the activation split leaves in the scale table.
// IQ4_XS maps its nibbles through the 16-entry table (reference/iq_shared.rs:16-18) to s8
// with three byte permutes per four nibbles, so it stays exact integer work as well.
//
// A 256-column span of a tile ("column") is, per format (8 rows, block-major):
//   Q8_0    8 blocks x [2 x 8 rows x 16 int8 | 8 x f16 d]                    = 8 x 272
//   Q4_0    8 blocks x [8 rows x 16 nibble bytes | 8 x f16 d]                = 8 x 144
//   IQ4_XS  [8 sub-blocks x 8 rows x 16 nibble bytes | 8 rows x 8 header]    = 1088
//   Q6_K    [12 x 8 rows x 16 bytes of ql+qh | 8 rows x 16 scales | 8 x d]   = 1680
#pragma once
#include "qk_gemv_skel.cuh"

namespace qkdec {

template <int OFF>
__device__ __forceinline__ uint32_t lds32o(uint32_t addr) {
  uint32_t v;
  asm volatile("ld.shared.u32 %0, [%1+%2];" : "=r"(v) : "r"(addr), "n"(OFF));
  return v;
}
template <int OFF>
__device__ __forceinline__ uint32_t lds16o(uint32_t addr) {
  uint32_t v;
  asm volatile("{\n\t.reg .u16 t;\n\tld.shared.u16 t, [%1+%2];\n\tcvt.u32.u16 %0, t;\n\t}" : "=r"(v) : "r"(addr), "n"(OFF));
  return v;
}
__device__ __forceinline__ void mma_s8s8(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
  asm("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%10,%11,%12,%13};"
      : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0), "r"(0), "r"(0), "r"(0));
}
__device__ __forceinline__ float digit_weight(uint32_t tig) {
  return tig == 0 ? 1.f : tig == 1 ? 1.f / 254.f : tig == 2 ? 1.f / (254.f * 254.f) : 0.f;
}
__device__ __forceinline__ void store_digits_natural(unsigned char *row_img, uint32_t PS, uint32_t e0, uint32_t w0,
                                                     uint32_t w1, uint32_t w2) {
  unsigned char *p = row_img + e0;
  *reinterpret_cast<uint32_t *>(p) = w0;
  *reinterpret_cast<uint32_t *>(p + PS) = w1;
  *reinterpret_cast<uint32_t *>(p + 2 * PS) = w2;
}

// What Q8_0, Q4_0 and IQ4_XS share: the lane's digit fragment of MMA gq is 8 consecutive
// bytes of the digit plane of block 2 gq (+ 1 for an odd column); scale table entries are
// (sx, Sx) pairs and the lane reads those of blocks 2 tig and 2 tig + 1.
struct LaneCommon {
  float kD;
  uint32_t xl, xsl, xm, xsm;
  __device__ __forceinline__ void init_common(uint32_t lane, uint32_t wl, uint32_t ximg, uint32_t PS,
                                              uint32_t xs_off, uint32_t Kp) {
    const uint32_t g = lane >> 2, tig = lane & 3;
    kD = digit_weight(tig);
    const uint32_t b_off = (g < 6 ? (g >> 1) : 2u) * PS + (g & 1u) * 32u + tig * 8;
    xl = ximg + b_off + wl * 256;
    xsl = ximg + xs_off + (wl * 8 + 2 * tig) * 8;
    xm = 3 * PS, xsm = (Kp / 32) * 8;
  }
};
template <int M, int J, int WG, class D, class B, class LN>
__device__ __forceinline__ void load_x_common(D &d, const B &b, const LN &ln) {
#pragma unroll
  for (int m = 0; m < M; m++) {
    d.xs[m] = lds128fo<J * WG * 64>(b.xs + m * ln.xsm);
    const uint32_t xb = b.x + m * ln.xm;
    static_for<0, 4>([&](auto gq) { d.b[m][decltype(gq)::value] = lds64o<J * WG * 256 + decltype(gq)::value * 64>(xb); });
  }
}

// ---------------------------------------------------------------------------- Q8_0
// reference/q8_0.rs:46-97: y = sum_blocks d * sum_i q_i x_i, q signed 8-bit.
struct DecQ80 {
  static constexpr uint32_t COLB = 8 * 272, XSB = 8;
  static constexpr int MAX_M = 4;
  static constexpr bool HAS_DUAL = false;
  static constexpr bool SPLIT_PRODUCER = false;  // the tile producer as a warp of its own (measured per format)
  // digit order inside a 32-column block: the lane's 8 bytes are columns 4 tig .. + 3 and
  // 16 + 4 tig .. + 3, the two 4-byte pieces of its A fragment (bytes 4 tig of both 16-byte granules)
  __device__ static __forceinline__ void store_digits(unsigned char *row_img, uint32_t PS, uint32_t e0, uint32_t w0,
                                                      uint32_t w1, uint32_t w2) {
    const uint32_t i = e0 & 31u;
    store_digits_natural(row_img, PS, (e0 & ~31u) + ((i & 12u) << 1) + ((i & 16u) >> 2), w0, w1, w2);
  }
  __device__ static __forceinline__ void store_xs(unsigned char *tab, size_t blk, float sx, float s32, float, float) {
    *reinterpret_cast<float2 *>(tab + blk * 8) = make_float2(sx, s32);
  }
  template <int M>
  struct Data {
    uint32_t a[4][4];  // per MMA: the A fragment as is
    uint32_t dd[2];    // f16 d of blocks 2 tig, 2 tig + 1 of row g
    float4 xs[M];
    uint2 b[M][4];
  };
  struct Lane : LaneCommon {
    uint32_t wl0, dl;
    __device__ __forceinline__ void init(uint32_t lane, uint32_t wl, uint32_t ximg, uint32_t PS, uint32_t xs_off,
                                         uint32_t Kp) {
      init_common(lane, wl, ximg, PS, xs_off, Kp);
      const uint32_t g = lane >> 2, tig = lane & 3;
      wl0 = wl * COLB + g * 16 + tig * 4;
      dl = wl * COLB + tig * 544 + 256 + 2 * g;
    }
  };
  struct Base {
    uint32_t w, d, x, xs;
  };
  __device__ static __forceinline__ Base base(const Lane &LN, uint32_t tile, uint32_t kt) {
    return {tile + LN.wl0, tile + LN.dl, LN.xl + kt * (QK_TILE_ELEMS / 32) * 32, LN.xsl + kt * (QK_TILE_ELEMS / 32) * 8};
  }
  template <int M, int J, int WG>
  __device__ static __forceinline__ void load(Data<M> &D, const Base &B, const Lane &LN) {
    static_for<0, 4>([&](auto gq) {
      constexpr int G = decltype(gq)::value, O = J * WG * (int)COLB + 2 * G * 272;
      D.a[G][0] = lds32o<O>(B.w), D.a[G][2] = lds32o<O + 128>(B.w);
      D.a[G][1] = lds32o<O + 272>(B.w), D.a[G][3] = lds32o<O + 272 + 128>(B.w);
    });
    D.dd[0] = lds16o<J * WG * (int)COLB>(B.d), D.dd[1] = lds16o<J * WG * (int)COLB + 272>(B.d);
    load_x_common<M, J, WG>(D, B, LN);
  }
  template <int M>
  __device__ static __forceinline__ void compute(const Data<M> &D, const Lane &LN, float (&acc)[M][3]) {
    const float d0 = h2f_bits(D.dd[0]), d1 = h2f_bits(D.dd[1]);
#pragma unroll
    for (int m = 0; m < M; m++) {
      const float tx = d0 * D.xs[m].x, ty = d1 * D.xs[m].z;
      int c[4][4];
#pragma unroll
      for (int gq = 0; gq < 4; gq++)
        mma_s8s8(c[gq], D.a[gq][0], D.a[gq][1], D.a[gq][2], D.a[gq][3], D.b[m][gq].x, D.b[m][gq].y);
#pragma unroll
      for (int gq = 0; gq < 4; gq++) {
        acc[m][0] = fmaf(__shfl_sync(0xffffffffu, tx, gq, 4), __int2float_rn(c[gq][0]), acc[m][0]);
        acc[m][1] = fmaf(__shfl_sync(0xffffffffu, ty, gq, 4), __int2float_rn(c[gq][3]), acc[m][1]);
      }
    }
  }
  __device__ static __forceinline__ float finish(const float (&a)[3], const Lane &LN) { return LN.kD * (a[0] + a[1]); }
};

// ---------------------------------------------------------------------------- Q4_0
// reference/q4_0.rs:51-107: byte i of a block holds elements 2 i (low nibble) and 2 i + 1
// (high nibble), value (q - 8) d.
struct DecQ40 {
  static constexpr uint32_t COLB = 8 * 144, XSB = 8;
  static constexpr int MAX_M = 4;
  static constexpr bool HAS_DUAL = false;
  static constexpr bool SPLIT_PRODUCER = false;  // the tile producer as a warp of its own (measured per format)
  // The lane's word (bytes 4 tig .. + 3 of the block) holds elements 8 tig .. + 7: low
  // nibbles the even ones, high nibbles the odd ones.  Digits go evens first, then odds,
  // inside every group of 8 columns.
  __device__ static __forceinline__ void store_digits(unsigned char *row_img, uint32_t PS, uint32_t e0, uint32_t w0,
                                                      uint32_t w1, uint32_t w2) {
    unsigned char *p = row_img + (e0 & ~7u) + ((e0 & 4u) >> 1);
    const uint32_t w[3] = {w0, w1, w2};
#pragma unroll
    for (int d = 0; d < 3; d++) {
      *reinterpret_cast<unsigned short *>(p + d * PS) = (unsigned short)__byte_perm(w[d], 0, 0x4420);      // columns e0, e0 + 2
      *reinterpret_cast<unsigned short *>(p + d * PS + 4) = (unsigned short)__byte_perm(w[d], 0, 0x4431);  // e0 + 1, e0 + 3
    }
  }
  __device__ static __forceinline__ void store_xs(unsigned char *tab, size_t blk, float sx, float s32, float, float) {
    *reinterpret_cast<float2 *>(tab + blk * 8) = make_float2(sx, s32);
  }
  template <int M>
  struct Data {
    uint32_t w[8];   // the lane's word of each of the 8 blocks
    uint32_t dd[2];
    float4 xs[M];
    uint2 b[M][4];
  };
  struct Lane : LaneCommon {
    uint32_t wl0, dl;
    __device__ __forceinline__ void init(uint32_t lane, uint32_t wl, uint32_t ximg, uint32_t PS, uint32_t xs_off,
                                         uint32_t Kp) {
      init_common(lane, wl, ximg, PS, xs_off, Kp);
      const uint32_t g = lane >> 2, tig = lane & 3;
      wl0 = wl * COLB + g * 16 + tig * 4;
      dl = wl * COLB + tig * 288 + 128 + 2 * g;
    }
  };
  using Base = DecQ80::Base;
  __device__ static __forceinline__ Base base(const Lane &LN, uint32_t tile, uint32_t kt) {
    return {tile + LN.wl0, tile + LN.dl, LN.xl + kt * (QK_TILE_ELEMS / 32) * 32, LN.xsl + kt * (QK_TILE_ELEMS / 32) * 8};
  }
  template <int M, int J, int WG>
  __device__ static __forceinline__ void load(Data<M> &D, const Base &B, const Lane &LN) {
    static_for<0, 8>([&](auto bq) { D.w[decltype(bq)::value] = lds32o<J * WG * (int)COLB + decltype(bq)::value * 144>(B.w); });
    D.dd[0] = lds16o<J * WG * (int)COLB>(B.d), D.dd[1] = lds16o<J * WG * (int)COLB + 144>(B.d);
    load_x_common<M, J, WG>(D, B, LN);
  }
  template <int M>
  __device__ static __forceinline__ void compute(const Data<M> &D, const Lane &LN, float (&acc)[M][3]) {
    const float d0 = h2f_bits(D.dd[0]), d1 = h2f_bits(D.dd[1]);
    uint32_t a[4][4];
#pragma unroll
    for (int gq = 0; gq < 4; gq++) {
      a[gq][0] = D.w[2 * gq] & 0x0F0F0F0Fu, a[gq][2] = (D.w[2 * gq] >> 4) & 0x0F0F0F0Fu;
      a[gq][1] = D.w[2 * gq + 1] & 0x0F0F0F0Fu, a[gq][3] = (D.w[2 * gq + 1] >> 4) & 0x0F0F0F0Fu;
    }
#pragma unroll
    for (int m = 0; m < M; m++) {
      const float tx = d0 * D.xs[m].x, ty = d1 * D.xs[m].z;
      acc[m][2] = fmaf(8.f * d0, D.xs[m].y, acc[m][2]);  // the zero point: 8 d Sx
      acc[m][2] = fmaf(8.f * d1, D.xs[m].w, acc[m][2]);
      int c[4][4];
#pragma unroll
      for (int gq = 0; gq < 4; gq++)
        mma_u8s8(c[gq], a[gq][0], a[gq][1], a[gq][2], a[gq][3], D.b[m][gq].x, D.b[m][gq].y);
#pragma unroll
      for (int gq = 0; gq < 4; gq++) {
        acc[m][0] = fmaf(__shfl_sync(0xffffffffu, tx, gq, 4), __int2float_rn(c[gq][0]), acc[m][0]);
        acc[m][1] = fmaf(__shfl_sync(0xffffffffu, ty, gq, 4), __int2float_rn(c[gq][3]), acc[m][1]);
      }
    }
  }
  __device__ static __forceinline__ float finish(const float (&a)[3], const Lane &LN) {
    return LN.kD * (a[0] + a[1]) - a[2];
  }
};

// ---------------------------------------------------------------------------- IQ4_XS
// reference/iq4_xs.rs:99-168: sub-block s of a super-block = nibble bytes 16 s .. + 15, byte
// i holding elements 2 i (low) and 2 i + 1 (high); value = d (ls_s - 32) K[nibble].
struct DecIQ4XS {
  static constexpr uint32_t COLB = 1088, XSB = 8;
  static constexpr int MAX_M = 4;
  static constexpr bool HAS_DUAL = false;
  static constexpr bool SPLIT_PRODUCER = false;  // the tile producer as a warp of its own (measured per format)
  __device__ static __forceinline__ void store_digits(unsigned char *row_img, uint32_t PS, uint32_t e0, uint32_t w0,
                                                      uint32_t w1, uint32_t w2) {
    store_digits_natural(row_img, PS, e0, w0, w1, w2);
  }
  __device__ static __forceinline__ void store_xs(unsigned char *tab, size_t blk, float sx, float s32, float, float) {
    *reinterpret_cast<float2 *>(tab + blk * 8) = make_float2(sx, s32);
  }
  // Four nibbles (the low 16 bits of s) -> their table values as four s8, in nibble order:
  // the low three bits of each nibble pick one of eight bytes from each half of the table,
  // the top bit picks the half.
  // `lo3` holds the low three bits of each nibble, `pick` = 0x3210 + 4 * (top bit of each nibble),
  // both already shifted so that the four nibbles wanted sit in bits 0-15.
  __device__ static __forceinline__ uint32_t lookup4(uint32_t lo3, uint32_t pick) {
    constexpr uint32_t T0 = 0xBFAD9881u, T1 = 0xF6EADDCFu, T2 = 0x26190D01u, T3 = 0x71594535u;  // K[0..15] as bytes
    uint32_t va, vb, r;  // prmt reads only bits 0-15 of its selector
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(va) : "r"(T0), "r"(T1), "r"(lo3));
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(vb) : "r"(T2), "r"(T3), "r"(lo3));
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(va), "r"(vb), "r"(pick));
    return r;
  }
  // Eight nibbles of one word -> two fragments (elements 0-3 and 4-7): the masks are formed
  // once for the whole word.
  __device__ static __forceinline__ void lookup8(uint32_t w, uint32_t &lo, uint32_t &hi) {
    const uint32_t lo3 = w & 0x77777777u, pick = ((w >> 1) & 0x44444444u) | 0x32103210u;
    lo = lookup4(lo3, pick);
    hi = lookup4(lo3 >> 16, pick >> 16);
  }
  template <int M>
  struct Data {
    uint32_t w[8];  // the lane's word (8 nibbles = elements 8 tig .. + 7) of each sub-block
    uint2 h;        // d | scales_h << 16, scales_l
    float4 xs[M];
    uint2 b[M][4];
  };
  struct Lane : LaneCommon {
    uint32_t wl0, hl, shl, shh;
    __device__ __forceinline__ void init(uint32_t lane, uint32_t wl, uint32_t ximg, uint32_t PS, uint32_t xs_off,
                                         uint32_t Kp) {
      init_common(lane, wl, ximg, PS, xs_off, Kp);
      const uint32_t g = lane >> 2, tig = lane & 3;
      wl0 = wl * COLB + g * 16 + tig * 4;
      hl = wl * COLB + 1024 + g * 8;
      shl = 8 * tig, shh = 16 + 4 * tig;  // where sub-block 2 tig sits in scales_l and in (d | scales_h << 16)
    }
  };
  struct Base {
    uint32_t w, h, x, xs;
  };
  __device__ static __forceinline__ Base base(const Lane &LN, uint32_t tile, uint32_t kt) {
    return {tile + LN.wl0, tile + LN.hl, LN.xl + kt * (QK_TILE_ELEMS / 32) * 32, LN.xsl + kt * (QK_TILE_ELEMS / 32) * 8};
  }
  template <int M, int J, int WG>
  __device__ static __forceinline__ void load(Data<M> &D, const Base &B, const Lane &LN) {
    static_for<0, 8>([&](auto sq) { D.w[decltype(sq)::value] = lds32o<J * WG * (int)COLB + decltype(sq)::value * 128>(B.w); });
    D.h = lds64o<J * WG * (int)COLB>(B.h);
    load_x_common<M, J, WG>(D, B, LN);
  }
  template <int M>
  __device__ static __forceinline__ void compute(const Data<M> &D, const Lane &LN, float (&acc)[M][3]) {
    // reference/iq4_xs.rs:47-53 for sub-blocks 2 tig and 2 tig + 1
    const float d = h2f_bits(D.h.x);
    const uint32_t sl = D.h.y >> LN.shl, sh = D.h.x >> LN.shh;
    const int ls0 = (int)((sl & 0xFu) | ((sh & 3u) << 4)), ls1 = (int)(((sl >> 4) & 0xFu) | (((sh >> 2) & 3u) << 4));
    const float sc0 = d * (float)(ls0 - 32), sc1 = d * (float)(ls1 - 32);
    uint32_t a[4][4];
#pragma unroll
    for (int gq = 0; gq < 4; gq++) {
      lookup8(D.w[2 * gq], a[gq][0], a[gq][2]);
      lookup8(D.w[2 * gq + 1], a[gq][1], a[gq][3]);
    }
#pragma unroll
    for (int m = 0; m < M; m++) {
      const float tx = sc0 * D.xs[m].x, ty = sc1 * D.xs[m].z;
      int c[4][4];
#pragma unroll
      for (int gq = 0; gq < 4; gq++)
        mma_s8s8(c[gq], a[gq][0], a[gq][1], a[gq][2], a[gq][3], D.b[m][gq].x, D.b[m][gq].y);
#pragma unroll
      for (int gq = 0; gq < 4; gq++) {
        acc[m][0] = fmaf(__shfl_sync(0xffffffffu, tx, gq, 4), __int2float_rn(c[gq][0]), acc[m][0]);
        acc[m][1] = fmaf(__shfl_sync(0xffffffffu, ty, gq, 4), __int2float_rn(c[gq][3]), acc[m][1]);
      }
    }
  }
  __device__ static __forceinline__ float finish(const float (&a)[3], const Lane &LN) { return LN.kD * (a[0] + a[1]); }
};

// ---------------------------------------------------------------------------- Q6_K
// reference/q6_k.rs:77-172.  Element (half G, strip k, l) of a super-block: column
// 128 G + 32 k + l, q = (ql[64 G + 32 (k & 1) + l] nibble (k >> 1)) | (qh[32 G + l] bits 2k, 2k+1) << 4,
// value d sc[8 G + 2 k + l / 16] (q - 32).
struct DecQ6K {
  static constexpr uint32_t COLB = 1680, XSB = 16;
  static constexpr bool HAS_DUAL = false;
  static constexpr bool SPLIT_PRODUCER = false;  // the tile producer as a warp of its own (measured per format)
  static constexpr int MAX_M = 2;  // three rows and up spill heavily (twelve weight words and sixteen fragments per column)
  __device__ static __forceinline__ void store_digits(unsigned char *row_img, uint32_t PS, uint32_t e0, uint32_t w0,
                                                      uint32_t w1, uint32_t w2) {
    store_digits_natural(row_img, PS, e0, w0, w1, w2);
  }
  // (sx, sum over the 32 columns, sums over its two 16-column strips)
  __device__ static __forceinline__ void store_xs(unsigned char *tab, size_t blk, float sx, float s32, float s16a,
                                                  float s16b) {
    *reinterpret_cast<float4 *>(tab + blk * 16) = make_float4(sx, s32, s16a, s16b);
  }
  template <int M>
  struct Data {
    uint32_t ql[8];  // [G * 4 + (k & 1) * 2 + is]: bytes 4 tig .. + 3 of the strip's 16 ql bytes
    uint32_t qh[4];  // [G * 2 + is]
    uint32_t sc, dd; // scales 4 tig .. + 3 of row g (int8 x 4), f16 d
    float4 xs[M][2]; // scale table entries of 32-column blocks 2 tig, 2 tig + 1
    uint32_t b[M][8];  // [G * 4 + k]: the lane's four digits of its strip of block 4 G + k
  };
  struct Lane {
    float kD;
    uint32_t wl0, sl0, dl, xl, xsl, xm, xsm, m0, m1;
    __device__ __forceinline__ void init(uint32_t lane, uint32_t wl, uint32_t ximg, uint32_t PS, uint32_t xs_off,
                                         uint32_t Kp) {
      const uint32_t g = lane >> 2, tig = lane & 3;
      kD = digit_weight(tig);
      wl0 = wl * COLB + g * 16 + tig * 4;
      sl0 = wl * COLB + 1536 + g * 16 + tig * 4;
      dl = wl * COLB + 1664 + 2 * g;
      // B column g: digit g / 2 of strip g & 1 (columns 6, 7 unused): four bytes of the natural-order plane
      const uint32_t b_off = (g < 6 ? (g >> 1) : 2u) * PS + (g & 1u) * 16u + tig * 4;
      xl = ximg + b_off + wl * 256;
      xsl = ximg + xs_off + (wl * 8 + 2 * tig) * 16;
      xm = 3 * PS, xsm = (Kp / 32) * 16;
      m0 = (g & 1u) ? 0u : 0xFFFFFFFFu, m1 = ~m0;  // an even column is zero in k-slots 16-31, an odd one in 0-15
    }
  };
  struct Base {
    uint32_t w, s, d, x, xs;
  };
  __device__ static __forceinline__ Base base(const Lane &LN, uint32_t tile, uint32_t kt) {
    return {tile + LN.wl0, tile + LN.sl0, tile + LN.dl, LN.xl + kt * (QK_TILE_ELEMS / 32) * 32,
            LN.xsl + kt * (QK_TILE_ELEMS / 32) * 16};
  }
  template <int M, int J, int WG>
  __device__ static __forceinline__ void load(Data<M> &D, const Base &B, const Lane &LN) {
    constexpr int C0 = J * WG * (int)COLB;
    static_for<0, 8>([&](auto iq) {  // granule 4 G + 2 (k & 1) + is of ql
      constexpr int I = decltype(iq)::value;
      D.ql[I] = lds32o<C0 + I * 128>(B.w);
    });
    static_for<0, 4>([&](auto iq) {  // granule 8 + 2 G + is: qh
      constexpr int I = decltype(iq)::value;
      D.qh[I] = lds32o<C0 + (8 + I) * 128>(B.w);
    });
    D.sc = lds32o<C0>(B.s), D.dd = lds16o<C0>(B.d);
#pragma unroll
    for (int m = 0; m < M; m++) {
      D.xs[m][0] = lds128fo<J * WG * 128>(B.xs + m * LN.xsm);
      D.xs[m][1] = lds128fo<J * WG * 128 + 16>(B.xs + m * LN.xsm);
      const uint32_t xb = B.x + m * LN.xm;
      static_for<0, 8>([&](auto iq) {
        constexpr int I = decltype(iq)::value;  // G * 4 + k: columns 128 G + 32 k
        D.b[m][I] = lds32o<J * WG * 256 + I * 32>(xb);
      });
    }
  }
  template <int M>
  __device__ static __forceinline__ void compute(const Data<M> &D, const Lane &LN, float (&acc)[M][3]) {
    const float d = h2f_bits(D.dd);
    // this lane's four scales: index 4 tig + j = 8 G + 2 k + is with G = tig / 2, k = 2 (tig & 1) + j / 2, is = j & 1
    float ds[4];
#pragma unroll
    for (int j = 0; j < 4; j++) ds[j] = d * (float)(int)(signed char)((D.sc >> (8 * j)) & 0xFFu);
    // the A fragments: strip is = 0 in k-slots 0-15 (a[.][0]), is = 1 in slots 16-31 (a[.][1])
    uint32_t a[8][2];
#pragma unroll
    for (int G = 0; G < 2; G++)
#pragma unroll
      for (int k = 0; k < 4; k++)
#pragma unroll
        for (int is = 0; is < 2; is++) {
          const uint32_t lw = D.ql[G * 4 + (k & 1) * 2 + is], hw = D.qh[G * 2 + is];
          const uint32_t lo = (k >> 1) ? (lw >> 4) : lw;
          const uint32_t hi = k == 0 ? (hw << 4) : k == 1 ? (hw << 2) : k == 2 ? hw : (hw >> 2);
          a[G * 4 + k][is] = (lo & 0x0F0F0F0Fu) | (hi & 0x30303030u);
        }
#pragma unroll
    for (int m = 0; m < M; m++) {
      const float4 x0 = D.xs[m][0], x1 = D.xs[m][1];
      const float t[4] = {ds[0] * x0.x, ds[1] * x0.x, ds[2] * x1.x, ds[3] * x1.x};
      // the zero point: 32 d sc (sum of x over the strip)
      float z = ds[0] * x0.z;
      z = fmaf(ds[1], x0.w, z), z = fmaf(ds[2], x1.z, z), z = fmaf(ds[3], x1.w, z);
      acc[m][2] = fmaf(32.f, z, acc[m][2]);
      int c[8][4];
#pragma unroll
      for (int i = 0; i < 8; i++)
        mma_u8s8(c[i], a[i][0], 0u, a[i][1], 0u, D.b[m][i] & LN.m0, D.b[m][i] & LN.m1);
#pragma unroll
      for (int G = 0; G < 2; G++)
#pragma unroll
        for (int k = 0; k < 4; k++) {
          // block 4 G + k's scales live in lane 2 G + k / 2 of the quad, entries 2 (k & 1), + 1
          const int src = 2 * G + (k >> 1);
          const float ta = __shfl_sync(0xffffffffu, t[2 * (k & 1)], src, 4);
          const float tb = __shfl_sync(0xffffffffu, t[2 * (k & 1) + 1], src, 4);
          acc[m][0] = fmaf(ta, __int2float_rn(c[G * 4 + k][0]), acc[m][0]);
          acc[m][1] = fmaf(tb, __int2float_rn(c[G * 4 + k][1]), acc[m][1]);
        }
    }
  }
  __device__ static __forceinline__ float finish(const float (&a)[3], const Lane &LN) {
    return LN.kD * (a[0] + a[1]) - a[2];
  }
};

}  // namespace qkdec
