// Q4_K policy of the decode kernel (qk_gemv_skel.cuh).
//
// One 256-column span = one super-block per row: the tile holds, per span, the eight rows'
// 16-byte headers (d, dmin, 12 bytes of 6-bit scales / mins) and then four 32-byte groups of
// nibbles per row, [group][row][32 bytes].  k = 32 of the MMA is exactly one sub-block:
//
//   A (16 x 32, u8): rows 0-7  = the eight weight rows, low nibbles of one
//                                32-byte group            (sub-block 2p: q)
//                    rows 8-15 = same rows, the raw bytes (q_lo + 16 q_hi)
//   B (32 x 8,  s8): even column 2j = digit j of the activations of sub-block 2p,
//                    odd column 2j+1 = digit j of those of sub-block 2p+1 (j = 0..2;
//                    columns 6, 7 unused)
//   C (16 x 8, s32): C[r][2j]     = sum q_lo D_j(2p)              wanted
//                    C[r][2j+1]   = sum q_lo D_j(2p+1)            cross term
//                    C[8+r][2j+1] = sum (q_lo + 16 q_hi) D_j(2p+1)
//                    so 16 * (high-nibble dot) = C[8+r][2j+1] - C[r][2j+1]: the cross
//                    term pays for not masking the high nibbles.
//
//   y[row] = sum_sub  d sc_sub sx_sub (I0 + I1/254 + I2/254^2)  -  dmin mn_sub Sx_sub
// with d, dmin, sc, mn decoded as reference/q4_k.rs:27-49,141-157 and Sx the
// f32 sum of x over the sub-block (the `- m1` term of reference/q4_k.rs:163).
#pragma once
#include "qk_gemv_skel.cuh"

namespace qkdec {

struct DecQ4K {
  static constexpr uint32_t COLB = 1152;  // 8 x 16 header bytes + 4 x 8 x 32 nibble bytes
  static constexpr uint32_t XSB = 8;      // (sx, Sx) per 32-column block
  static constexpr int MAX_M = 4;
  static constexpr bool HAS_DUAL = true;
  static constexpr bool SPLIT_PRODUCER = true;  // the tile producer as a warp of its own (measured per format)

  // digit planes in natural column order
  __device__ static __forceinline__ void store_digits(unsigned char *row_img, uint32_t PS, uint32_t e0, uint32_t w0,
                                                      uint32_t w1, uint32_t w2) {
    unsigned char *p = row_img + e0;
    *reinterpret_cast<uint32_t *>(p) = w0;
    *reinterpret_cast<uint32_t *>(p + PS) = w1;
    *reinterpret_cast<uint32_t *>(p + 2 * PS) = w2;
  }
  __device__ static __forceinline__ void store_xs(unsigned char *tab, size_t blk, float sx, float s32, float, float) {
    *reinterpret_cast<float2 *>(tab + blk * 8) = make_float2(sx, s32);
  }

  // One super-block column of a tile as a compute warp holds it in registers:
  // row g's 16-byte header, the lane's 8 bytes of each of the four 32-byte groups,
  // and per activation row the (sx, Sx) pairs and digit fragments that meet them.
  template <int M>
  struct Data {
    uint4 h;
    uint2 w[4];
    float4 xs[M];
    uint2 b[M][4];
  };

  struct Lane {
    float kD;
    bool hi_half;
    uint32_t m1, m2, sel0, sel1;  // header decode constants (the lane unpacks sub-blocks 2 tig, 2 tig + 1)
    uint32_t hl, ql, xl, xsl, xm, xsm;
    __device__ __forceinline__ void init(uint32_t lane, uint32_t wl, uint32_t ximg, uint32_t PS, uint32_t xs_off,
                                         uint32_t Kp) {
      const uint32_t g = lane >> 2, tig = lane & 3;
      // lane (g, tig) owns digit j = tig of both sub-blocks of a group; tig == 3 holds the two
      // unused columns: weight 0.  The x16 of the high-nibble dot is folded into the sub-block scale.
      kD = tig == 0 ? 1.f : tig == 1 ? 1.f / 254.f : tig == 2 ? 1.f / (254.f * 254.f) : 0.f;
      // B column g of this lane: digit g / 2 of sub-block 2p (g even) or 2p + 1 (g odd);
      // columns 6 and 7 are never used, so they may hold anything (digit plane 2 again)
      const uint32_t b_off = (g < 6 ? (g >> 1) : 2u) * PS + (g & 1u) * 32u + tig * 8;
      hi_half = tig >= 2;
      m1 = hi_half ? 0x0F0F0F0Fu : 0x3F3F3F3Fu, m2 = hi_half ? 0x30303030u : 0u;
      sel0 = 0x7540u | (2u * (tig & 1u)), sel1 = sel0 + 1u;
      // header of row g, the lane's 8 nibble bytes, its digit fragment and scales
      hl = wl * COLB + g * 16, ql = wl * COLB + 128 + g * 32 + tig * 8;
      xl = ximg + b_off + wl * 256;
      xsl = ximg + xs_off + (wl * 8 + 2 * tig) * 8;
      xm = 3 * PS, xsm = (Kp / 32) * 8;  // per activation row
    }
  };

  struct Base {
    uint32_t h, q, x, xs;
  };
  __device__ static __forceinline__ Base base(const Lane &LN, uint32_t tile, uint32_t kt) {
    return {tile + LN.hl, tile + LN.ql, LN.xl + kt * (QK_TILE_ELEMS / 32) * 32,
            LN.xsl + kt * (QK_TILE_ELEMS / 32) * 8};
  }

  // Column J of this warp is super-block wl + J * WG of the tile.
  template <int M, int J, int WG>
  __device__ static __forceinline__ void load(Data<M> &D, const Base &B, const Lane &LN) {
    D.h = lds128o<J * WG * 1152>(B.h);
    static_for<0, 4>([&](auto gq) {
      D.w[decltype(gq)::value] = lds64o<J * WG * 1152 + decltype(gq)::value * 256>(B.q);
    });
#pragma unroll
    for (int m = 0; m < M; m++) {
      D.xs[m] = lds128fo<J * WG * 64>(B.xs + m * LN.xsm);
      const uint32_t xb = B.x + m * LN.xm;
      static_for<0, 4>([&](auto gq) {
        D.b[m][decltype(gq)::value] = lds64o<J * WG * 256 + decltype(gq)::value * 64>(xb);
      });
    }
  }

  // acc[m] = {low-nibble sums, 16 x high-nibble sums (scale pre-divided), min terms}
  template <int M>
  __device__ static __forceinline__ void compute(const Data<M> &D, const Lane &LN, float (&acc)[M][3]) {
    // this lane decodes sub-blocks (2 tig, 2 tig + 1) of row g's header:
    // reference/q4_k.rs:27-49 on four 6-bit fields at a time, then byte -> f32 by
    // dropping the byte into the mantissa of 2^23
    const uint4 h = D.h;
    const float d = h2f_bits(h.x), dmin = h2f_bits(h.x >> 16);
    const uint32_t scw = ((LN.hi_half ? h.w : h.y) & LN.m1) | ((h.y >> 2) & LN.m2);
    const uint32_t mnw = ((LN.hi_half ? (h.w >> 4) : h.z) & LN.m1) | ((h.z >> 2) & LN.m2);
    const float ds0 = d * (__int_as_float(__byte_perm(scw, 0x4B000000u, LN.sel0)) - 8388608.f);
    const float ds1 =
        d * (1.f / 16.f) * (__int_as_float(__byte_perm(scw, 0x4B000000u, LN.sel1)) - 8388608.f);
    const float dm0 = dmin * (__int_as_float(__byte_perm(mnw, 0x4B000000u, LN.sel0)) - 8388608.f);
    const float dm1 = dmin * (__int_as_float(__byte_perm(mnw, 0x4B000000u, LN.sel1)) - 8388608.f);
#pragma unroll
    for (int m = 0; m < M; m++) {
      const float tx = ds0 * D.xs[m].x, ty = ds1 * D.xs[m].z;
      acc[m][2] = fmaf(dm0, D.xs[m].y, acc[m][2]);
      acc[m][2] = fmaf(dm1, D.xs[m].w, acc[m][2]);
      // four MMAs back to back (one per 32-byte group), then their scaling
      int c[4][4];
#pragma unroll
      for (int gq = 0; gq < 4; gq++)
        mma_u8s8(c[gq], D.w[gq].x & 0x0F0F0F0Fu, D.w[gq].x, D.w[gq].y & 0x0F0F0F0Fu, D.w[gq].y,
                 D.b[m][gq].x, D.b[m][gq].y);
#pragma unroll
      for (int gq = 0; gq < 4; gq++) {
        // lane gq of this lane's group of four (width 4: the source lane is an immediate)
        const float sx = __shfl_sync(0xffffffffu, tx, gq, 4);
        const float sy = __shfl_sync(0xffffffffu, ty, gq, 4);
        acc[m][0] = fmaf(sx, __int2float_rn(c[gq][0]), acc[m][0]);
        acc[m][1] = fmaf(sy, __int2float_rn(c[gq][3] - c[gq][1]), acc[m][1]);
      }
    }
  }

  __device__ static __forceinline__ float finish(const float (&a)[3], const Lane &LN) {
    return LN.kD * (a[0] + a[1]) - a[2];
  }
};

}  // namespace qkdec
