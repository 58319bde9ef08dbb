// Batched dequant-matmul (prefill and larger decode batches) for Q4_K on the
// 5th-generation tensor cores: tcgen05.mma with the accumulator in tensor memory.
//
//   y[t][n] = sum_k  w(n, k) * x[t][k]          w = d sc q - dmin mn   (reference/q4_k.rs:79-93)
//
// A real dense contraction, so it goes to the tensor cores: 128 weight rows are
// the MMA's M dimension, BN activation rows (tokens) its N dimension, fp16
// operands with f32 accumulation in TMEM (kind::f16).
//
// One CTA per SM, persistent over (128 RH-row block) x (BN-token block) tiles; a
// tile walks K in super-blocks of 256 columns = four 64-column steps.
//   warps 0-3   MMA issuers.  Warp j issues the MMAs of 64-column group j of every
//               super-block: two K = 16 MMAs per 32-column half-stage unit, then a
//               tcgen05.commit to the unit's "empty" barrier.  Measured on B200: an
//               MMA holds the tensor pipe for 128 cycles whatever M <= 128 and
//               N <= 256 are, and holds its issuing thread meanwhile, with the
//               thread's barrier polls not hidden behind it; four issuers keep the
//               pipe fed.  All accumulate into the same TMEM columns.
//   warp 4      activation producer: one TMA tile load (128-byte swizzle, no
//               multicast) per step brings the fp16 activations of the BN tokens
//   warps 5-20  four groups of four warps; group g expands columns [64 g, 64 g + 64)
//               of every super-block, one thread per weight row: 16 + 32 packed bytes
//               straight from global memory (a super-block ahead in registers, six
//               ahead as L2 prefetches), 6-bit scales decoded, nibbles turned into
//               fp16 (magic-number nibble -> half2, one HFMA2 and one HSUB2 per
//               pair) and stored as 64-byte rows of two K-major units with 64-byte
//               swizzle.  The same warps run the epilogue (tcgen05.ld, store y with
//               lanes = consecutive weight rows = consecutive addresses, zero the
//               columns), in pieces between the super-blocks of the next tile.
//
// The activations are converted to fp16 once per call by qk_x16_kernel, with
// the columns of every 64-group permuted into the order in which a packed word
// yields its nibbles (both operands use the same order, so the sum is
// unchanged).  fp16 operands put the result at ~5e-4 of the output's inf-norm
// against the f32 reference (its stated tolerance is 1e-3).
//
// Every mbarrier wait is time-bounded; a wait that runs out raises
// QK_DEV_TIMEOUT and the CTA falls through to the common exit, which always
// frees its tensor memory.
#include <cuda.h>

#include <cfloat>
#include <cstdlib>

#include "qk_kernels.h"
#include "qk_pipe.cuh"

using namespace qkpipe;

namespace {

constexpr int BM = 128;            // weight rows per tile (UMMA M)
constexpr int BK = 64;             // columns per stage: one 128-byte swizzle row of fp16
constexpr int NDW = 16;            // dequant / epilogue warps: four groups of four, group g owns A stage g
// MMA-issuing warps 0 .. NI - 1, then the activation producer (warp NI), then the NDW expanding warps.
// Four issuers (warp j issues the steps of A stage j) make 21 warps, which are charged as 768 threads
// when the register file is divided: 80 registers per thread.  Q6_K's expansion spills 250-360 bytes
// at 80 and is the slower for it, so it runs three issuers (groups 0, 1 and (2, 3) of every
// super-block): 20 warps, 96 registers, 4096 x 14336 x 512 in 93.5 us instead of 113.7.  The other
// formats lose with three (Q4_K 14336 x 4096 x 512: 66.3 against 62.8 us; 32-128 tokens: 33 against
// 29 us) and keep four.
template <int T>
constexpr int n_issuers() { return T == QK_T_Q6_K ? 3 : 4; }
template <int T>
constexpr int n_threads() { return (n_issuers<T>() + 1 + NDW) * 32; }
constexpr int MAX_RING = 8;        // most stages of the activation ring
constexpr uint32_t A_HALF = BM * 64;  // bytes of one A half-stage: 128 rows of 32 fp16
#ifndef QK_GEMM_UPG
#define QK_GEMM_UPG 2                 // A units per dequant group: one per half-stage of a super-block (3 measured no faster)
#endif

struct GemmSmem {
  uint32_t a_full, a_empty, b_full, b_empty, acc_full, acc_empty, tmem_slot, lut;
  uint32_t a, b;  // ring bases, 1024-byte aligned
  uint32_t a_stage, b_stage;
  int b_stages;
};

#ifdef QK_TRACE
// Developer build only: block 0 timestamps its pipeline into a global buffer.
__device__ unsigned long long *qk_gemm_trace_buf = nullptr;
#define QK_GSTAMP(cond, idx)                                                          \
  do {                                                                                \
    if ((cond) && qk_gemm_trace_buf && blockIdx.x == 0 && (threadIdx.x & 31) == 0) {  \
      unsigned long long t__;                                                         \
      asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t__));                        \
      qk_gemm_trace_buf[idx] = t__;                                                   \
    }                                                                                 \
  } while (0)
#else
#define QK_GSTAMP(cond, idx) do {} while (0)
#endif

__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap *map, int x, int y,
                                            uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
          dst),
      "l"(map), "r"(x), "r"(y), "r"(bar)
      : "memory");
}
// K-major operand tile, 128-byte swizzle, rows 128 bytes apart, 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t umma_desc(uint32_t smem_addr) {
  return (uint64_t)((smem_addr >> 4) & 0x3FFFu) | ((uint64_t)1 << 16) | ((uint64_t)(1024 >> 4) << 32) |
         ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
}
// K-major operand tile of 32 fp16 per row: 64-byte swizzle, rows 64 bytes apart, 8-row groups 512 bytes apart.
__device__ __forceinline__ uint64_t umma_desc_sw64(uint32_t smem_addr) {
  return (uint64_t)((smem_addr >> 4) & 0x3FFFu) | ((uint64_t)1 << 16) | ((uint64_t)(512 >> 4) << 32) |
         ((uint64_t)1 << 46) | ((uint64_t)4 << 61);
}
__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc,
                                         uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      :
      : "r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
               : "memory");
}
__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// ---------------------------------------------------------------- weight formats
// What differs between the formats is how a thread fetches the packed bytes of one
// row-step (one weight row x 64 columns: group g of a 256-column super-block) and
// expands them into 64 fp16 values, 8 chunks of 8.  Each format expands in the order
// its packed words yield values; SRC(p) names the column (inside the super-block) that
// lands at position p, and the activations are laid out in the same order, so the
// contraction is unchanged.
//
//   Pk        the packed bytes of one row-step, held in registers a super-block ahead
//   load      fetch Pk for (8-row chunk at cb, row-in-chunk rr, group g, super-block s)
//   prefetch  the same bytes as L2 prefetches
//   expand    half hf (32 columns) of the row-step -> four 16-byte chunks
template <int T>
struct WFmt;

__device__ __forceinline__ uint4 ldg16(const uint8_t *p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}
__device__ __forceinline__ void pf_l2(const uint8_t *p) { asm volatile("prefetch.global.L2 [%0];" ::"l"(p)); }
__device__ __forceinline__ uint32_t h2_bits(__half2 v) { return *reinterpret_cast<uint32_t *>(&v); }
__device__ __forceinline__ __half2 bits_h2(uint32_t v) { return *reinterpret_cast<__half2 *>(&v); }
__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
  uint32_t d;
  asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(sel));
  return d;
}
// Four nibble pairs of one packed word -> 8 halves: low nibbles q become 1024 + q
// (0x6400 | q), high nibbles 64 + q (0x5400 | q << 4, no shift needed); values come out
// as pairs (byte 0, byte 2), (byte 1, byte 3) of the low nibbles, then of the high ones.
__device__ __forceinline__ void nibbles_to_magic(uint32_t w, uint32_t e[4]) {
  const uint32_t wj = w >> 8;
  e[0] = (w & 0x000F000Fu) | 0x64006400u, e[1] = (wj & 0x000F000Fu) | 0x64006400u;
  e[2] = (w & 0x00F000F0u) | 0x54005400u, e[3] = (wj & 0x00F000F0u) | 0x54005400u;
}
// Four unsigned bytes -> halves 1024 + b, in byte order.
__device__ __forceinline__ void bytes_to_magic(uint32_t w, uint32_t &lo, uint32_t &hi) {
  lo = prmt(w, 0x64646464u, 0x4140), hi = prmt(w, 0x64646464u, 0x4342);
}
// Start of block `blk` (of the row) in the 8-row chunk: tiles are block-major, so the
// 8 x bb bytes of one block column are one span and block columns follow one another.
__device__ __forceinline__ const uint8_t *chunk_addr(const QkLayout &L, const uint8_t *W, uint32_t chunk) {
  return W + (uint64_t)chunk * L.chunk_bytes;
}
template <uint32_t BB>
__device__ __forceinline__ const uint8_t *blk_addr(const uint8_t *chunk_base, uint32_t blk) {
  return chunk_base + (size_t)(blk * (QK_TILE_ROWS * BB));
}

template <>
struct WFmt<QK_T_Q4_K> {
  static constexpr bool HAS_LUT = false;
  __device__ static void fill_lut(uint32_t *, uint32_t, uint32_t) {}  // super-block of 256: d, dmin, 12 bytes of 6-bit scales/mins, 128 bytes of nibbles (reference/q4_k.rs:27-102)
  struct Pk { uint4 h, q0, q1; };
  // position 8 i + j of a row-step <- column 4 i + {0,2,1,3}[j & 3] + 32 (j >> 2): byte 4 i + b of
  // the group's 32 holds column 4 i + b (low nibble) and 32 + 4 i + b (high nibble)
  __host__ __device__ static uint32_t src(uint32_t p) {
    const uint32_t g = p >> 6, i = (p >> 3) & 7u, j = p & 7u, jj = j & 3u;
    return 64 * g + 4 * i + (jj == 1 ? 2 : jj == 2 ? 1 : jj) + 32 * (j >> 2);
  }
  __device__ static const uint8_t *base(const uint8_t *cb, uint32_t s) {
    return blk_addr<144>(cb, s);  // [8 rows x 16 header | 4 groups x 8 rows x 32 nibble bytes]
  }
  __device__ static void load(Pk &k, const QkLayout &L, const uint8_t *cb, uint32_t rr, uint32_t g,
                              uint32_t s) {
    const uint8_t *p = base(cb, s);
    k.h = ldg16(p + rr * 16), k.q0 = ldg16(p + 128 + g * 256 + rr * 32), k.q1 = ldg16(p + 128 + g * 256 + rr * 32 + 16);
  }
  __device__ static void prefetch(const QkLayout &L, const uint8_t *cb, uint32_t rr, uint32_t g, uint32_t s) {
    const uint8_t *p = base(cb, s);
    pf_l2(p + 128 + g * 256 + rr * 32);
    if (g == 0 && rr == 0) pf_l2(p);
  }
  struct Sc { __half2 s_lo, s_hi, c_lo, c_hi, m_lo, m_hi; };
  __device__ static void scales(const Pk &k, uint32_t g, Sc &c) {
    const float d = h2f_bits(k.h.x), dmin = h2f_bits(k.h.x >> 16);
    // sub-blocks 2 g (low nibbles) and 2 g + 1 (high nibbles)
    const uint32_t scw = g < 2 ? (k.h.y & 0x3F3F3F3Fu) : ((k.h.w & 0x0F0F0F0Fu) | ((k.h.y >> 2) & 0x30303030u));
    const uint32_t mnw = g < 2 ? (k.h.z & 0x3F3F3F3Fu) : (((k.h.w >> 4) & 0x0F0F0F0Fu) | ((k.h.z >> 2) & 0x30303030u));
    const uint32_t sh = (g & 1u) * 16;
    c.s_lo = __float2half2_rn(d * (float)((scw >> sh) & 0xFF)), c.s_hi = __float2half2_rn(d * (float)((scw >> (sh + 8)) & 0xFF));
    c.m_lo = __float2half2_rn(dmin * (float)((mnw >> sh) & 0xFF)), c.m_hi = __float2half2_rn(dmin * (float)((mnw >> (sh + 8)) & 0xFF));
    // (K + q) * s - K * s is exact in the FMA, so q * s is rounded once
    c.c_lo = __hmul2(c.s_lo, __float2half2_rn(-1024.f)), c.c_hi = __hmul2(c.s_hi, __float2half2_rn(-64.f));
  }
  __device__ static void expand(const Pk &k, const Sc &c, uint32_t g, int hf, uint32_t o[4][4], uint32_t) {
    const uint4 q = hf ? k.q1 : k.q0;
    const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
    for (int i = 0; i < 4; i++) {
      uint32_t e[4];
      nibbles_to_magic(w[i], e);
      o[i][0] = h2_bits(__hsub2(__hfma2(bits_h2(e[0]), c.s_lo, c.c_lo), c.m_lo));
      o[i][1] = h2_bits(__hsub2(__hfma2(bits_h2(e[1]), c.s_lo, c.c_lo), c.m_lo));
      o[i][2] = h2_bits(__hsub2(__hfma2(bits_h2(e[2]), c.s_hi, c.c_hi), c.m_hi));
      o[i][3] = h2_bits(__hsub2(__hfma2(bits_h2(e[3]), c.s_hi, c.c_hi), c.m_hi));
    }
  }
};

template <>
struct WFmt<QK_T_Q8_0> {
  static constexpr bool HAS_LUT = false;
  __device__ static void fill_lut(uint32_t *, uint32_t, uint32_t) {}  // block of 32: f16 d, 32 int8 (reference/q8_0.rs)
  struct Pk { uint4 q[4]; uint32_t d2; };
  __host__ __device__ static uint32_t src(uint32_t p) { return p; }
  // Blocks past the end of the row (a last super-block that is not full) read as d = 0, q = 0.
  // A block's 8 rows: [2 granules x 8 rows x 16 int8][8 x d].
  __device__ static void load(Pk &k, const QkLayout &L, const uint8_t *cb, uint32_t rr, uint32_t g,
                              uint32_t s) {
    const uint4 z = make_uint4(0, 0, 0, 0);
    k.q[0] = k.q[1] = k.q[2] = k.q[3] = z, k.d2 = 0;
    const uint32_t b = 8 * s + 2 * g;  // first of the row-step's two blocks
    if (b >= L.nb) return;
    const uint8_t *p = blk_addr<34>(cb, b);
    k.q[0] = ldg16(p + rr * 16), k.q[1] = ldg16(p + 128 + rr * 16);
    k.d2 = __ldg(reinterpret_cast<const unsigned short *>(p + 256) + rr);
    if (b + 1 < L.nb) {
      k.q[2] = ldg16(p + 272 + rr * 16), k.q[3] = ldg16(p + 272 + 128 + rr * 16);
      k.d2 |= (uint32_t)__ldg(reinterpret_cast<const unsigned short *>(p + 272 + 256) + rr) << 16;
    }
  }
  __device__ static void prefetch(const QkLayout &L, const uint8_t *cb, uint32_t rr, uint32_t g, uint32_t s) {
    const uint32_t b = 8 * s + 2 * g;
    if (b >= L.nb || rr >= 5) return;
    pf_l2(blk_addr<34>(cb, b) + rr * 128);  // two blocks = 544 bytes = up to five lines
  }
  struct Sc { __half2 d[2]; };
  __device__ static void scales(const Pk &k, uint32_t, Sc &c) {
    c.d[0] = bits_h2((k.d2 & 0xFFFFu) * 0x10001u), c.d[1] = bits_h2((k.d2 >> 16) * 0x10001u);
  }
  __device__ static void expand(const Pk &k, const Sc &c, uint32_t, int hf, uint32_t o[4][4], uint32_t) {
    const __half2 off = __float2half2_rn(1152.f);  // 1024 + 128: (1024 + (q ^ 0x80)) - 1152 = q, exact; q * d rounded once
#pragma unroll
    for (int i = 0; i < 4; i++) {
      const uint4 q = k.q[2 * hf + (i >> 1)];
      const uint32_t w0 = ((i & 1) ? q.z : q.x) ^ 0x80808080u, w1 = ((i & 1) ? q.w : q.y) ^ 0x80808080u;
      uint32_t a, b2;
      bytes_to_magic(w0, a, b2);
      o[i][0] = h2_bits(__hmul2(__hsub2(bits_h2(a), off), c.d[hf]));
      o[i][1] = h2_bits(__hmul2(__hsub2(bits_h2(b2), off), c.d[hf]));
      bytes_to_magic(w1, a, b2);
      o[i][2] = h2_bits(__hmul2(__hsub2(bits_h2(a), off), c.d[hf]));
      o[i][3] = h2_bits(__hmul2(__hsub2(bits_h2(b2), off), c.d[hf]));
    }
  }
};

template <>
struct WFmt<QK_T_Q4_0> {
  static constexpr bool HAS_LUT = false;
  __device__ static void fill_lut(uint32_t *, uint32_t, uint32_t) {}  // block of 32: f16 d, 16 bytes; byte j = elements 2 j (low nibble) and 2 j + 1 (high) (reference/q4_0.rs:36-46)
  struct Pk { uint4 q[2]; uint32_t d2; };
  // chunk c of a row-step is word c & 3 of block c >> 2; a word yields its elements as
  // (byte 0, byte 2), (byte 1, byte 3) low nibbles, then the same of the high nibbles
  __host__ __device__ static uint32_t src(uint32_t p) {
    const uint32_t c = (p >> 3) & 7u, j = p & 7u;
    const uint32_t order = 0x73516240u;  // positions 0..7 <- elements 0, 4, 2, 6, 1, 5, 3, 7 of the word
    return (p & ~63u) + 32 * (c >> 2) + 8 * (c & 3u) + ((order >> (4 * j)) & 7u);
  }
  // A block's 8 rows: [8 rows x 16 nibble bytes][8 x d].
  __device__ static void load(Pk &k, const QkLayout &L, const uint8_t *cb, uint32_t rr, uint32_t g,
                              uint32_t s) {
    k.q[0] = k.q[1] = make_uint4(0, 0, 0, 0), k.d2 = 0;
    const uint32_t b = 8 * s + 2 * g;
    if (b >= L.nb) return;
    const uint8_t *p = blk_addr<18>(cb, b);
    k.q[0] = ldg16(p + rr * 16), k.d2 = __ldg(reinterpret_cast<const unsigned short *>(p + 128) + rr);
    if (b + 1 < L.nb) {
      k.q[1] = ldg16(p + 144 + rr * 16);
      k.d2 |= (uint32_t)__ldg(reinterpret_cast<const unsigned short *>(p + 144 + 128) + rr) << 16;
    }
  }
  __device__ static void prefetch(const QkLayout &L, const uint8_t *cb, uint32_t rr, uint32_t g, uint32_t s) {
    const uint32_t b = 8 * s + 2 * g;
    if (b >= L.nb || rr >= 3) return;
    pf_l2(blk_addr<18>(cb, b) + rr * 128);  // two blocks = 288 bytes
  }
  using Sc = WFmt<QK_T_Q8_0>::Sc;
  __device__ static void scales(const Pk &k, uint32_t, Sc &c) {
    c.d[0] = bits_h2((k.d2 & 0xFFFFu) * 0x10001u), c.d[1] = bits_h2((k.d2 >> 16) * 0x10001u);
  }
  __device__ static void expand(const Pk &k, const Sc &c, uint32_t, int hf, uint32_t o[4][4], uint32_t) {
    const __half2 off_lo = __float2half2_rn(1032.f), off_hi = __float2half2_rn(72.f);  // K + 8: (K + q) - (K + 8) = q - 8, exact
    const uint4 q = k.q[hf];
    const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
    for (int i = 0; i < 4; i++) {
      uint32_t e[4];
      nibbles_to_magic(w[i], e);
      o[i][0] = h2_bits(__hmul2(__hsub2(bits_h2(e[0]), off_lo), c.d[hf]));
      o[i][1] = h2_bits(__hmul2(__hsub2(bits_h2(e[1]), off_lo), c.d[hf]));
      o[i][2] = h2_bits(__hmul2(__hsub2(bits_h2(e[2]), off_hi), c.d[hf]));
      o[i][3] = h2_bits(__hmul2(__hsub2(bits_h2(e[3]), off_hi), c.d[hf]));
    }
  }
};

template <>
struct WFmt<QK_T_Q6_K> {
  static constexpr bool HAS_LUT = false;
  __device__ static void fill_lut(uint32_t *, uint32_t, uint32_t) {}  // super-block of 256: ql 128, qh 64, 16 int8 scales, f16 d (reference/q6_k.rs)
  // group g: half hh = g >> 1 of the super-block, nibble n = g & 1 of ql[64 hh ..], bit pairs 4 n + {0, 2} of qh[32 hh ..]
  struct Pk { uint4 ql[4], qh[2]; uint32_t sc4, d; };
  __host__ __device__ static uint32_t src(uint32_t p) { return p; }
  // A block's 8 rows: [12 granules x 8 rows x 16 bytes of ql+qh][8 rows x 16 scales][8 x d].
  __device__ static void load(Pk &k, const QkLayout &L, const uint8_t *cb, uint32_t rr, uint32_t g,
                              uint32_t s) {
    const uint32_t hh = g >> 1;
    const uint8_t *p = blk_addr<210>(cb, s) + rr * 16;
#pragma unroll
    for (int i = 0; i < 4; i++) k.ql[i] = ldg16(p + (4 * hh + i) * 128);
    k.qh[0] = ldg16(p + (8 + 2 * hh) * 128), k.qh[1] = ldg16(p + (9 + 2 * hh) * 128);
    k.sc4 = __ldg(reinterpret_cast<const uint32_t *>(p + 1536 + 8 * hh + 4 * (g & 1u)));
    k.d = __ldg(reinterpret_cast<const unsigned short *>(p - rr * 16 + 1664) + rr);
  }
  __device__ static void prefetch(const QkLayout &L, const uint8_t *cb, uint32_t rr, uint32_t g, uint32_t s) {
    const uint32_t line = g * 8 + rr;  // 1680 bytes = up to 14 lines, one per thread of the row group
    if (line < 14) pf_l2(blk_addr<210>(cb, s) + line * 128);
  }
  struct Sc { __half2 s[4]; };
  __device__ static void scales(const Pk &k, uint32_t, Sc &c) {
    const float d = h2f_bits(k.d);
#pragma unroll
    for (int i = 0; i < 4; i++) c.s[i] = __float2half2_rn(d * (float)(int)(signed char)((k.sc4 >> (8 * i)) & 0xFF));
  }
  __device__ static void expand(const Pk &k, const Sc &c, uint32_t g, int hf, uint32_t o[4][4], uint32_t) {
    // half hf of the row-step = columns 32 hf .. + 32 of the group: ql bytes 32 hf + l, qh byte l, bit pair 4 n + 2 hf
    const __half2 off = __float2half2_rn(1056.f);  // (1024 + q) - 1056 = q - 32, exact; then one rounding in the product
    const uint32_t nsh = 4 * (g & 1u), hsh = 4 * (g & 1u) + 2 * hf;
#pragma unroll
    for (int i = 0; i < 4; i++) {
      const uint4 l4 = k.ql[2 * hf + (i >> 1)], h4 = k.qh[i >> 1];
#pragma unroll
      for (int e = 0; e < 2; e++) {
        const uint32_t lw = (i & 1) ? (e ? l4.w : l4.z) : (e ? l4.y : l4.x);
        const uint32_t hw = (i & 1) ? (e ? h4.w : h4.z) : (e ? h4.y : h4.x);
        const uint32_t q6 = ((lw >> nsh) & 0x0F0F0F0Fu) | (((hw >> hsh) & 0x03030303u) << 4);
        uint32_t a, b2;
        bytes_to_magic(q6, a, b2);
        const __half2 sc = c.s[2 * hf + ((2 * i + e) >> 2)];  // 16 columns per scale
        o[i][2 * e + 0] = h2_bits(__hmul2(__hsub2(bits_h2(a), off), sc));
        o[i][2 * e + 1] = h2_bits(__hmul2(__hsub2(bits_h2(b2), off), sc));
      }
    }
  }
};

template <>
struct WFmt<QK_T_IQ4_XS> {  // super-block of 256: f16 d, scales_h, scales_l[4], 128 nibble bytes (reference/iq4_xs.rs:47-97)
  // sub-block s = nibble bytes 16 s ..; byte j holds elements 2 j (low) and 2 j + 1 (high); value =
  // d (ls - 32) K[nibble] with the non-linear table K (iq_shared.rs:16-18).  A 256-entry table in
  // shared memory maps a byte straight to the half2 (K[low], K[high]) of its two adjacent elements.
  struct Pk { uint4 q[2]; uint2 h; };
  static constexpr bool HAS_LUT = true;
  __host__ __device__ static uint32_t src(uint32_t p) { return p; }
  __device__ static void fill_lut(uint32_t *lut, uint32_t tid, uint32_t nthreads) {
    const int K[16] = {-127, -104, -83, -65, -49, -35, -22, -10, 1, 13, 25, 38, 53, 69, 89, 113};
    for (uint32_t b = tid; b < 256; b += nthreads) {
      int lo = 0, hi = 0;
#pragma unroll
      for (int i = 0; i < 16; i++) lo = (int)(b & 15u) == i ? K[i] : lo, hi = (int)(b >> 4) == i ? K[i] : hi;
      lut[b] = h2_bits(__floats2half2_rn((float)lo, (float)hi));
    }
  }
  // A block's 8 rows: [8 granules x 8 rows x 16 nibble bytes][8 rows x 8 header bytes].
  __device__ static void load(Pk &k, const QkLayout &L, const uint8_t *cb, uint32_t rr, uint32_t g,
                              uint32_t s) {
    const uint8_t *p = blk_addr<136>(cb, s);
    k.q[0] = ldg16(p + (2 * g) * 128 + rr * 16), k.q[1] = ldg16(p + (2 * g + 1) * 128 + rr * 16);
    k.h = __ldg(reinterpret_cast<const uint2 *>(p + 1024 + rr * 8));
  }
  __device__ static void prefetch(const QkLayout &L, const uint8_t *cb, uint32_t rr, uint32_t g, uint32_t s) {
    const uint32_t line = g * 8 + rr;  // 1088 bytes = up to 9 lines
    if (line < 9) pf_l2(blk_addr<136>(cb, s) + line * 128);
  }
  struct Sc { __half2 dl[2]; };
  __device__ static void scales(const Pk &k, uint32_t g, Sc &c) {
    const float d = h2f_bits(k.h.x);
    const uint32_t sh = k.h.x >> 16, sl = k.h.y;
#pragma unroll
    for (int hf = 0; hf < 2; hf++) {
      const uint32_t sb = 2 * g + hf;
      const int ls = (int)(((sl >> (4 * sb)) & 0xFu) | (((sh >> (2 * sb)) & 3u) << 4));
      c.dl[hf] = __float2half2_rn(d * (float)(ls - 32));
    }
  }
  __device__ static void expand(const Pk &k, const Sc &c, uint32_t, int hf, uint32_t o[4][4], uint32_t lut) {
    const uint4 q = k.q[hf];
    const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
    for (int i = 0; i < 4; i++)
#pragma unroll
      for (int b = 0; b < 4; b++)
        o[i][b] = h2_bits(__hmul2(bits_h2(lds32(lut + (((w[i] >> (8 * b)) & 0xFFu) << 2))), c.dl[hf]));
  }
};

// ---------------------------------------------------------------- activations -> fp16
// X16[t][256 s + p] = x[t][256 s + SRC(p)] / scale[t] in fp16, where scale[t] is the power
// of two that puts the row's largest magnitude in [512, 1024): the division is exact, no
// activation overflows or falls into fp16's subnormals, and the epilogue multiplies the
// row of results by scale[t] again (also exact).  Rows t >= m and columns >= cols are
// zero.  One CTA per token row at a time: a pass for the maximum, a pass to convert.
// With zero_rows != 0 it also clears y[m][zero_rows] (row stride ldy), for the split-K
// launches, whose tiles add their partial sums into y.
template <int T>
__global__ void __launch_bounds__(256)
    qk_x16_kernel(const float *__restrict__ x, uint32_t m, uint32_t cols, uint32_t m_pad,
                  uint32_t Kp, __half *__restrict__ out, float *__restrict__ scales,
                  float *__restrict__ y, uint64_t ldy, uint32_t zero_rows, uint32_t cached,
                  const int *__restrict__ counts, uint32_t cap, uint32_t bn, const int *__restrict__ lists,
                  uint32_t list_stride, uint32_t list_div) {
  extern __shared__ __align__(16) float row[];  // the row, when it fits (cached != 0)
  __shared__ float red[8];
  pdl_launch_dependents();
  pdl_wait();
  if (zero_rows) {
    const uint64_t nz = (uint64_t)m * zero_rows;
    for (uint64_t i = blockIdx.x * 256ull + threadIdx.x; i < nz; i += (uint64_t)gridDim.x * 256)
      y[(i / zero_rows) * ldy + (i % zero_rows)] = 0.f;
  }
  const uint32_t per_row = Kp / 8;
  const bool vec = (cols & 3u) == 0 && ((uintptr_t)x & 15u) == 0;  // rows start 16-byte aligned
  for (uint32_t t = blockIdx.x; t < m_pad; t += gridDim.x) {
    // Grouped call (counts != nullptr): row t is row t % cap of group t / cap, live below the
    // group's count; rows of token blocks that hold no live row are never read and are skipped.
    bool live = t < m;
    const float *xr = x + (uint64_t)t * cols;
    if (counts) {
      const uint32_t e = t / cap, tl = t % cap, cnt = (uint32_t)counts[e];
      if ((tl / bn) * bn >= cnt) continue;  // block-uniform
      live = tl < cnt;
      if (lists && live) xr = x + (uint64_t)(lists[(uint64_t)e * list_stride + tl] / (int)list_div) * cols;
    }
    float amax = 0.f;
    __syncthreads();  // the previous row's readers of `row` and `red` are done
    if (live) {
      if (vec) {
        for (uint32_t k = threadIdx.x * 4; k < cols; k += 1024) {
          const float4 v = __ldg(reinterpret_cast<const float4 *>(xr + k));
          amax = fmaxf(fmaxf(amax, fmaxf(fabsf(v.x), fabsf(v.y))), fmaxf(fabsf(v.z), fabsf(v.w)));
          if (cached) *reinterpret_cast<float4 *>(row + k) = v;
        }
      } else {
        for (uint32_t k = threadIdx.x; k < cols; k += 256) {
          const float v = __ldg(xr + k);
          amax = fmaxf(amax, fabsf(v));
          if (cached) row[k] = v;
        }
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = amax;
    __syncthreads();
    amax = red[0];
#pragma unroll
    for (int w = 1; w < 8; w++) amax = fmaxf(amax, red[w]);
    float scale = 1.f;
    if (amax > 0.f && amax <= FLT_MAX) {  // finite and non-zero (a NaN row keeps scale 1 and stays NaN)
      int e;
      frexpf(amax, &e);  // amax = f * 2^e, f in [0.5, 1)
      scale = ldexpf(1.f, e - 10);
    }
    const float inv = 1.f / scale;  // a power of two: exact
    if (threadIdx.x == 0) scales[t] = scale;
    for (uint32_t c = threadIdx.x; c < per_row; c += 256) {
      __align__(16) __half h[8];
#pragma unroll
      for (int j = 0; j < 8; j++) {
        const uint32_t p = 8 * c + j;
        const uint32_t k = (p & ~255u) + WFmt<T>::src(p & 255u);
        float v = 0.f;
        if (live && k < cols) v = (cached ? row[k] : __ldg(xr + k)) * inv;
        h[j] = __float2half_rn(v);
      }
      *reinterpret_cast<uint4 *>(out + (uint64_t)t * Kp + 8ull * c) = *reinterpret_cast<const uint4 *>(h);
    }
  }
}

// ---------------------------------------------------------------- main kernel
// T: weight format.  BN: tokens per tile (the MMA's N).  RH: 128-row halves per tile;
// with RH = 2 one activation stage feeds the MMAs of both halves.
// TBU: token blocks per work unit.  With TBU = 2 a unit multiplies one expanded weight tile into
// two token blocks (two accumulators of BN columns: all of tensor memory at BN = 256), so the
// weights of a row block are expanded once for 512 tokens instead of twice.
template <int T, int BN, int RH, bool GRP, int TBU>
__global__ void __launch_bounds__(n_threads<T>(), 1)
    qk_gemm_tc_kernel(QkLayout L, const uint8_t *__restrict__ W,
                          const __grid_constant__ CUtensorMap xmap, const float *__restrict__ xscale,
                          float *__restrict__ y, uint64_t ldy, uint32_t m_tokens, uint32_t tok_blocks, uint32_t row_blocks,
                          uint32_t KS, unsigned *status, GemmSmem S, const __grid_constant__ QkGroups G) {
  extern __shared__ __align__(1024) unsigned char smem[];
  constexpr int NI = n_issuers<T>(), FIRST_DW = NI + 1, NTHREADS = n_threads<T>();
  const uint32_t sbase = smem_u32(smem);
  const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t NB = (uint32_t)S.b_stages;
  const uint32_t nsb_all = (L.cols + 255u) / 256u;  // super-blocks (256 columns) along K
  // Work unit t = (tile t % n_tiles, K split t / n_tiles): with KS > 1 a tile's K range is cut
  // into KS runs of super-blocks, done by different CTAs, which add their partial sums into y.
  const uint32_t n_tiles = tok_blocks * row_blocks, n_units = n_tiles * KS;
  auto sb_begin = [&](uint32_t t) { return (t / n_tiles) * nsb_all / KS; };
  auto sb_end = [&](uint32_t t) { return (t / n_tiles + 1) * nsb_all / KS; };
  // Grouped call: row block rb belongs to group rb / G.rbpg, whose weights are G.w[group] and
  // whose activation / output rows are token blocks group * G.tbpg .. of the padded arrays; a
  // unit whose token block lies beyond the group's row count is skipped by every role alike
  // (the counts do not change while the kernel runs).
  constexpr bool grouped = GRP;  // a separate instantiation: the one-matrix kernel keeps its registers
  // (tok_blocks counts work units along the tokens: TBU token blocks each)
  auto u_rb = [&](uint32_t t) { return (t % n_tiles) / tok_blocks; };
  auto u_tbl = [&](uint32_t t) { return ((t % n_tiles) % tok_blocks) * TBU; };
  auto u_group = [&](uint32_t t) { return grouped ? u_rb(t) / G.rbpg : 0u; };
  auto u_agroup = [&](uint32_t t) { return grouped ? u_group(t) % G.n_act : 0u; };  // whose activations it reads
  auto u_rows = [&](uint32_t t) { return grouped ? (uint32_t)__ldg(G.counts + u_agroup(t)) : m_tokens; };
  auto u_valid = [&](uint32_t t) { return !grouped || u_tbl(t) * BN < u_rows(t); };
  auto u_tb = [&](uint32_t t) { return grouped ? u_group(t) * G.tbpg + u_tbl(t) : u_tbl(t); };        // output rows
  auto u_tba = [&](uint32_t t) { return grouped ? u_agroup(t) * G.tbpg + u_tbl(t) : u_tbl(t); };     // activation rows
  constexpr uint32_t IDESC = (1u << 4) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
  // Accumulators: RH of BN columns per tile.  Where tensor memory holds two sets, the
  // MMAs of tile i+1 overlap the epilogue of tile i.  Every MMA accumulates; the
  // epilogue leaves the columns it has read zeroed.
  constexpr uint32_t ACC_COLS = RH * BN * TBU;  // accumulator columns of one unit
  constexpr uint32_t NBUF = 2 * ACC_COLS <= 512 ? 2 : 1;
  constexpr uint32_t TMEM_COLS = NBUF * ACC_COLS < 32 ? 32 : NBUF * ACC_COLS;
  // A half-stage units: each of the four groups writes its half-stages round-robin into
  // UPG units of its own.
  constexpr int UPG = RH == 1 ? QK_GEMM_UPG : 2 * RH;
  constexpr int NAU = 4 * UPG;

  pdl_launch_dependents();
  QK_GSTAMP(threadIdx.x == 0, 0);
  if (threadIdx.x == 0) {
    for (int s = 0; s < NAU; s++) {
      mbar_init(sbase + S.a_full + s * 8, 4);   // the four warps of the owning group
      mbar_init(sbase + S.a_empty + s * 8, 1);  // tcgen05.commit
    }
    for (uint32_t s = 0; s < 2 * MAX_RING; s++) mbar_init(sbase + S.b_full + s * 8, 1);  // expect_tx
    for (uint32_t s = 0; s < NB; s++) mbar_init(sbase + S.b_empty + s * 8, 1);           // tcgen05.commit
    for (int s = 0; s < 2; s++) {
      mbar_init(sbase + S.acc_full + s * 8, NI);  // one commit per issuing warp
      mbar_init(sbase + S.acc_empty + s * 8, NDW);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (WFmt<T>::HAS_LUT) WFmt<T>::fill_lut(reinterpret_cast<uint32_t *>(smem + S.lut), threadIdx.x, NTHREADS);
  if (warp == 0) {  // tensor memory for the accumulator columns
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     sbase + S.tmem_slot),
                 "r"(TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t *>(smem + S.tmem_slot);
  if (warp >= FIRST_DW && warp < FIRST_DW + 4) {  // zero the accumulators: lanes 32 (warp % 4) ..
    for (uint32_t c = 0; c < TMEM_COLS; c += 8)
      asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1,%1,%1,%1,%1,%1,%1,%1};" ::"r"(
                       tmem_base + ((32 * (warp & 3u)) << 16) + c),
                   "r"(0u)
                   : "memory");
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  // The weights are immutable, so the dequant warps start at once; the activation
  // producer (X16) and the epilogue (y, the activation scales) wait for the previous
  // kernel below, each before its first access.
  QK_GSTAMP(threadIdx.x == 0, 1);

  bool dead = false;
  if (warp == NI) {
    // ======================= activation producer =======================
    // Stage s is refilled when the MMAs of its previous use have retired.  Its "full"
    // barrier alternates between two per stage (by use parity), so that a consumer
    // waiting for use u can never mistake the completion of use u - 2 for it.
    if (lane == 0) {
      pdl_wait();  // X16 belongs to the previous kernel until it has finished
      uint32_t st = 0, use = 0, gstep = 0;
      for (uint32_t t = blockIdx.x; t < n_units && !dead; t += gridDim.x) {
        if (!u_valid(t)) continue;
        const uint32_t tb = u_tba(t);
        for (uint32_t step = sb_begin(t) * 4; step < sb_end(t) * 4 && !dead; step++, gstep++) {
#pragma unroll
          for (int j = 0; j < TBU; j++) {  // the step's tile of each token block of the unit, in consecutive stages
            if (use >= 1 && !mbar_wait_bounded(sbase + S.b_empty + st * 8, (use - 1) & 1u)) {
              dead = true;
              break;
            }
            const uint32_t bar = sbase + S.b_full + ((use & 1u) * MAX_RING + st) * 8;
            mbar_expect_tx(bar, BN * 128);
            tma_load_2d(sbase + S.b + st * S.b_stage, &xmap, (int)(step * 64), (int)((tb + (uint32_t)j) * BN), bar);
            if (++st == NB) st = 0, use++;
          }
          QK_GSTAMP(gstep < 256, 256 + gstep);
        }
      }
      if (dead) atomicOr(status, QK_DEV_TIMEOUT);
    }
  } else if (warp < NI) {
    // ======================= MMA issuers =======================
    // A tcgen05.mma occupies the tensor pipe for the same 128 cycles whatever its M and
    // N, and the thread that issues it is held until the pipe has taken it, its barrier
    // polls not hidden behind its own MMAs.  So several warps issue: with four, warp j the
    // steps of 64-column group j of every super-block; with three, warps 0 and 1 those of
    // groups 0 and 1 and warp 2 those of groups 2 and 3.  While one is held, the others poll
    // or queue behind it, and the pipe never waits for a poll.  A group's steps stay on one
    // warp, which therefore waits on the group's barriers in order and is never more than
    // one phase ahead of them.  All accumulate into the same columns (a tile's sum does not
    // depend on the order).
    if constexpr (NI == 4) {
      if (lane == 0) {
        const uint32_t me = warp;
        uint32_t bst = (me * TBU) % NB, buse = (me * TBU) / NB, usea = 0, i = 0;  // first of the TBU stages of this warp's next step
        uint32_t unit = 0, upar = 0;  // the group's next unit and the parity of its use count
        const uint32_t abar = sbase + S.a_full + me * UPG * 8, aebar = sbase + S.a_empty + me * UPG * 8;
        const uint32_t a0 = sbase + S.a + me * UPG * A_HALF;
        for (uint32_t t = blockIdx.x; t < n_units && !dead; t += gridDim.x) {
          if (!u_valid(t)) continue;
          const uint32_t buf = i % NBUF, use = i / NBUF, nsb = sb_end(t) - sb_begin(t);
          // the epilogue of the tile that last used these accumulators must have drained and zeroed them
          if (use >= 1 && !mbar_wait_bounded(sbase + S.acc_empty + buf * 8, (use - 1) & 1u)) {
            dead = true;
            break;
          }
          tc_fence_after();
          const uint32_t tmem_d = tmem_base + buf * ACC_COLS;
          for (uint32_t sbk = 0; sbk < nsb && !dead; sbk++, usea++) {
            const uint32_t bbar = sbase + S.b_full + ((buse & 1u) * MAX_RING + bst) * 8, bpar = (buse >> 1) & 1u;
            // the second token block's tile sits in the next stage (which may be the ring's first again)
            const uint32_t bst1 = bst + 1 == NB ? 0u : bst + 1, buse1 = bst + 1 == NB ? buse + 1 : buse;
            const uint32_t bbar1 = sbase + S.b_full + ((buse1 & 1u) * MAX_RING + bst1) * 8, bpar1 = (buse1 >> 1) & 1u;
            // both polls in flight together; the slow path only when one is not ready yet
            const bool a_ok = mbar_try_wait(abar + unit * 8, upar), b_ok = mbar_try_wait(bbar, bpar);
            if (!(a_ok && b_ok) && (!mbar_wait_bounded(abar + unit * 8, upar) || !mbar_wait_bounded(bbar, bpar))) {
              dead = true;
              break;
            }
            if (TBU == 2 && !mbar_wait_bounded(bbar1, bpar1)) {
              dead = true;
              break;
            }
            QK_GSTAMP(usea < 64, 512 + usea * 4 + me);
            const uint32_t b0 = sbase + S.b + bst * S.b_stage, b1 = sbase + S.b + bst1 * S.b_stage;
  #pragma unroll
            for (int rh = 0; rh < RH; rh++) {
  #pragma unroll
              for (int hf = 0; hf < 2; hf++) {
                if ((rh | hf) && !mbar_wait_bounded(abar + unit * 8, upar)) {
                  dead = true;
                  break;
                }
                const uint32_t au = a0 + unit * A_HALF;
                umma_f16(tmem_d + rh * BN, umma_desc_sw64(au), umma_desc(b0 + hf * 64), IDESC, 1u);
                umma_f16(tmem_d + rh * BN, umma_desc_sw64(au + 32), umma_desc(b0 + hf * 64 + 32), IDESC, 1u);
                if (TBU == 2) {  // the same weights into the second token block's accumulator
                  umma_f16(tmem_d + (RH + rh) * BN, umma_desc_sw64(au), umma_desc(b1 + hf * 64), IDESC, 1u);
                  umma_f16(tmem_d + (RH + rh) * BN, umma_desc_sw64(au + 32), umma_desc(b1 + hf * 64 + 32), IDESC, 1u);
                }
                umma_commit(aebar + unit * 8);  // the unit is free when these retire
                if (++unit == (uint32_t)UPG) unit = 0, upar ^= 1u;
              }
              if (dead) break;
            }
            if (dead) break;
            umma_commit(sbase + S.b_empty + bst * 8);
            if (TBU == 2) umma_commit(sbase + S.b_empty + bst1 * 8);
            bst += NI * TBU;
            while (bst >= NB) bst -= NB, buse++;
          }
          if (dead) break;
          umma_commit(sbase + S.acc_full + buf * 8);  // this warp's share of the tile has retired
          i++;
        }
        if (dead) atomicOr(status, QK_DEV_TIMEOUT);
      }
    } else {
      if (lane == 0) {
        const uint32_t me = warp;
        // Steps are numbered through the whole run of this CTA: step 4 q + g is the 64-column group g of
        // the q-th super-block it walks.  Everything a step needs follows from its number: the A units of
        // group g (2 RH half-units per super-block, round-robin over the group's UPG units) and the
        // TBU activation stages of the step (round-robin over the ring).
        uint32_t q = 0, i = 0;  // super-blocks and tiles done
        for (uint32_t t = blockIdx.x; t < n_units && !dead; t += gridDim.x) {
          if (!u_valid(t)) continue;
          const uint32_t buf = i % NBUF, use = i / NBUF, nsb = sb_end(t) - sb_begin(t);
          // the epilogue of the tile that last used these accumulators must have drained and zeroed them
          if (use >= 1 && !mbar_wait_bounded(sbase + S.acc_empty + buf * 8, (use - 1) & 1u)) {
            dead = true;
            break;
          }
          tc_fence_after();
          const uint32_t tmem_d = tmem_base + buf * ACC_COLS;
          for (uint32_t sbk = 0; sbk < nsb && !dead; sbk++, q++) {
            for (uint32_t g = 0; g < 4 && !dead; g++) {
              if ((g < 2 ? g : 2u) != me) continue;  // a group's steps always on the same warp, hence in order
              const uint32_t abar = sbase + S.a_full + g * UPG * 8, aebar = sbase + S.a_empty + g * UPG * 8;
              const uint32_t a0 = sbase + S.a + g * UPG * A_HALF;
              uint32_t h = q * (2 * RH);  // the group's half-units before this super-block
              const uint32_t tile = (q * 4 + g) * TBU;
              const uint32_t bst = tile % NB, buse = tile / NB;
              const uint32_t bbar = sbase + S.b_full + ((buse & 1u) * MAX_RING + bst) * 8, bpar = (buse >> 1) & 1u;
              // the second token block's tile sits in the next stage (which may be the ring's first again)
              const uint32_t bst1 = bst + 1 == NB ? 0u : bst + 1, buse1 = bst + 1 == NB ? buse + 1 : buse;
              const uint32_t bbar1 = sbase + S.b_full + ((buse1 & 1u) * MAX_RING + bst1) * 8, bpar1 = (buse1 >> 1) & 1u;
              {
                const uint32_t unit = h % (uint32_t)UPG, upar = (h / (uint32_t)UPG) & 1u;
                // both polls in flight together; the slow path only when one is not ready yet
                const bool a_ok = mbar_try_wait(abar + unit * 8, upar), b_ok = mbar_try_wait(bbar, bpar);
                if (!(a_ok && b_ok) && (!mbar_wait_bounded(abar + unit * 8, upar) || !mbar_wait_bounded(bbar, bpar))) {
                  dead = true;
                  break;
                }
              }
              if (TBU == 2 && !mbar_wait_bounded(bbar1, bpar1)) {
                dead = true;
                break;
              }
              const uint32_t b0 = sbase + S.b + bst * S.b_stage, b1 = sbase + S.b + bst1 * S.b_stage;
  #pragma unroll
              for (int rh = 0; rh < RH; rh++) {
  #pragma unroll
                for (int hf = 0; hf < 2; hf++, h++) {
                  const uint32_t unit = h % (uint32_t)UPG, upar = (h / (uint32_t)UPG) & 1u;
                  if ((rh | hf) && !mbar_wait_bounded(abar + unit * 8, upar)) {
                    dead = true;
                    break;
                  }
                  const uint32_t au = a0 + unit * A_HALF;
                  umma_f16(tmem_d + rh * BN, umma_desc_sw64(au), umma_desc(b0 + hf * 64), IDESC, 1u);
                  umma_f16(tmem_d + rh * BN, umma_desc_sw64(au + 32), umma_desc(b0 + hf * 64 + 32), IDESC, 1u);
                  if (TBU == 2) {  // the same weights into the second token block's accumulator
                    umma_f16(tmem_d + (RH + rh) * BN, umma_desc_sw64(au), umma_desc(b1 + hf * 64), IDESC, 1u);
                    umma_f16(tmem_d + (RH + rh) * BN, umma_desc_sw64(au + 32), umma_desc(b1 + hf * 64 + 32), IDESC, 1u);
                  }
                  umma_commit(aebar + unit * 8);  // the unit is free when these retire
                }
                if (dead) break;
              }
              if (dead) break;
              umma_commit(sbase + S.b_empty + bst * 8);
              if (TBU == 2) umma_commit(sbase + S.b_empty + bst1 * 8);
            }
          }
          if (dead) break;
          umma_commit(sbase + S.acc_full + buf * 8);  // this warp's share of the tile has retired
          i++;
        }
        if (dead) atomicOr(status, QK_DEV_TIMEOUT);
      }
    }
  } else if (warp >= FIRST_DW) {
    // ======================= dequant + epilogue warps =======================
    const uint32_t grp = (warp - FIRST_DW) >> 2;  // columns [64 grp, 64 grp + 64) of every super-block
    const uint32_t r = 32 * (warp & 3u) + lane;   // weight row inside a 128-row half = accumulator lane (a warp reads lanes 32 (warp % 4) ..)
    const uint32_t chunk_in_half = r >> 3, rr = r & 7u;
    // this row in the group's half-stage units: 64-byte rows, 16-byte chunk c at c ^ ((r >> 1) & 3)
    const uint32_t arow = sbase + S.a + grp * UPG * A_HALF + r * 64, asw = (r >> 1) & 3u;
    const uint32_t aaddr[4] = {arow + ((0u ^ asw) << 4), arow + ((1u ^ asw) << 4), arow + ((2u ^ asw) << 4),
                               arow + ((3u ^ asw) << 4)};
    const uint32_t a_full = sbase + S.a_full + grp * UPG * 8, a_empty = sbase + S.a_empty + grp * UPG * 8;
    uint32_t unit = 0, upar = 0, wrapped = 0;  // next unit, parity of its use count, whether it was used before
    // Epilogue of a finished tile, in pieces of 16 columns.  With two accumulator sets the
    // pieces go between the super-blocks of the next tile, so that the stores are spread
    // out and the MMAs stay fed; with one set the next tile's MMAs wait for them, so they
    // all go after the next tile's first super-block.  This warp reads accumulator lanes
    // 32 (warp % 4) .. + 32 and its group's share of the columns of every row half.
    constexpr int CPG = BN >= 128 ? BN / 4 : 32;  // columns per group
    constexpr uint32_t NCH1 = RH * CPG / 16;      // pieces per token block
    constexpr uint32_t NCH = TBU * NCH1;          // pieces per unit
    bool epi_active = false;
    uint32_t epi_it = 0, epi_rb = 0, epi_tb = 0, epi_next = 0;  // epi_rb: row block inside its matrix; epi_tb: token block of the padded arrays
    uint32_t epi_t0 = 0, epi_m = 0;                              // first token of the block inside its group, and the group's row count
    uint32_t epi_tba = 0;                                        // token block of the activation arrays (the scales)
    auto epi_piece = [&]() -> bool {
      const uint32_t buf = epi_it % NBUF;
      if (epi_it == 0 && epi_next == 0) pdl_wait();  // y and the activation scales: see above
      if (epi_next == 0) {
        if (!__all_sync(0xffffffffu, mbar_wait_bounded(sbase + S.acc_full + buf * 8, (epi_it / NBUF) & 1u)))
          return false;
        tc_fence_after();
        QK_GSTAMP(grp == 0 && (warp & 3u) == 0 && epi_it < 16, 1900 + epi_it);
      }
      const uint32_t tbj = epi_next / NCH1, piece = epi_next % NCH1;  // token block of the unit, piece inside it
      const uint32_t rh = piece / (CPG / 16);
      const int c0 = (int)grp * CPG + (int)(piece % (CPG / 16)) * 16;
      if ((int)grp * CPG < BN) {
        const uint32_t row = (epi_rb * RH + rh) * BM + r;
        const uint32_t taddr =
            tmem_base + ((32 * (warp & 3u)) << 16) + buf * ACC_COLS + (tbj * RH + rh) * BN + (uint32_t)c0;
        uint32_t v[16];
        asm volatile(
            "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
            "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
            : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]),
              "=r"(v[7]), "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]),
              "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
            : "r"(taddr));
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
        for (int c = 0; c < 16; c += 8)  // leave the columns zeroed for their next tile
          asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1,%1,%1,%1,%1,%1,%1,%1};" ::"r"(
                           taddr + (uint32_t)c),
                       "r"(0u)
                       : "memory");
        if (row < L.rows) {
          float *yp = y + (uint64_t)((epi_tb + tbj) * BN + c0) * ldy + row;
          const float *sp = xscale + (epi_tba + tbj) * BN + c0;  // the tokens' activation scales (inside the padded array)
          if (KS == 1) {
#pragma unroll
            for (int j = 0; j < 16; j++)
              if (epi_t0 + tbj * BN + c0 + j < epi_m) yp[(uint64_t)j * ldy] = __uint_as_float(v[j]) * __ldg(sp + j);
          } else {
#pragma unroll
            for (int j = 0; j < 16; j++)
              if (epi_t0 + tbj * BN + c0 + j < epi_m)
                atomicAdd(yp + (uint64_t)j * ldy, __uint_as_float(v[j]) * __ldg(sp + j));
          }
        }
      }
      if (++epi_next == NCH) {
        asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(sbase + S.acc_empty + buf * 8);
        QK_GSTAMP(grp == 0 && (warp & 3u) == 0 && epi_it < 16, 1920 + epi_it);
        epi_active = false;
      }
      return true;
    };

    // Packed weights come straight from global memory, one super-block ahead in registers
    // and PF_AHEAD super-blocks ahead as L2 prefetches.
    using F = WFmt<T>;
    constexpr uint32_t PF_AHEAD = 6;
    auto chunk_of = [&](uint32_t t, int rh) -> uint32_t {  // inside the unit's own matrix
      const uint32_t rbl = grouped ? u_rb(t) % G.rbpg : u_rb(t);
      const uint32_t chunk = (rbl * RH + rh) * 16 + chunk_in_half;
      return chunk < L.chunks ? chunk : L.chunks - 1;  // rows past the end: valid bytes, results unused
    };
    uint32_t it = 0, u = 0;  // u: super-blocks done = uses of each of this group's A units
    // cursor of the next super-block to load, and of the next one to prefetch
    uint32_t lt = blockIdx.x, pt = blockIdx.x;
    uint32_t lsb = 0, lse = 0, psb = 0, pse = 0;  // runs [lsb, lse), [psb, pse) of super-blocks
    const uint8_t *lchunk[RH], *pchunk[RH];       // and where their 8-row chunks start
    auto enter = [&](uint32_t &t, uint32_t &sb, uint32_t &se, const uint8_t **chunk) {
      while (t < n_units && !u_valid(t)) t += gridDim.x;  // the cursors skip what the main loop skips
      if (t >= n_units) return;
      sb = sb_begin(t), se = sb_end(t);
      const uint8_t *Wm = grouped ? G.w[u_group(t)] : W;
#pragma unroll
      for (int rh = 0; rh < RH; rh++) chunk[rh] = chunk_addr(L, Wm, chunk_of(t, rh));
    };
    enter(lt, lsb, lse, lchunk), enter(pt, psb, pse, pchunk);
    typename F::Pk nk[RH];
    auto load_next = [&]() {
      if (lt >= n_units) return;
#pragma unroll
      for (int rh = 0; rh < RH; rh++) F::load(nk[rh], L, lchunk[rh], rr, grp, lsb);
      if (++lsb == lse) lt += gridDim.x, enter(lt, lsb, lse, lchunk);
    };
    auto prefetch_next = [&](bool issue) {
      if (pt >= n_units) return;
      if (issue) {
#pragma unroll
        for (int rh = 0; rh < RH; rh++) F::prefetch(L, pchunk[rh], rr, grp, psb);
      }
      if (++psb == pse) pt += gridDim.x, enter(pt, psb, pse, pchunk);
    };
    load_next();
    for (uint32_t k = 0; k <= PF_AHEAD; k++) prefetch_next(k > 0);

    for (uint32_t t = blockIdx.x; t < n_units && !dead; t += gridDim.x) {
      if (!u_valid(t)) continue;
      const uint32_t rb = grouped ? u_rb(t) % G.rbpg : u_rb(t), tb = u_tb(t);
      const uint32_t nsb = sb_end(t) - sb_begin(t);
      for (uint32_t sbk = 0; sbk < nsb && !dead; sbk++, u++) {
        typename F::Pk pk[RH];
#pragma unroll
        for (int rh = 0; rh < RH; rh++) pk[rh] = nk[rh];
        load_next();
        prefetch_next(true);
#pragma unroll
        for (int rh = 0; rh < RH; rh++) {
          typename F::Sc sc;
          F::scales(pk[rh], grp, sc);
#pragma unroll
          for (int hf = 0; hf < 2; hf++) {
            uint32_t o[4][4];
            F::expand(pk[rh], sc, grp, hf, o, sbase + S.lut);
            // the MMAs that read this unit's previous contents must have retired
            if (wrapped && !__all_sync(0xffffffffu, mbar_wait_bounded(a_empty + unit * 8, upar ^ 1u))) {
              dead = true;  // warp-uniform: these warps execute .aligned tcgen05 instructions later
              break;
            }
#pragma unroll
            for (int i = 0; i < 4; i++)
              asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(aaddr[i] + unit * A_HALF), "r"(o[i][0]),
                           "r"(o[i][1]), "r"(o[i][2]), "r"(o[i][3])
                           : "memory");
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // generic writes -> MMA reads
            __syncwarp();
            if (lane == 0) mbar_arrive(a_full + unit * 8);
            if (++unit == (uint32_t)UPG) unit = 0, upar ^= 1u, wrapped = 1;
          }
          if (dead) break;
        }
        if (dead) break;
        // pieces of the previous tile's epilogue, once this tile's first stages are under way
        if (NBUF == 1) {
          while (epi_active && !dead)
            if (!epi_piece()) dead = true;
        } else if (epi_active && sbk >= 1 && !epi_piece()) {
          dead = true;
        }
      }
      while (epi_active && !dead)  // a tile too short to have carried all the pieces
        if (!epi_piece()) dead = true;
      epi_active = true, epi_it = it, epi_rb = rb, epi_tb = tb, epi_next = 0;
      epi_t0 = u_tbl(t) * BN, epi_m = u_rows(t), epi_tba = u_tba(t);
      it++;
    }
    while (epi_active && !dead)
      if (!epi_piece()) dead = true;
    if (dead && lane == 0) atomicOr(status, QK_DEV_TIMEOUT);
  }

  // common exit: the tensor memory is always returned
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (warp == 0)
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                 "r"(TMEM_COLS)
                 : "memory");
}

// ---------------------------------------------------------------- host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *,
                                  const cuuint64_t *, const cuuint64_t *, const cuuint32_t *,
                                  const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void *p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = (EncodeTiledFn)p;
  }
  return fn;
}

bool plan_gemm(int bn, int rh, GemmSmem *S, uint32_t *total) {
  uint32_t off = 0;
  GemmSmem s;
  s.a_full = off, off += 16 * 8;
  s.a_empty = off, off += 16 * 8;
  s.b_full = off, off += 2 * MAX_RING * 8;
  s.b_empty = off, off += MAX_RING * 8;
  s.acc_full = off, off += 16;
  s.acc_empty = off, off += 16;
  s.tmem_slot = off, off += 16;
  s.lut = off, off += 1024;  // byte -> half2 table of the formats that need one
  off = (off + 1023u) & ~1023u;
  s.a_stage = A_HALF;
  s.b_stage = (uint32_t)bn * 128;
  // What the fp16 weight units leave goes to the activation ring: a stage is refilled
  // only after the MMAs that read it have retired, so its depth is what hides the L2
  // latency of the tile loads.
  const uint32_t budget = 227u * 1024u;
  const uint32_t a_bytes = 4u * (rh == 1 ? QK_GEMM_UPG : 2u * rh) * A_HALF;
  int b_stages = (int)((budget - off - a_bytes) / s.b_stage);
  if (b_stages > MAX_RING) b_stages = MAX_RING;
  if (const char *e = qk_knob("QK_GEMM_BSTAGES")) {
    const int v = atoi(e);
    if (v >= 2 && v <= b_stages) b_stages = v;
  }
  if (b_stages < 2) return false;
  s.b_stages = b_stages;
  s.a = off, off += a_bytes;
  s.b = off, off += b_stages * s.b_stage;
  *S = s, *total = off;
  return true;
}

// Grouped call: the groups' weights and row counts, the rows reserved per group in the
// activation and output arrays, and (optionally) the lists the activation rows are gathered by.
struct GroupArgs {
  QkGroups G;
  uint32_t cap;
  const int *lists;
  uint32_t list_stride, list_div;
};

template <int T, int BN>
cudaError_t launch_gemm(const QkLayout &L, const uint8_t *W, const float *x, float *y, uint32_t m,
                        uint64_t ldy, unsigned *status, unsigned char *scratch, int sm_count,
                        cudaStream_t s, const GroupArgs *ga = nullptr) {
  // RH = 2 (256-row tiles, half the activation traffic per MMA) measured slower on B200
  // (76 us against 61 us at Q4_K 14336 x 4096, 512 tokens): its activation ring is only
  // three stages deep.  The kernel keeps the parameter; only RH = 1 is built.
  constexpr int RH = 1;
  GemmSmem S;
  uint32_t total;
  if (!plan_gemm(BN, RH, &S, &total)) return cudaErrorInvalidConfiguration;
  // Two token blocks per unit (the weights of a row block expanded once for both) where the
  // batch has an even number of 256-token blocks and the matrix still has units for most SMs
  // (measured: Q4_K 14336 x 4096 x 512, 112 units, 70.2 -> 64.2 us; Q8_0 4096^2 x 512, which then
  // needs four K splits instead of two, 36.9 -> 39.1 us); only built for BN = 256.
  constexpr bool HAS2 = BN == 256;
  const uint32_t units2 = ((L.rows + RH * BM - 1) / (RH * BM)) * (((m + BN - 1) / BN) / 2);
  // (four issuers two stages each: with fewer than four stages a stage would be three uses ahead of
  // its slowest reader, more than the two "full" barriers per stage tell apart)
  const bool two = HAS2 && !ga && S.b_stages >= 4 && m > (uint32_t)BN && ((m + BN - 1) / BN) % 2 == 0 &&
                   (units2 * 5 >= (uint32_t)sm_count * 3 || qk_knob("QK_GEMM_TBU2")) && !qk_knob("QK_GEMM_TBU1");
  auto kern = ga ? qk_gemm_tc_kernel<T, BN, RH, true, 1>
                 : (two ? qk_gemm_tc_kernel<T, BN, RH, false, HAS2 ? 2 : 1> : qk_gemm_tc_kernel<T, BN, RH, false, 1>);
  static QkPerDevice attr_set;
  if (attr_set.first()) {
    cudaError_t e = cudaFuncSetAttribute(qk_gemm_tc_kernel<T, BN, RH, false, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(qk_gemm_tc_kernel<T, BN, RH, true, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
    if (e == cudaSuccess && HAS2)
      e = cudaFuncSetAttribute(qk_gemm_tc_kernel<T, BN, RH, false, HAS2 ? 2 : 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
    if (e != cudaSuccess) return attr_set.reset(), e;
  }
  EncodeTiledFn enc = encode_fn();
  if (!enc) return cudaErrorNotSupported;
  const uint32_t Kp = ((L.cols + 255u) / 256u) * 256u;
  // grouped: m = rows reserved per group (a multiple of BN); the arrays hold G.n * m rows
  QkGroups G = {};
  uint32_t tok_blocks = (m + BN - 1) / BN, m_pad = tok_blocks * BN;
  uint32_t row_blocks = (L.rows + RH * BM - 1) / (RH * BM);
  if (ga) {
    G = ga->G;
    G.rbpg = row_blocks, G.tbpg = tok_blocks;
    m_pad = G.n_act * ga->cap;  // activation rows; the output has G.n * cap rows
    row_blocks *= G.n;
  }
  __half *x16 = reinterpret_cast<__half *>(scratch);
  float *xscale = reinterpret_cast<float *>(scratch + (((size_t)m_pad * Kp * 2 + 255) & ~(size_t)255));

  CUtensorMap map;
  cuuint64_t dims[2] = {Kp, m_pad};
  cuuint64_t strides[1] = {(cuuint64_t)Kp * 2};
  cuuint32_t box[2] = {BK, (cuuint32_t)BN};
  cuuint32_t estr[2] = {1, 1};
  if (enc(&map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, x16, dims, strides, box, estr,
          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
    return cudaErrorInvalidValue;

  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[0].val.programmaticStreamSerializationAllowed = 1;
  const uint64_t n8 = (uint64_t)m_pad * (Kp / 8);
  cudaLaunchConfig_t c0 = {};
  (void)n8;
  c0.gridDim = dim3(m_pad > 148u * 8u ? 148u * 8u : m_pad);
  c0.blockDim = dim3(256), c0.stream = s, c0.attrs = at, c0.numAttrs = 1;
  // Split K when the tiles alone would leave most SMs idle.  Partial sums meet in y
  // through atomic adds: bit-reproducible for two splits (a + b = b + a), order of
  // rounding not fixed for more.
  const uint32_t tok_units = two ? tok_blocks / 2 : tok_blocks;  // work units along the tokens
  const uint32_t n_tiles = tok_units * row_blocks, nsb = Kp / 256u;
  uint32_t ks = 1;
  if (n_tiles * 4 < (uint32_t)sm_count * 3 && !ga) ks = (uint32_t)sm_count / n_tiles;
  if (ks > 8) ks = 8;
  if (ks > nsb) ks = nsb;
  if (const char *ev = qk_knob("QK_GEMM_KS")) {
    const uint32_t v = (uint32_t)atoi(ev);
    if (v >= 1 && v <= 8 && v <= nsb) ks = v;
  }
  // the row is staged in shared memory between the maximum pass and the conversion when it fits
  // The row is staged in shared memory between the two passes (measured a little faster
  // than a second read, although a CTA holding shared memory cannot share an SM with a
  // matmul CTA starting under it); QK_X16_STAGE=0 turns the staging off.
  static const bool stage_rows = !(qk_knob("QK_X16_STAGE") && atoi(qk_knob("QK_X16_STAGE")) == 0);
  const uint32_t row_bytes = L.cols * 4u, cached = (stage_rows && row_bytes <= 96u * 1024u) ? 1u : 0u;
  static QkPerDevice x16_attr;
  if (x16_attr.first()) {
    cudaError_t ea = cudaFuncSetAttribute(qk_x16_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024);
    if (ea != cudaSuccess) return x16_attr.reset(), ea;
  }
  c0.dynamicSmemBytes = cached ? ((row_bytes + 15u) & ~15u) : 0u;
  cudaError_t e = cudaLaunchKernelEx(&c0, qk_x16_kernel<T>, x, m, L.cols, m_pad, Kp, x16, xscale, y, ldy,
                                     ks > 1 ? L.rows : 0u, cached, ga ? ga->G.counts : (const int *)nullptr,
                                     ga ? ga->cap : 0u, (uint32_t)BN, ga ? ga->lists : (const int *)nullptr,
                                     ga ? ga->list_stride : 0u, ga ? ga->list_div : 1u);
  if (e != cudaSuccess) return e;

  uint32_t grid = n_tiles * ks;
  if (grid > (uint32_t)sm_count) grid = sm_count;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid), cfg.blockDim = dim3(n_threads<T>()), cfg.dynamicSmemBytes = total, cfg.stream = s;
  cfg.attrs = at, cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kern, L, W, map, (const float *)xscale, y, ldy, m, tok_units, row_blocks, ks, status, S, G);
}

int pick_bn(uint32_t m) {
  if (const char *e = qk_knob("QK_GEMM_BN")) {  // developer knob: force the token-tile width
    const int v = atoi(e);
    if (v == 32 || v == 64 || v == 128 || v == 256) return v;
  }
  return m <= 32 ? 32 : m <= 64 ? 64 : m <= 128 ? 128 : 256;
}

template <int T>
cudaError_t launch_fmt(const QkLayout &L, const uint8_t *tiled, const float *x, float *y, uint32_t m,
                       uint64_t ldy, unsigned *status, unsigned char *scratch, int sm_count,
                       cudaStream_t s, const GroupArgs *ga = nullptr) {
  switch (pick_bn(m)) {
    case 32:
      return launch_gemm<T, 32>(L, tiled, x, y, m, ldy, status, scratch, sm_count, s, ga);
    case 64:
      return launch_gemm<T, 64>(L, tiled, x, y, m, ldy, status, scratch, sm_count, s, ga);
    case 128:
      return launch_gemm<T, 128>(L, tiled, x, y, m, ldy, status, scratch, sm_count, s, ga);
    default:
      return launch_gemm<T, 256>(L, tiled, x, y, m, ldy, status, scratch, sm_count, s, ga);
  }
}

cudaError_t launch_type(const QkLayout &L, const uint8_t *tiled, const float *x, float *y, uint32_t m,
                        uint64_t ldy, unsigned *status, unsigned char *scratch, int sm_count, cudaStream_t s,
                        const GroupArgs *ga) {
  switch (L.type) {
    case QK_T_Q4_K:
      return launch_fmt<QK_T_Q4_K>(L, tiled, x, y, m, ldy, status, scratch, sm_count, s, ga);
    case QK_T_Q8_0:
      return launch_fmt<QK_T_Q8_0>(L, tiled, x, y, m, ldy, status, scratch, sm_count, s, ga);
    case QK_T_Q4_0:
      return launch_fmt<QK_T_Q4_0>(L, tiled, x, y, m, ldy, status, scratch, sm_count, s, ga);
    case QK_T_Q6_K:
      return launch_fmt<QK_T_Q6_K>(L, tiled, x, y, m, ldy, status, scratch, sm_count, s, ga);
    case QK_T_IQ4_XS:
      return launch_fmt<QK_T_IQ4_XS>(L, tiled, x, y, m, ldy, status, scratch, sm_count, s, ga);
    default:
      return cudaErrorInvalidValue;
  }
}

}  // namespace

#ifdef QK_TRACE
extern "C" void qk_gemm_trace_set(unsigned long long *p) {
  cudaMemcpyToSymbol(qk_gemm_trace_buf, &p, sizeof(p));
}
#endif

bool qk_gemm_tc_supported(const QkLayout &L, uint32_t m) {
  const bool fmt = L.type == QK_T_Q4_K || L.type == QK_T_Q8_0 || L.type == QK_T_Q4_0 || L.type == QK_T_Q6_K ||
                   L.type == QK_T_IQ4_XS;
  return fmt && m >= 1 && L.rows >= 1 && L.nb >= 1;
}

size_t qk_gemm_tc_scratch_bytes(const QkLayout &L, uint32_t m) {
  const int bn = pick_bn(m);
  const uint64_t m_pad = ((m + bn - 1) / bn) * (uint64_t)bn;
  const size_t x16 = (size_t)(m_pad * ((L.cols + 255ull) / 256ull) * 256ull * 2ull);
  return ((x16 + 255) & ~(size_t)255) + (size_t)m_pad * 4;  // fp16 activations, then one scale per token
}

cudaError_t qk_launch_gemm_tc(const QkLayout &L, const uint8_t *tiled, const float *x, float *y,
                              uint32_t m, uint64_t ldy, unsigned *status, unsigned char *scratch,
                              int sm_count, cudaStream_t s) {
  return launch_type(L, tiled, x, y, m, ldy, status, scratch, sm_count, s, nullptr);
}

uint32_t qk_gemm_tc_group_cap(uint32_t max_rows_per_group) {
  const uint32_t bn = (uint32_t)pick_bn(max_rows_per_group ? max_rows_per_group : 1u);
  return ((max_rows_per_group + bn - 1) / bn) * bn + (max_rows_per_group ? 0u : bn);
}

size_t qk_gemm_tc_grouped_scratch_bytes(const QkLayout &L, uint32_t n_groups, uint32_t max_rows_per_group) {
  const uint64_t m_pad = (uint64_t)n_groups * qk_gemm_tc_group_cap(max_rows_per_group);
  const size_t x16 = (size_t)(m_pad * ((L.cols + 255ull) / 256ull) * 256ull * 2ull);
  return ((x16 + 255) & ~(size_t)255) + (size_t)m_pad * 4;
}

cudaError_t qk_launch_gemm_tc_grouped(const QkLayout &L, const uint8_t *const *tiled, uint32_t n_groups, uint32_t n_act,
                                      const int *counts_dev, uint32_t max_rows_per_group, const float *x,
                                      const int *lists, uint32_t list_stride, uint32_t list_div, float *y,
                                      uint64_t ldy, unsigned *status, unsigned char *scratch, int sm_count,
                                      cudaStream_t s) {
  if (n_groups == 0 || n_groups > QK_MAX_GROUPS || n_act == 0 || n_groups % n_act || !counts_dev ||
      !qk_gemm_tc_supported(L, 1))
    return cudaErrorInvalidValue;
  GroupArgs ga = {};
  ga.G.n = n_groups, ga.G.n_act = n_act, ga.G.counts = counts_dev;
  for (uint32_t e = 0; e < n_groups; e++) ga.G.w[e] = tiled[e];
  ga.cap = qk_gemm_tc_group_cap(max_rows_per_group);
  ga.lists = lists, ga.list_stride = list_stride, ga.list_div = list_div ? list_div : 1u;
  return launch_type(L, tiled[0], x, y, ga.cap, ldy, status, scratch, sm_count, s, &ga);
}
