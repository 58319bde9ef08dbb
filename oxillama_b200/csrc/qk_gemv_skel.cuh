// Decode-path dequant-dot (1..4 activation rows) on the integer tensor-core MMA: the part
// that is the same for every weight format.  A format's policy F (qk_dec_*.cuh) says how one
// 256-column span of eight weight rows lies in a tile, which registers hold it, how it is
// loaded and what the MMAs and the scaling are; everything else is here.
//
// The matvec is HBM-bound; what limits a CUDA-core version on this part is the
// issue rate of the per-weight multiply (dp4a runs at a quarter of the FP32
// rate here).  So the multiply-accumulate of every 32-weight group is handed to
// mma.sync.m16n8k32 (8-bit x s8 -> s32) and the CUDA cores only unpack weight bits and
// apply one scale per group.  The matrix is NOT reshaped into a GEMM: each MMA still
// computes plain row dot products, eight weight rows at a time.
//
// Activations are split per 32-column block as x ~= sx (D0 + D1/254 + D2/254^2)
// with |D| <= 127 (error <= amax * 6.1e-8), so the integer dots are exact and
// the result carries f32-grade accuracy.  The B operand's eight columns hold the three
// digits of two 32-weight groups (even columns one group, odd columns the other), so each
// lane of an MMA quad owns digit j = lane % 4 of both groups in fixed registers.
//
// qk_gemv_imma_kernel, persistent, one CTA per SM: a producer warp streams 8-row
// tiles into a ring of shared-memory stages with cp.async.bulk (mbarrier completion);
// the compute warps (8 in four groups; 12 in three for short matrices) first split x
// into the digit planes and scale table in shared memory, then a group takes every
// G-th chunk, each warp its share of the tile's 256-column spans, and leaves its row
// partials in a small ring; the producer warp sums a chunk's partials, writes the outputs
// (into y, or as tagged words into every rank's slots for a row-sharded layer) and refills
// the chunk's stages.  No CTA-wide barrier and no compute warp ever waits for another in
// steady state.  When M * K is too large for every CTA to redo the split, qk_xsplit_kernel
// does it once into a scratch image in global memory, which each CTA brings in with one
// more bulk copy.
// Both kernels use programmatic dependent launch: call i+1 is resident and has its first
// weight tiles (weights are immutable) under way before call i has finished;
// griddepcontrol.wait orders everything that touches x, y or the scratch image, and the
// rest of the ring is issued behind the activation loads, not ahead of them.  Every wait on an
// mbarrier is bounded: when one runs out the warp stops, QK_DEV_TIMEOUT is
// raised in the status word, and the other warps run into their own bounds.
#pragma once
#include <cstdlib>
#include <type_traits>

#include "qk_formats.cuh"
#include "qk_kernels.h"
#include "qk_peer.cuh"
#include "qk_pipe.cuh"

#ifdef QK_TRACE
// Developer build only: block 0 timestamps its pipeline into a global buffer.
extern __device__ unsigned long long *qk_trace_buf;
#define QK_STAMP(cond, idx)                                                        \
  do {                                                                             \
    if ((cond) && qk_trace_buf && blockIdx.x == 0 && (threadIdx.x & 31) == 0) {    \
      unsigned long long t__;                                                      \
      asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t__));                     \
      qk_trace_buf[idx] = t__;                                                     \
    }                                                                              \
  } while (0)
#else
#define QK_STAMP(cond, idx) do {} while (0)
#endif

namespace qkdec {

using namespace qkpipe;

constexpr int MAX_CW = 16;                      // compute warps: 8 or 16 (+ one producer warp)
constexpr uint32_t NBT = QK_TILE_ELEMS / 256;   // super-blocks per full k-tile (16)
constexpr int MAX_STAGE = 12;
constexpr int MAX_SLOT = MAX_STAGE + 1;

struct SmemMma {
  uint32_t full, redfull, xbar;  // mbarriers (8 B each)
  uint32_t prog;                 // chunks the reducer warp has read so far (one word, polled by the producer warp)
  uint32_t red, ximg, stage;
  uint32_t PS;         // digit plane stride, bytes
  uint32_t xs_off;     // offset of the (sx, Sx) table inside the x image
  uint32_t ximg_bytes;
};

// Loads at a compile-time byte offset from a register base: the offset rides in the
// instruction, where an address built in C++ costs an integer add per load.
template <int OFF>
__device__ __forceinline__ uint2 lds64o(uint32_t addr) {
  uint2 v;
  asm volatile("ld.shared.v2.u32 {%0,%1}, [%2+%3];" : "=r"(v.x), "=r"(v.y) : "r"(addr), "n"(OFF));
  return v;
}
template <int OFF>
__device__ __forceinline__ uint4 lds128o(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4+%5];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "r"(addr), "n"(OFF));
  return v;
}
template <int OFF>
__device__ __forceinline__ float4 lds128fo(uint32_t addr) {
  float4 v;
  asm volatile("ld.shared.v4.f32 {%0,%1,%2,%3}, [%4+%5];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "r"(addr), "n"(OFF));
  return v;
}
template <int I, int N, typename Fn>
__device__ __forceinline__ void static_for(Fn &&f) {
  if constexpr (I < N) {
    f(std::integral_constant<int, I>{});
    static_for<I + 1, N>(f);
  }
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mma_u8s8(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                         uint32_t a3, uint32_t b0, uint32_t b1) {
  asm(  // a pure function of its operands: left free for the scheduler to interleave
      "mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%10,%11,%12,%13};"
      : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0), "r"(0), "r"(0), "r"(0));
}
// Exact int -> float for |v| < 2^22 on the full-rate pipes (no I2F).
__device__ __forceinline__ float small_int_to_float(int v) {
  return __int_as_float(0x4B400000 + v) - 12582912.0f;
}

// Four activations of one 32-column block -> their three balanced base-254 digits, one
// packed word per digit plane: x ~ (amax / 127) (d0 + d1 / 254 + d2 / 254^2).  Adding
// 1.5 * 2^23 rounds to the nearest integer and leaves it, as two's complement, in the low
// mantissa byte; with |v| <= amax every digit lies in [-127, 127] without a clamp.  (Values
// that are not finite give arbitrary digits: the product is meaningless for them anyway.)
__device__ __forceinline__ void split_quad(const float (&v)[4], float inv, uint32_t &w0, uint32_t &w1,
                                           uint32_t &w2) {
  constexpr float MAGIC = 12582912.f;
  uint32_t b0[4], b1[4], b2[4];
#pragma unroll
  for (int i = 0; i < 4; i++) {
    const float t0 = fmaf(v[i], inv, MAGIC);
    const float r1 = fmaf(v[i], inv, -(t0 - MAGIC));  // exact residual of the first digit
    const float t1 = fmaf(r1, 254.f, MAGIC);
    const float r2 = fmaf(r1, 254.f, -(t1 - MAGIC));
    const float t2 = fmaf(r2, 254.f, MAGIC);
    b0[i] = __float_as_uint(t0), b1[i] = __float_as_uint(t1), b2[i] = __float_as_uint(t2);
  }
  w0 = __byte_perm(__byte_perm(b0[0], b0[1], 0x0040), __byte_perm(b0[2], b0[3], 0x0040), 0x5410);
  w1 = __byte_perm(__byte_perm(b1[0], b1[1], 0x0040), __byte_perm(b1[2], b1[3], 0x0040), 0x5410);
  w2 = __byte_perm(__byte_perm(b2[0], b2[1], 0x0040), __byte_perm(b2[2], b2[3], 0x0040), 0x5410);
}

// Activations e0 .. e0 + 3 of one row out of the tagged slots of a gathered buffer (columns
// past `cols` read as zero); false if a slot's tag did not arrive within the wait's bound.
__device__ __forceinline__ bool load_quad_slots(const unsigned long long *row, unsigned want, uint32_t e0,
                                                uint32_t cols, float (&v)[4]) {
  if (e0 + 4 <= cols) return qkpeer::slot_wait4(row + e0, want, v);
  bool ok = true;
#pragma unroll
  for (int i = 0; i < 4; i++) {
    v[i] = 0.f;
    if (e0 + i < cols) ok &= qkpeer::slot_wait(row + e0 + i, want, v[i]);
  }
  return ok;
}

// ---------------------------------------------------------------- x image
// [M][3 digit planes of PS bytes, columns in the format's order F::store_digits][M][Kp/32] scale entries
// of F::XSB bytes: (sx, sum over the 32 columns) and, for formats with 16-column scales, the two half sums
template <class F>
__global__ void __launch_bounds__(256)
    qk_xsplit_kernel(const float *__restrict__ x, uint32_t m_rows, uint32_t cols, uint32_t Kp,
                     uint32_t PS, uint32_t xs_off, unsigned char *__restrict__ img,
                     const unsigned long long *wait_slots, const unsigned *wait_epoch, uint64_t wait_ld,
                     unsigned *status) {
  pdl_launch_dependents();
  pdl_wait();  // x may be the previous kernel's output; the image may still be in use by it
  const uint32_t quads = Kp / 4, total = m_rows * quads;
  const uint32_t it = blockIdx.x * 256 + threadIdx.x;
  if (it >= total) return;  // warp-uniform: total is a multiple of 64
  const uint32_t m = it / quads, e0 = (it % quads) * 4;
  float v[4];
  if (wait_slots) {  // x is gathered from other GPUs: read it from the tagged slots as it arrives
    if (!load_quad_slots(wait_slots + (uint64_t)m * wait_ld, *wait_epoch, e0, cols, v)) atomicOr(status, QK_DEV_TIMEOUT);
  } else {
#pragma unroll
    for (int i = 0; i < 4; i++) v[i] = (e0 + i < cols) ? __ldg(x + (uint64_t)m * cols + e0 + i) : 0.f;
  }
  float amax = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));
  float s4 = (v[0] + v[1]) + (v[2] + v[3]);
#pragma unroll
  for (int o = 1; o < 8; o <<= 1)  // the 8 threads of one 32-column block
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  s4 += __shfl_xor_sync(0xffffffffu, s4, 1);
  s4 += __shfl_xor_sync(0xffffffffu, s4, 2);  // this thread's 16-column half
  const float other = __shfl_xor_sync(0xffffffffu, s4, 4);
  if (!(amax < 8.0e37f)) amax = 8.0e37f;  // inf/nan/huge x: keep the scale finite (__fdividef: y < 2^126)
  const float inv = amax > 0.f ? __fdividef(127.f, amax) : 0.f;
  uint32_t w0, w1, w2;
  split_quad(v, inv, w0, w1, w2);
  F::store_digits(img + (size_t)m * 3 * PS, PS, e0, w0, w1, w2);
  if ((threadIdx.x & 7) == 0)
    F::store_xs(img + xs_off, (size_t)m * (Kp / 32) + e0 / 32, amax * (1.f / 127.f), s4 + other, s4, other);
}

// ---------------------------------------------------------------- main kernel
// The same split as qk_xsplit_kernel, done by the compute warps straight into the
// CTA's shared-memory x image (used when x is small enough that every CTA
// redoing it is cheaper than a second kernel and a copy).
template <class F, int M, int CW, bool PEER>
__device__ void xsplit_in_cta(const float *__restrict__ x, uint32_t cols, uint32_t Kp,
                              unsigned char *img, uint32_t PS, uint32_t xs_off, bool tell_producer,
                              const QkPeers &peers, unsigned *status) {
  constexpr int CT = CW * 32;  // compute threads
  const uint32_t quads = Kp / 4, total = (uint32_t)M * quads;
  // Every CTA of the grid reads the same few KB of x at the same moment: each starts at
  // a different 32-column block (whole blocks, so the 8 threads of a block stay together)
  // to spread the requests over the L2 slices, and loads 16 bytes at a time when it can.
  const uint32_t rot = (blockIdx.x * 40u) % total;  // a multiple of 8 quads
  const bool vec = (cols & 3u) == 0 && ((uintptr_t)x & 15u) == 0;
  const bool from_slots = PEER && peers.wait_slots != nullptr;
  const unsigned want = from_slots ? *peers.wait_epoch : 0u;
  bool arrived = true;  // false once a slot has failed to arrive in time: this thread waits no more
  constexpr int U = (M * 4096 / 4 + CT - 1) / CT < 4 ? (M * 4096 / 4 + CT - 1) / CT : 4;  // quads in flight per thread
  for (uint32_t base = 0; base < total; base += CT * U) {
    float v[U][4];
    uint32_t qidx[U];
#pragma unroll
    for (int j = 0; j < U; j++) {
      const uint32_t it0 = base + j * CT + threadIdx.x;
      uint32_t it = it0 + rot;
      if (it >= total) it -= total;
      qidx[j] = it0 < total ? it : 0xFFFFFFFFu;
      const uint32_t m = M == 1 ? 0u : it / quads, e0 = (M == 1 ? it : it % quads) * 4;
      if (from_slots) {  // gathered activations: straight from the tagged slots, as they arrive
        v[j][0] = v[j][1] = v[j][2] = v[j][3] = 0.f;
        if (it0 < total && arrived &&
            !load_quad_slots(peers.wait_slots + (uint64_t)m * peers.wait_ld, want, e0, cols, v[j])) {
          arrived = false;
          atomicOr(status, QK_DEV_TIMEOUT);
        }
      } else if (it0 < total && vec && e0 + 4 <= cols) {
        const float4 q = __ldg(reinterpret_cast<const float4 *>(x + (uint64_t)m * cols + e0));
        v[j][0] = q.x, v[j][1] = q.y, v[j][2] = q.z, v[j][3] = q.w;
      } else {
#pragma unroll
        for (int i = 0; i < 4; i++)
          v[j][i] = (it0 < total && e0 + i < cols) ? __ldg(x + (uint64_t)m * cols + e0 + i) : 0.f;
      }
    }
    // This thread's first activation loads are on their way: the producer may send the rest
    // of the ring behind them.
    if (tell_producer && base == 0) asm volatile("bar.arrive 2, %0;" ::"n"((CW + 1) * 32) : "memory");
#pragma unroll
    for (int j = 0; j < U; j++) {
      const uint32_t it = qidx[j];
      if (it == 0xFFFFFFFFu) continue;  // warp-uniform: total and CT are multiples of 32
      const uint32_t m = M == 1 ? 0u : it / quads, e0 = (M == 1 ? it : it % quads) * 4;
      float amax = fmaxf(fmaxf(fabsf(v[j][0]), fabsf(v[j][1])), fmaxf(fabsf(v[j][2]), fabsf(v[j][3])));
      float s4 = (v[j][0] + v[j][1]) + (v[j][2] + v[j][3]);
#pragma unroll
      for (int o = 1; o < 8; o <<= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
      s4 += __shfl_xor_sync(0xffffffffu, s4, 1);
      s4 += __shfl_xor_sync(0xffffffffu, s4, 2);  // this thread's 16-column half
      const float other = __shfl_xor_sync(0xffffffffu, s4, 4);
      if (!(amax < 8.0e37f)) amax = 8.0e37f;
      QK_STAMP(threadIdx.x == 0 && j == 0 && amax >= 0.f, 122);
      const float inv = amax > 0.f ? __fdividef(127.f, amax) : 0.f;
      uint32_t w0, w1, w2;
      split_quad(v[j], inv, w0, w1, w2);
      F::store_digits(img + (size_t)m * 3 * PS, PS, e0, w0, w1, w2);
      if ((threadIdx.x & 7) == 0)
        F::store_xs(img + xs_off, (size_t)m * (Kp / 32) + e0 / 32, amax * (1.f / 127.f), s4 + other, s4, other);
    }
  }
}

// The previous sharded call's gathered result, from its tagged slots into its plain buffer:
// the calling warps of all CTAs share the slots, eight loads in flight per lane; a slot whose
// tag has not arrived yet is waited for (bounded).
__device__ __forceinline__ void unpack_slots(const QkPeers &peers, unsigned uwant, uint32_t lane, unsigned *status) {
  const uint64_t stride = (uint64_t)gridDim.x * 32;
  bool arrived = true;
  for (uint64_t base = (uint64_t)blockIdx.x * 32 + lane; base < peers.unpack_n; base += 8 * stride) {
    unsigned long long w[8];
#pragma unroll
    for (int j = 0; j < 8; j++) {
      const uint64_t i = base + j * stride;
      w[j] = i < peers.unpack_n ? qkpeer::slot_load(peers.unpack_slots + i) : 0ull;
    }
#pragma unroll
    for (int j = 0; j < 8; j++) {
      const uint64_t i = base + j * stride;
      if (i >= peers.unpack_n) break;
      float v = __uint_as_float((unsigned)w[j]);
      if ((unsigned)(w[j] >> 32) != uwant) {  // not there yet: the bounded wait
        if (arrived && !qkpeer::slot_wait(peers.unpack_slots + i, uwant, v)) {
          arrived = false;
          atomicOr(status, QK_DEV_TIMEOUT);
        }
        if (!arrived) v = 0.f;
      }
      peers.unpack_out[i] = v;
    }
  }
}

// PEER: the variant that can store its results into every rank's tagged slots and read
// gathered activations out of slots (kept out of the single-GPU variant, whose speed is
// sensitive to its code size).
// F: the weight format's policy (tile geometry, register image of one 256-column span,
// its loads and its arithmetic; see qk_dec_*.cuh).
// MODE: 0 = one matrix, results into y; 1 = the same with the sharded-layer fan-out (the
// old PEER: results as tagged words into every rank's slots, activations optionally out of
// slots); 2 = two matrices of the same shape and format at once, W as the gate and W2 as the
// up projection of a feed-forward block: a CTA's chunks alternate (gate rows 8 i .., up rows
// 8 i ..), both see the same split activations, and the reducer writes
// silu(gate) * up (crates/oxillama-arch/src/common/swiglu.rs:15-21) where a plain matvec
// writes its dot products.
template <class F, int M, bool INCTA, int CW, int G, int MODE>
__global__ void __launch_bounds__((CW + 1 + (F::SPLIT_PRODUCER ? 1 : 0) + (MODE == 1 ? 1 : 0)) * 32, 1)
    qk_gemv_imma_kernel(QkLayout L, const uint8_t *__restrict__ W, const uint8_t *__restrict__ W2,
                           const float *__restrict__ x,
                           const unsigned char *__restrict__ ximg_g, float *__restrict__ y,
                           uint64_t ldy, unsigned *status, int nstage, int nslot,
                           uint32_t stage_bytes, SmemMma S, uint32_t Kp, QkPeers peers, int npre) {
  constexpr int WG = CW / G;  // warps per group; a group owns every G-th chunk
  // The tile producer as a warp of its own (F::SPLIT_PRODUCER) or as a second job of the reducer
  // warp: measured per format (Q4_K 14336 x 4096: 8.2 -> 7.8 us with its own warp; Q6_K
  // 128256 x 4096: 85 -> 90 us).
  constexpr bool SPLIT = F::SPLIT_PRODUCER;
  constexpr int XW = CW + 1 + (SPLIT ? 1 : 0);  // first warp behind the compute, reducer and producer warps
  constexpr bool PEER = MODE == 1, DUAL = MODE == 2;
  extern __shared__ __align__(128) unsigned char smem[];
  const uint32_t sbase = smem_u32(smem);
  const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  // chunks of this CTA, in the order it takes them; with two matrices every 8-row group counts twice
  const uint32_t my_chunks =
      (blockIdx.x < L.chunks ? (L.chunks - blockIdx.x + gridDim.x - 1) / gridDim.x : 0) * (DUAL ? 2u : 1u);
  const uint32_t my_items = my_chunks * L.ktiles;

  QK_STAMP(warp == 0, 0);
  pdl_launch_dependents();
  if (threadIdx.x == 0) {
    for (int s = 0; s < nstage; s++) mbar_init(sbase + S.full + s * 8, 1);
    for (int s = 0; s < nslot; s++) mbar_init(sbase + S.redfull + s * 8, WG);
    mbar_init(sbase + S.xbar, 1);
    *reinterpret_cast<volatile uint32_t *>(smem + S.prog) = 0u;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  __syncthreads();

  // tile issue state and helpers of whichever warp streams the tiles
  uint32_t pc = 0, pkt = 0, pst = 0;  // chunk ordinal, k-tile and stage of the next item
  const uint64_t policy = stream_policy();
  auto issue = [&]() {                // lane 0 only
    const uint32_t chunk = blockIdx.x + (DUAL ? pc >> 1 : pc) * gridDim.x;
    const uint8_t *Wc = (DUAL && (pc & 1u)) ? W2 : W;
    const uint32_t bytes = QK_TILE_ROWS * qk_tile_nb(L, pkt) * L.bb;
    const uint32_t bar = sbase + S.full + pst * 8;
    mbar_expect_tx(bar, bytes);
    bulk_g2s_stream(sbase + S.stage + pst * stage_bytes, Wc + qk_tile_offset(L, chunk, pkt), bytes, bar, policy);
    if (++pkt == L.ktiles) pkt = 0, pc++;
    if (++pst == (uint32_t)nstage) pst = 0;
  };
  uint32_t item = 0;  // items issued so far; kept in step by every lane
  auto issue_upto = [&](uint32_t limit) {
    const uint32_t end = limit < my_items ? limit : my_items;
    if (lane == 0)
      for (uint32_t i = item; i < end; i++) issue();
    if (end > item) item = end;
  };
  if (SPLIT && warp == CW + 1) {
    // ================= producer warp =================
    // Lane 0 streams the tiles: the first ring fill, then the k-tiles of chunk c + (ring depth)
    // as soon as the compute warps have handed chunk c over (they are done with its stages
    // then).  A warp of its own, because a copy instruction does not return until the copy
    // unit has room for it -- a third of a microsecond and more under a saturated stream --
    // and behind the reducer's sums the refills went out up to 1.7 us late, leaving the
    // stream idle between the first ring fill and the refills.  The producer stays at most
    // one chunk ahead of the reducer (S.prog), which is what makes the ring of `nslot`
    // partial buffers safe: chunk c + nslot cannot be computed, let alone handed over,
    // before the reducer has read chunk c.
    issue_upto((uint32_t)npre);  // weights are immutable: their prefetch need not wait for the previous kernel
    pdl_wait();                  // the x image belongs to the previous kernel until it has finished
    if (!INCTA && lane == 0) {
      mbar_expect_tx(sbase + S.xbar, S.ximg_bytes);
      bulk_g2s(sbase + S.ximg, ximg_g, S.ximg_bytes, sbase + S.xbar);
    }
    if (npre < nstage) {
      // The rest of the first ring fill goes out once the compute warps' activation loads
      // have landed (named barrier 2), so that those loads do not queue behind a whole
      // ring of weight tiles from every CTA: measured 11.1 -> 9.7 us per launch at 14336 x 4096.
      if (INCTA) asm volatile("bar.sync 2, %0;" ::"n"((CW + 1) * 32) : "memory");
      issue_upto((uint32_t)nstage);
    }
    uint32_t slot = 0, sph = 0;
    const volatile uint32_t *prog = reinterpret_cast<const volatile uint32_t *>(smem + S.prog);
    for (uint32_t c = 0; c < my_chunks && item < my_items; c++) {
      if (!mbar_wait_bounded(sbase + S.redfull + slot * 8, sph)) {  // chunk c handed over
        if (lane == 0) atomicOr(status, QK_DEV_TIMEOUT);
        break;
      }
      unsigned long long t0 = 0;
      uint32_t polls = 0;
      bool dead = false;
      while (*prog < c) {  // the reducer has read the chunks before c
        if ((++polls & 1023u) == 0) {
          unsigned long long t;
          asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
          if (!t0) t0 = t;
          if (t - t0 > 250000000ull) {
            dead = true;
            break;
          }
        }
      }
      if (dead) {
        if (lane == 0) atomicOr(status, QK_DEV_TIMEOUT);
        break;
      }
      issue_upto(item + L.ktiles);
      if (++slot == (uint32_t)nslot) slot = 0, sph ^= 1;
    }
    return;
  }

  if (warp == CW) {
    // ================= reducer warp (and, without a producer warp, the tile producer) =================
    // When a chunk's partials are complete the warp sums them and writes the 8 x M outputs
    // (or stores them into every rank's slots), then says so in S.prog.  Where it also streams
    // the tiles (!SPLIT) it refills the chunk's stages first: gating the refills on the
    // reduction bounds how far the compute warps can run ahead, which is what makes the ring
    // of `nslot` partial buffers safe without a second handshake.
    if (!SPLIT) issue_upto((uint32_t)npre);  // weights are immutable: their prefetch need not wait for the previous kernel
    pdl_wait();  // the x image and y belong to the previous kernel until it has finished
    QK_STAMP(true, 120);
    if (!SPLIT && !INCTA && lane == 0) {
      mbar_expect_tx(sbase + S.xbar, S.ximg_bytes);
      bulk_g2s(sbase + S.ximg, ximg_g, S.ximg_bytes, sbase + S.xbar);
    }
    // Sharded output: this call's tag is the object's call count + 1.  Lane 0 reads the
    // count, then counts this CTA in (the add carries a dependency on the value read, so it
    // cannot overtake the read); the CTA that is counted in last knows that every CTA of the
    // launch has read the count and moves it on.  The round trips run while the compute
    // warps load the activations; nothing of this sits at the end of the kernel.
    unsigned e_count = 0, uwant = 0;
    if (PEER && peers.unpack_n)  // needed further down; asked for now, together with the count
      asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(uwant) : "l"(peers.unpack_epoch) : "memory");
    if (PEER && peers.n && lane == 0) {
      unsigned one;
      asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(e_count) : "l"(peers.epoch) : "memory");
      asm volatile("and.b32 %0, %1, 0;\n\tadd.u32 %0, %0, 1;" : "=r"(one) : "r"(e_count));
      if (atomicAdd(peers.counter, one) == gridDim.x - 1) {
        *reinterpret_cast<volatile unsigned *>(peers.counter) = 0;
        *reinterpret_cast<volatile unsigned *>(peers.epoch) = e_count + 1u;
      }
    }
    if (!SPLIT && npre < nstage) {
      // the rest of the first ring fill, once the activation loads are out (see the producer warp)
      if (INCTA) asm volatile("bar.sync 2, %0;" ::"n"((CW + 1) * 32) : "memory");
      issue_upto((uint32_t)nstage);
    }
    const unsigned tag = (PEER && peers.n) ? __shfl_sync(0xffffffffu, e_count, 0) + 1u : 0u;
    // this lane's two destination ranks (lane / 8 and lane / 8 + 4), held in registers: an
    // indexed read of the kernel parameters per chunk costs a constant-cache miss each time
    unsigned long long *slots_a = nullptr, *slots_b = nullptr;
    if (PEER && peers.n) {
      const uint32_t q = lane >> 3;
#pragma unroll
      for (uint32_t p = 0; p < QK_MAX_PEERS; p++) {
        if (p == q && p < peers.n) slots_a = peers.slots[p];
        if (p == q + 4 && p < peers.n) slots_b = peers.slots[p];
      }
    }
    // In passing: the previous sharded call's gathered result goes from its slots into its
    // plain buffer -- by a warp of its own when the launch has one (see below), else here,
    // where this warp has nothing else to do until the first chunk is reduced.
    if (PEER && peers.unpack_n && blockDim.x == XW * 32) unpack_slots(peers, uwant, lane, status);
    uint32_t slot = 0, sph = 0;
    float gate_v = 0.f;  // two matrices: the gate chunk's sum, kept until the up chunk's arrives
    for (uint32_t c = 0; c < my_chunks; c++) {
      if (!mbar_wait_bounded(sbase + S.redfull + slot * 8, sph)) {
        if (lane == 0) atomicOr(status, QK_DEV_TIMEOUT);
        break;
      }
      // (!SPLIT) every warp of the owning group released the chunk's stages before it posted its
      // partials: refill them first, the sums and stores below follow the copies out
      if (!SPLIT) issue_upto(item + L.ktiles);
      const float *red = reinterpret_cast<const float *>(smem + S.red) + slot * (WG * M * 8);
      float v = 0.f;
      if (PEER && M == 1 && peers.n) {
        // One activation row, sharded output: every lane sums the row it stores (lane (q, r):
        // row r, for ranks q and q + 4), so that no shuffle sits between the sums and the
        // stores -- the last chunks of a CTA are reduced one after the other, and what each
        // costs here is the tail of the launch.
        const uint32_t r = lane & 7u, row = (blockIdx.x + c * gridDim.x) * 8 + r;
#pragma unroll
        for (int wv = 0; wv < WG; wv++) v += red[wv * 8 + r];
        if (row < L.rows) {
          if (slots_a) qkpeer::slot_store(slots_a + row, v, tag);
          if (slots_b) qkpeer::slot_store(slots_b + row, v, tag);
        }
      } else if (lane < 8 * M) {
        const uint32_t m = lane >> 3, r = lane & 7u;
#pragma unroll
        for (int wv = 0; wv < WG; wv++) v += red[(wv * M + m) * 8 + r];
        const uint32_t row = (blockIdx.x + (DUAL ? c >> 1 : c) * gridDim.x) * 8 + r;
        if (DUAL) {
          if ((c & 1u) == 0) {
            gate_v = v;
          } else if (row < L.rows) {
            // swiglu_inplace: sigmoid = 1 / (1 + exp(-g)); g * sigmoid * u, each step rounded
            const float sg = __fdiv_rn(1.f, __fadd_rn(1.f, expf(-gate_v)));
            y[(uint64_t)m * ldy + row] = __fmul_rn(__fmul_rn(gate_v, sg), v);
          }
        } else if (!(PEER && peers.n) && row < L.rows) {
          y[(uint64_t)m * ldy + row] = v;
        }
      }
      if (PEER && peers.n && M > 1) {
        // The same (value, tag) word into the slot of every rank: lane (q, r) stores row r
        // to ranks q, q + 4 (eight consecutive slots = 64 bytes per rank and activation row).
        const uint32_t r = lane & 7u, row = (blockIdx.x + c * gridDim.x) * 8 + r;
#pragma unroll
        for (int m = 0; m < M; m++) {
          const float vm = __shfl_sync(0xffffffffu, v, m * 8 + (int)r);
          if (row < L.rows) {
            if (slots_a) qkpeer::slot_store(slots_a + (uint64_t)m * ldy + row, vm, tag);
            if (slots_b) qkpeer::slot_store(slots_b + (uint64_t)m * ldy + row, vm, tag);
          }
        }
      }
      __syncwarp();
      if (SPLIT && lane == 0) *reinterpret_cast<volatile uint32_t *>(smem + S.prog) = c + 1u;  // read: its slot may be written again
      QK_STAMP(c < 30, 64 + c);
      if (++slot == (uint32_t)nslot) slot = 0, sph ^= 1;
    }
    return;
  }

  if (PEER && warp == XW) {
    // ================= unpack warp (launched only when there is something to unpack) =================
    // On the producer / reducer warp the unpacking (two or three rounds of slot loads, about
    // a microsecond each) held up the first reductions; a warp of its own runs beside them.
    pdl_wait();
    if (peers.unpack_n) {
      unsigned uwant;
      asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(uwant) : "l"(peers.unpack_epoch) : "memory");
      unpack_slots(peers, uwant, lane, status);
    }
    return;
  }

  // ================= compute warps =================
  const uint32_t group = warp / WG, wl = warp % WG;
  const uint32_t g = lane >> 2, tig = lane & 3;
  typename F::Lane LN;  // this lane's constants: which bytes, digits and scales it handles
  LN.init(lane, wl, sbase + S.ximg, S.PS, S.xs_off, Kp);

  pdl_wait();  // x may be the previous kernel's output; y may be read or written by it
  QK_STAMP(warp == 0, 121);
  bool dead = false;
  if (INCTA) {
    xsplit_in_cta<F, M, CW, PEER>(x, L.cols, Kp, smem + S.ximg, S.PS, S.xs_off, npre < nstage, peers, status);
    QK_STAMP(warp == 0, 123);
    asm volatile("bar.sync 1, %0;" ::"n"(CW * 32) : "memory");  // compute warps only
  } else if (!mbar_wait_bounded(sbase + S.xbar, 0)) {
    dead = true;
  }
  float acc[M][3];  // per activation row: the format's running sums (see F::compute / F::finish)
#pragma unroll
  for (int m = 0; m < M; m++) acc[m][0] = acc[m][1] = acc[m][2] = 0.f;
  using Data = typename F::template Data<M>;

  QK_STAMP(warp == 0, 1);
  // loop state kept as counters: no integer division on the critical path
  uint32_t st = 0, fph = 0, slot = 0;
  auto advance_stage = [&](uint32_t n) {
    st += n;
    while (st >= (uint32_t)nstage) st -= nstage, fph ^= 1;
  };
  advance_stage(group * L.ktiles);
  slot = group % nslot;
  uint32_t tstamp = 0;
  for (uint32_t c = group; c < my_chunks && !dead; c += G) {
    for (uint32_t kt = 0; kt < L.ktiles; kt++) {
      const uint32_t nbt = qk_tile_nb(L, kt) * L.bs / 256u;  // 256-column spans in this tile
      const uint32_t tile = sbase + S.stage + st * stage_bytes;
      if (!mbar_wait_bounded(sbase + S.full + st * 8, fph)) {
        dead = true;
        break;
      }
      QK_STAMP(warp == 0 && tstamp < 30, 2 + 2 * tstamp);
      // software pipeline over this warp's columns (fully unrolled, two register
      // buffers): the next column's loads are in flight while the current one is
      // decoded, multiplied and scaled.  A full tile (all but the last k-tile of a K that
      // is not a multiple of the tile width) runs without the per-column bound checks.
      // every shared-memory load of a column is a compile-time offset from these per-tile bases
      const typename F::Base B = F::base(LN, tile, kt);
      auto load_sb = [&](Data &D, auto jt) { F::template load<M, decltype(jt)::value, WG>(D, B, LN); };
      auto compute_sb = [&](const Data &D) { F::template compute<M>(D, LN, acc); };
      auto tile_body = [&](auto full_tag) {
        constexpr bool FULL = decltype(full_tag)::value;
        constexpr int NSB = NBT / WG;  // columns of a full tile per warp
        Data d0, d1;
        if (FULL || wl < nbt) load_sb(d0, std::integral_constant<int, 0>{});
        static_for<0, (NSB + 1) / 2>([&](auto pt) {
          constexpr int J = 2 * decltype(pt)::value;
          const uint32_t sb0 = wl + J * WG, sb1 = sb0 + WG, sb2 = sb1 + WG;
          if constexpr (J + 1 < NSB)
            if (FULL || sb1 < nbt) load_sb(d1, std::integral_constant<int, J + 1>{});
          if (FULL || sb0 < nbt) compute_sb(d0);
          if constexpr (J + 2 < NSB)
            if (FULL || sb2 < nbt) load_sb(d0, std::integral_constant<int, J + 2>{});
          if constexpr (J + 1 < NSB)
            if (FULL || sb1 < nbt) compute_sb(d1);
        });
      };
      if (nbt == NBT)
        tile_body(std::true_type{});
      else
        tile_body(std::false_type{});
      QK_STAMP(warp == 0 && tstamp < 30, 3 + 2 * tstamp);
      tstamp++;
      advance_stage(1);
    }
    if (dead) break;
    // chunk finished: leave the row partials for the reducer
    float *red = reinterpret_cast<float *>(smem + S.red) + slot * (WG * M * 8);
#pragma unroll
    for (int m = 0; m < M; m++) {
      float v = F::finish(acc[m], LN);
      v += __shfl_xor_sync(0xffffffffu, v, 1);
      v += __shfl_xor_sync(0xffffffffu, v, 2);
      if (tig == 0) red[(wl * M + m) * 8 + g] = v;
      acc[m][0] = acc[m][1] = acc[m][2] = 0.f;
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(sbase + S.redfull + slot * 8);
    slot += G;
    while (slot >= (uint32_t)nslot) slot -= nslot;
    advance_stage((G - 1) * L.ktiles);
  }
  if (dead) atomicOr(status, QK_DEV_TIMEOUT);  // a bounded wait ran out: results are invalid
  QK_STAMP(warp == 0, 100);
}

struct PlanMma {
  SmemMma S;
  uint32_t Kp, stage_bytes, total;
  int nstage, nslot, groups, cw;
};

// Compute warps per CTA (+ one producer / reducer warp).  With 16 the register budget is 96
// per thread and the column pipeline spills; 8 warps (up to 255 registers) stream as fast or
// faster at every M (14336 x 4096, M = 1: 8.2 us against 8.8 us).  12 warps in three groups
// (128 registers) start and finish sooner when a CTA has few chunks: 3.3 against 3.8 us at
// 1024 rows, 4.6 against 4.7 us at 4096, level from 14336 rows on.  Q6_K, whose fragment
// assembly costs the most arithmetic per byte, is bound by its compute warps with 8 of them:
// 12 take the 128256 x 4096 matvec from 86.4 to 74.1 us (0.76 -> 0.89 of the copy bandwidth),
// so it takes 12 at every row count (IQ4_XS gains 1 %, Q4_K loses 2 % at 14336 rows and both
// keep 8).  QK_CW overrides (developer knob: 8, 12 or 16).
inline int compute_warps(const QkLayout &L, uint32_t m) {
  static int cw_env = -1;
  if (cw_env < 0) {
    const char *e = qk_knob("QK_CW");
    const int v = e ? atoi(e) : 0;
    cw_env = (v == 8 || v == 12 || v == 16) ? v : 0;
  }
  if (m >= 2) return cw_env == 16 ? 16 : 8;  // the 12-warp kernel is built for M = 1 only
  if (cw_env) return cw_env;
  return (L.ktiles == 1 && (L.chunks <= 1024 || L.type == QK_T_Q6_K)) ? 12 : 8;
}

// force_cw8: always the 8-warp kernel (the route that takes its split activations from a
// caller-provided image is built for 8 warps only).
// xsb: bytes per 32-column block in the activation scale table (F::XSB).
inline bool make_plan_mma(const QkLayout &L, uint32_t m, PlanMma *P, uint32_t xsb, bool force_cw8 = false) {
  if (L.nb == 0 || L.chunks == 0) return false;  // nothing to stream: the callers handle empty shapes
  uint32_t Kp = L.nb * L.bs;
  if (Kp % 256u) return false;  // the kernels walk K in spans of 256 columns
  uint32_t nbt_max = L.nb < L.nbt ? L.nb : L.nbt;
  uint32_t stage_bytes = QK_TILE_ROWS * nbt_max * L.bb;
  stage_bytes = (stage_bytes + 127u) & ~127u;
  SmemMma S;
  uint32_t off = 0;
  S.full = off, off += MAX_STAGE * 8;
  S.redfull = off, off += MAX_SLOT * 8;
  S.xbar = off, off += 8;
  S.prog = off, off += 8;
  off = (off + 127u) & ~127u;
  S.red = off, off += MAX_SLOT * MAX_CW * m * 8 * 4;
  off = (off + 127u) & ~127u;
  S.PS = Kp + 64;
  S.xs_off = m * 3 * S.PS;
  S.ximg_bytes = S.xs_off + m * (Kp / 32) * xsb;  // multiple of 16: PS and Kp/32*8 both are
  S.ximg = off, off += S.ximg_bytes;
  off = (off + 127u) & ~127u;
  S.stage = off;
  const uint32_t budget = 227u * 1024u - 1024u;
  if (off + 2 * stage_bytes > budget) return false;
  int nstage = (int)((budget - off) / stage_bytes);
  if (nstage > MAX_STAGE) nstage = MAX_STAGE;
  if (const char *e = qk_knob("QK_NSTAGE")) {  // developer knob: shallower ring
    int v = atoi(e);
    if (v >= 2 && v < nstage) nstage = v;
  }
  // a chunk's stages are refilled only once the whole chunk is reduced: its k-tiles
  // must all fit in the ring with room to prefetch the next chunk
  if ((uint32_t)nstage < L.ktiles + 1) return false;
  // largest group count whose G * ktiles divides a ring depth we can afford
  int groups = 1;
  const char *ge = qk_knob("QK_GROUPS");
  const int gmax = ge ? atoi(ge) : 4;
  int cw = force_cw8 ? 8 : compute_warps(L, m);
  if (cw == 12) {  // three groups of four warps, if the ring can hold three chunks
    const int unit = 3 * (int)L.ktiles;
    if (nstage / unit >= 1 && (nstage / unit) * unit >= (int)L.ktiles + 1)
      groups = 3, nstage = (nstage / unit) * unit;
    else
      cw = 8;
  }
  for (int gtry = 4; gtry >= 2 && cw != 12; gtry >>= 1) {
    const int unit = gtry * (int)L.ktiles;
    if (gtry <= gmax && nstage / unit >= 1 && (nstage / unit) * unit >= (int)L.ktiles + 1) {
      groups = gtry;
      nstage = (nstage / unit) * unit;
      break;
    }
  }
  P->S = S, P->Kp = Kp, P->stage_bytes = stage_bytes, P->nstage = nstage, P->nslot = nstage + 1, P->groups = groups, P->cw = cw;
  P->total = off + nstage * stage_bytes;
  return true;
}

template <class F, int M, bool INCTA, int CW, int G, int MODE = 0>
cudaError_t launch_mma(const QkLayout &L, const uint8_t *W, const float *x, float *y, uint64_t ldy,
                       unsigned *status, unsigned char *ximg, int sm_count, const PlanMma &P,
                       cudaStream_t s, const QkPeers *peers = nullptr, const uint8_t *W2 = nullptr) {
  auto kern = qk_gemv_imma_kernel<F, M, INCTA, CW, G, MODE>;
  static QkPerDevice attr_set;
  if (attr_set.first()) {
    cudaError_t e =
        cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
    if (e != cudaSuccess) return attr_set.reset(), e;
  }
  static int use_pdl = -1;
  if (use_pdl < 0) {
    const char *e = qk_knob("QK_PDL");
    use_pdl = (e && e[0] == '0') ? 0 : 1;
  }
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[0].val.programmaticStreamSerializationAllowed = 1;

  if (!INCTA) {
    const uint32_t quads = (uint32_t)M * P.Kp / 4;
    cudaLaunchConfig_t c0 = {};
    c0.gridDim = dim3((quads + 255) / 256), c0.blockDim = dim3(256), c0.stream = s;
    c0.attrs = at, c0.numAttrs = use_pdl ? 1 : 0;
    cudaError_t e = cudaLaunchKernelEx(&c0, qk_xsplit_kernel<F>, x, (uint32_t)M, L.cols, P.Kp,
                                       P.S.PS, P.S.xs_off, ximg, peers ? peers->wait_slots : nullptr,
                                       peers ? peers->wait_epoch : nullptr, peers ? peers->wait_ld : (uint64_t)0, status);
    if (e != cudaSuccess) return e;
  }
  static int ctas = -1;  // developer knob: persistent CTAs per SM (they must fit: see QK_CW, QK_NSTAGE)
  if (ctas < 0) {
    const char *e = qk_knob("QK_CTAS");
    ctas = (e && atoi(e) == 2) ? 2 : 1;
  }
  uint32_t grid = (uint32_t)sm_count * (uint32_t)ctas;  // persistent
  if (grid > L.chunks) grid = L.chunks;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid), cfg.blockDim = dim3((CW + 1 + (F::SPLIT_PRODUCER ? 1 : 0) + ((MODE == 1 && peers && peers->unpack_n) ? 1 : 0)) * 32);
  cfg.dynamicSmemBytes = P.total, cfg.stream = s;
  cfg.attrs = at, cfg.numAttrs = use_pdl ? 1 : 0;
  QkPeers pv = {};
  if (peers) pv = *peers;
  // Weight tiles issued before the wait on the previous kernel; the rest of the ring follows
  // the activation loads.  Measured at 14336 x 4096, M = 1, 8 warps: with the producer a warp
  // of its own 1 tile 8.04 us, 2 7.81, 3 7.97; with the reducer issuing 1 tile 8.2 us, 2 8.3,
  // 3 8.6; M = 2: 2 tiles 13.1 us, 3 12.9, 4 12.7.  The 12-warp plans with one tile instead of
  // two: within 1 % over the layer's shapes (Q4_0 4096^2 4.7 -> 4.5 us, Q8_0 4096^2 5.2 -> 5.3).
  // QK_PRE overrides (developer knob).
  static int npre_env = -1;
  if (npre_env < 0) {
    const char *e = qk_knob("QK_PRE");
    npre_env = e ? atoi(e) : 0;
  }
  int npre = npre_env > 0 ? npre_env : (M == 1 ? ((F::SPLIT_PRODUCER || CW == 12) ? 2 : 1) : (M == 2 ? 4 : 3));
  if (npre > P.nstage) npre = P.nstage;
  return cudaLaunchKernelEx(&cfg, kern, L, W, W2, x, (const unsigned char *)ximg, y, ldy, status,
                            P.nstage, P.nslot, P.stage_bytes, P.S, P.Kp, pv, npre);
}

// Every CTA redoing the split costs ~M*K/512 quads per thread; past this size the
// separate split kernel plus one bulk copy of its image is cheaper.
inline bool split_in_cta(const PlanMma &P, uint32_t m) {
  static int force = -2;
  if (force == -2) {
    const char *e = qk_knob("QK_XSPLIT");
    force = e ? atoi(e) : -1;  // 0: always the split kernel, 1: always in-CTA
  }
  if (force >= 0) return force == 1;
  return m * P.Kp <= 8192;
}

template <class F, int M>
cudaError_t launch_mma_m(const QkLayout &L, const uint8_t *W, const float *x, float *y,
                         uint64_t ldy, unsigned *status, unsigned char *ximg, int sm_count,
                         const PlanMma &P, cudaStream_t s, const QkPeers *peers, const uint8_t *W2 = nullptr) {
  // Warp groups: a group owns every G-th chunk.  A stage must always be consumed by
  // the same group (a waiter on an mbarrier may be at most one phase ahead of it),
  // so the ring depth is a multiple of G * ktiles; P.groups was chosen to allow that.
  const int cw = P.cw;
  const bool peer = peers != nullptr;
#define QK_LAUNCH1(CWV, GV, PV)                                                                               \
  return split_in_cta(P, M)                                                                                   \
             ? launch_mma<F, M, true, CWV, GV, PV>(L, W, x, y, ldy, status, ximg, sm_count, P, s, peers, W2)  \
             : launch_mma<F, M, false, CWV, GV, PV>(L, W, x, y, ldy, status, ximg, sm_count, P, s, peers, W2)
#define QK_LAUNCH(CWV, GV)                \
  do {                                    \
    if constexpr (F::HAS_DUAL) {          \
      if (W2) {                           \
        QK_LAUNCH1(CWV, GV, 2);           \
      }                                   \
    }                                     \
    if (peer) {                           \
      QK_LAUNCH1(CWV, GV, 1);             \
    } else {                              \
      QK_LAUNCH1(CWV, GV, 0);             \
    }                                     \
  } while (0)
  if constexpr (M == 1)
    if (cw == 12) QK_LAUNCH(12, 3);
#ifdef QK_DEV_KNOBS  // the 16-warp variants exist for experiments only (QK_CW=16)
  if (cw == 16) {
    switch (P.groups) {
      case 4:
        QK_LAUNCH(16, 4);
      case 2:
        QK_LAUNCH(16, 2);
      default:
        QK_LAUNCH(16, 1);
    }
  }
#endif
  switch (P.groups) {
    case 4:
      QK_LAUNCH(8, 4);
    case 2:
      QK_LAUNCH(8, 2);
    default:
      QK_LAUNCH(8, 1);
  }
#undef QK_LAUNCH1
#undef QK_LAUNCH
}


// The public faces of one format's kernels.
template <class F>
bool supported(const QkLayout &L, uint32_t m) {
  if (m < 1 || m > (uint32_t)F::MAX_M) return false;
  PlanMma P;
  return make_plan_mma(L, m, &P, F::XSB);
}

template <class F>
size_t scratch_bytes(const QkLayout &L, uint32_t m) {
  PlanMma P;
  return make_plan_mma(L, m, &P, F::XSB) ? P.S.ximg_bytes : 0;
}

// tiled2 != nullptr: the two-matrix (feed-forward gate and up) mode, formats with F::HAS_DUAL only.
template <class F>
cudaError_t launch(const QkLayout &L, const uint8_t *tiled, const float *x, float *y, uint32_t m, uint64_t ldy,
                   unsigned *status, unsigned char *scratch, int sm_count, cudaStream_t s, const QkPeers *peers,
                   const uint8_t *tiled2 = nullptr) {
  PlanMma P;
  if (!make_plan_mma(L, m, &P, F::XSB)) return cudaErrorInvalidConfiguration;
  if (m < 1 || m > (uint32_t)F::MAX_M) return cudaErrorInvalidConfiguration;
  if (tiled2 && (!F::HAS_DUAL || peers)) return cudaErrorInvalidConfiguration;
  if (m == 1) return launch_mma_m<F, 1>(L, tiled, x, y, ldy, status, scratch, sm_count, P, s, peers, tiled2);
  if constexpr (F::MAX_M >= 2)
    if (m == 2) return launch_mma_m<F, 2>(L, tiled, x, y, ldy, status, scratch, sm_count, P, s, peers, tiled2);
  if constexpr (F::MAX_M >= 3)
    if (m == 3) return launch_mma_m<F, 3>(L, tiled, x, y, ldy, status, scratch, sm_count, P, s, peers, tiled2);
  if constexpr (F::MAX_M >= 4)
    if (m == 4) return launch_mma_m<F, 4>(L, tiled, x, y, ldy, status, scratch, sm_count, P, s, peers, tiled2);
  return cudaErrorInvalidConfiguration;
}

}  // namespace qkdec

// One translation unit per format instantiates its kernels and exports these three.
#define QK_DEC_DEFINE(NAME, F)                                                                                  \
  bool qk_dec_##NAME##_supported(const QkLayout &L, uint32_t m) { return qkdec::supported<F>(L, m); }           \
  size_t qk_dec_##NAME##_scratch(const QkLayout &L, uint32_t m) { return qkdec::scratch_bytes<F>(L, m); }       \
  cudaError_t qk_dec_##NAME##_launch(const QkLayout &L, const uint8_t *tiled, const float *x, float *y,         \
                                     uint32_t m, uint64_t ldy, unsigned *status, unsigned char *scratch,        \
                                     int sm_count, cudaStream_t s, const QkPeers *peers) {                      \
    return qkdec::launch<F>(L, tiled, x, y, m, ldy, status, scratch, sm_count, s, peers);                       \
  }
#define QK_DEC_DECLARE(NAME)                                                                                    \
  bool qk_dec_##NAME##_supported(const QkLayout &L, uint32_t m);                                                \
  size_t qk_dec_##NAME##_scratch(const QkLayout &L, uint32_t m);                                                \
  cudaError_t qk_dec_##NAME##_launch(const QkLayout &L, const uint8_t *tiled, const float *x, float *y,         \
                                     uint32_t m, uint64_t ldy, unsigned *status, unsigned char *scratch,        \
                                     int sm_count, cudaStream_t s, const QkPeers *peers);
