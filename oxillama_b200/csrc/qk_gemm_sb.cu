// Small-batch dequant-matmul (5 .. 16 activation rows) for Q4_K: still bound by the weight
// stream from HBM, so the kernel is built like the decode kernels (persistent CTAs, a
// producer warp that keeps a deep ring of bulk copies in flight, no CTA-wide barrier in the
// steady state), but the multiply goes to the fp16 tensor-core MMA so that one dequantised
// weight fragment serves every token of the batch:
//
//   mma.sync.m16n8k16  A = 16 tokens x 16 columns of activations (fp16, from shared memory),
//                      B = 16 columns x 8 weight rows, dequantised in registers by the lane
//                          that owns them (one 32-bit word of packed nibbles -> the B
//                          fragments of two MMAs: its low nibbles and its high nibbles),
//                      C = 16 tokens x 8 rows, f32.
//
// The batched tcgen05 kernel (qk_gemm_tc.cu) cannot reach the HBM roofline at these sizes:
// its 128-row tiles leave a quarter of the SMs without work at 14336 rows and every tile
// pays a fixed hand-off chain; here the unit of work is an 8-row chunk, as in the decode path.
// Above 16 tokens the activation fragments (one ldmatrix per MMA, no reuse) saturate shared
// memory and the tcgen05 kernel is the faster one; the dispatcher sends those there.  The
// kernel is bound by the integer and fp16 pipes that unpack the nibbles (about 50 issue
// cycles per 64 columns of 8 rows and warp), not by HBM: 14336 x 4096 at 8 tokens runs in
// 22.5 us against 28.4 us for the tcgen05 kernel and 5.5 us of pure weight streaming.  With
// few chunks per CTA (4096 rows) it loses to the tcgen05 kernel, so qk_gemm_sb_preferred()
// asks for at least eight chunks per SM.
//
// Activations: qk_x16_sb_kernel converts the batch once per call to fp16, each token row
// divided by the power of two that puts its largest magnitude in [512, 1024) (exact; the
// epilogue multiplies back), columns permuted inside every 64-column group into the order in
// which a packed word yields its values.  K is walked in slices of 1024 columns (outer loop)
// and the CTA's chunks in the inner loop: a slice of the activations [16 x 1024] is
// double-buffered in shared memory (bulk copies by a warp of its own, overlapped with the
// previous slice's work), every (slice, chunk) is one ring stage holding that chunk's 1024
// columns of packed weights (4608 bytes; 32 stages in flight, one per lane of the weight
// producer warp).  The sixteen compute
// warps form 16 / GW groups; a group owns up to two chunks of a pass and keeps their f32 sums
// in registers across all slices; the GW warps of a group split a stage's columns and meet
// once, at the end of the pass.  GW is chosen on the host so that one pass covers the CTA's
// chunks where it can (every further pass streams the activations again).
//
// Weights are rounded to fp16 once (q exact, then one fused q * scale - min), activations to
// fp16: results sit at ~3e-4 of the output's largest magnitude against the f32 reference
// (reference/q4_k.rs:104-201; the path's stated tolerance is 1e-3).  Every mbarrier wait is
// bounded (QK_DEV_TIMEOUT).
#include <cfloat>

#include <cuda_fp16.h>

#include "qk_kernels.h"
#include "qk_pipe.cuh"

using namespace qkpipe;

namespace {

constexpr int CW = 16;              // compute warps (+ two producer warps: weights, activations)
constexpr int CPG = 2;              // chunks a group of warps holds sums for
constexpr int MPAD = 16;            // token rows of an activation slice (one MMA tile)
constexpr uint32_t KS = 1024;       // columns per slice
constexpr int MAX_STAGES = 32;      // one ring slot per lane of the weight producer warp
constexpr uint32_t COLB = 1152;     // bytes of one 256-column span of 8 rows (block-major tile)

struct SbPlan {
  uint32_t full, empty, xfull, xfree;  // mbarrier arrays
  uint32_t acc, xbuf, ring;            // byte offsets
  uint32_t xstride;                    // bytes between token rows of an activation slice
  uint32_t xbuf_bytes, stage_bytes, total;
  uint32_t gw_log2;                    // log2 of the warps that share a stage
  int nst;
};

// Non-blocking poll.  mbarrier.try_wait may hold the thread for a system-dependent time
// before it answers "not yet"; the producer warp watches two barriers at once (a weight
// stage to refill, an activation buffer to reload) and must not sit in either poll:
// with try_wait in that loop it issued one stage every few microseconds (measured: 372 us
// for a 33 MB matrix at 64 tokens).
__device__ __forceinline__ bool mbar_test(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mma_f16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&a)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(a[0]), "=r"(a[1]), "=r"(a[2]), "=r"(a[3])
               : "r"(addr));
}
__device__ __forceinline__ __half2 bits_h2(uint32_t v) { return *reinterpret_cast<__half2 *>(&v); }
__device__ __forceinline__ uint32_t h2_bits(__half2 v) { return *reinterpret_cast<uint32_t *>(&v); }

__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
  uint32_t r;
  asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(sel));
  return r;
}
__device__ __forceinline__ uint2 lds64(uint32_t addr) {
  uint2 v;
  asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(addr));
  return v;
}

// Column (inside its 64-column group) whose activation sits at position p of the group's fp16
// run.  A lane (g = its weight row, t = lane % 4) holds bytes 8 t .. 8 t + 7 of the row's 32
// packed bytes of the group: word 0 = bytes 8 t .. + 3, word 1 = bytes 8 t + 4 .. + 7.  The
// group is four MMA steps (word 0 low nibbles, word 0 high nibbles, word 1 low, word 1 high);
// inside a step k-slot s meets byte 2 r + u of the word of lane t = (s % 8) / 2, with
// r = s % 2 and u = s / 8 (b0 = bytes 0 and 2 of the word, b1 = bytes 1 and 3).
__host__ __device__ inline uint32_t sb_src_col(uint32_t p) {
  const uint32_t step = p >> 4, s = p & 15u;
  const uint32_t byte = 8u * ((s & 7u) >> 1) + 4u * (step >> 1) + 2u * (s & 1u) + (s >> 3);
  return byte + 32u * (step & 1u);
}


// ---------------------------------------------------------------- activations -> fp16
// X16[t][64 G + p] = x[t][64 G + sb_src_col(p)] / scale[t]; rows t >= m and columns >= cols are zero.
__global__ void __launch_bounds__(256)
    qk_x16_sb_kernel(const float *__restrict__ x, uint32_t m, uint32_t cols, uint32_t m_pad, uint32_t Kp,
                     __half *__restrict__ out, float *__restrict__ scales) {
  __shared__ float red[8];
  pdl_launch_dependents();
  pdl_wait();
  for (uint32_t t = blockIdx.x; t < m_pad; t += gridDim.x) {
    const float *xr = x + (uint64_t)t * cols;
    float amax = 0.f;
    __syncthreads();
    if (t < m)
      for (uint32_t k = threadIdx.x; k < cols; k += 256) amax = fmaxf(amax, fabsf(__ldg(xr + k)));
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
      frexpf(amax, &e);
      scale = ldexpf(1.f, e - 10);
    }
    const float inv = 1.f / scale;
    if (threadIdx.x == 0) scales[t] = scale;
    for (uint32_t p = threadIdx.x; p < Kp; p += 256) {
      const uint32_t k = (p & ~63u) + sb_src_col(p & 63u);
      float v = 0.f;
      if (t < m && k < cols) v = __ldg(xr + k) * inv;
      out[(uint64_t)t * Kp + p] = __float2half_rn(v);
    }
  }
}


// ---------------------------------------------------------------- main kernel
__global__ void __launch_bounds__((CW + 2) * 32, 1)
    qk_gemm_sb_q4k_kernel(QkLayout L, const uint8_t *__restrict__ W, const __half *__restrict__ x16,
                          const float *__restrict__ xscale, float *__restrict__ y, uint64_t ldy, uint32_t m_tokens,
                          uint32_t Kp, unsigned *status, SbPlan P) {
  extern __shared__ __align__(128) unsigned char smem[];
  const uint32_t sbase = smem_u32(smem);
  const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t nst = (uint32_t)P.nst;
  const uint32_t n_slices = (Kp + KS - 1) / KS;
  const uint32_t GW = 1u << P.gw_log2, NG = (uint32_t)CW >> P.gw_log2, pass_chunks = NG * CPG;
  // A CTA's chunks are neighbours in memory (a few hundred KB): its bulk copies then stay inside
  // one or two pages, where chunks dealt round-robin over the CTAs put every copy on a page
  // of its own and each paid a translation miss (measured: 250 ns per copy, the whole kernel
  // bound by the producer's issue rate).
  const uint32_t cbase = L.chunks / gridDim.x, crem = L.chunks % gridDim.x;
  const uint32_t my_chunks = cbase + (blockIdx.x < crem ? 1u : 0u);
  const uint32_t chunk0 = blockIdx.x * cbase + min(blockIdx.x, crem);
  const uint32_t n_pass = (my_chunks + pass_chunks - 1) / pass_chunks;

  pdl_launch_dependents();
  if (threadIdx.x == 0) {
    for (uint32_t s = 0; s < nst; s++) {
      mbar_init(sbase + P.full + s * 8, 1);
      mbar_init(sbase + P.empty + s * 8, GW);  // the warps of the group that owns the stage
    }
    for (int b = 0; b < 2; b++) {
      mbar_init(sbase + P.xfull + b * 8, 1);
      mbar_init(sbase + P.xfree + b * 8, CW);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  __syncthreads();

  if (warp == CW) {
    // ================= weight producer warp =================
    // Lane l owns ring slot l and issues the stages l, l + nst, l + 2 nst, .. of the CTA's
    // stage sequence (pass, slice, chunk: the order the compute warps take them).  One thread
    // walking that sequence alone spends about 400 cycles of dependent arithmetic per stage,
    // which capped the whole kernel at the producer's issue rate; 32 lanes do it side by side.
    // The weights do not depend on the kernel before this one, so nothing here waits for it.
    const uint32_t total_stages = my_chunks * n_slices;
    const uint32_t full_pass_stages = n_slices * pass_chunks;                 // stages of a pass that holds pass_chunks chunks
    const uint32_t last_base = (n_pass ? n_pass - 1u : 0u) * full_pass_stages;  // first stage of the last pass
    const uint32_t nc_last = my_chunks - (n_pass ? n_pass - 1u : 0u) * pass_chunks;
    const uint64_t policy = stream_policy();
    uint32_t my_it = lane, round = 0, polls = 0;
    unsigned long long t0 = 0;
    bool dead = false;
    if (lane >= nst) my_it = total_stages;  // nst <= 32
    while (__any_sync(0xffffffffu, my_it < total_stages) && !dead) {
      bool can = my_it < total_stages;
      if (can && round) can = mbar_test(sbase + P.empty + lane * 8, (round - 1u) & 1u);
      if (can) {
        uint32_t pass, r, nc;
        if (my_it < last_base) pass = my_it / full_pass_stages, r = my_it - pass * full_pass_stages, nc = pass_chunks;
        else pass = n_pass - 1u, r = my_it - last_base, nc = nc_last;
        const uint32_t sl = r / nc, j = r - sl * nc;
        const uint32_t ncol = min(KS, Kp - sl * KS);
        const uint32_t kt = (sl * KS) / QK_TILE_ELEMS, span = ((sl * KS) % QK_TILE_ELEMS) / 256u;
        const uint32_t bytes = (ncol / 256u) * COLB;
        const uint32_t chunk = chunk0 + pass * pass_chunks + j;
        const uint32_t bar = sbase + P.full + lane * 8;
        mbar_expect_tx(bar, bytes);
        bulk_g2s_stream(sbase + P.ring + lane * P.stage_bytes, W + qk_tile_offset(L, chunk, kt) + span * COLB, bytes, bar, policy);
        my_it += nst, round++;
      }
      if (__any_sync(0xffffffffu, can)) {
        polls = 0, t0 = 0;
      } else if ((++polls & 1023u) == 0) {  // nothing moved for a while: check the clock
        unsigned long long t;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
        if (!t0) t0 = t;
        if (t - t0 > 250000000ull) dead = true;
      }
    }
    if (dead && lane == 0) atomicOr(status, QK_DEV_TIMEOUT);
    return;
  }
  if (warp == CW + 1) {
    // ================= activation producer warp =================
    // Slice s of the fp16 activations (the previous kernel's output) goes into buffer s % 2
    // once every compute warp has released slice s - 2.
    pdl_wait();
    const uint32_t total_slices = n_pass * n_slices;
    for (uint32_t xs = 0; xs < total_slices; xs++) {
      const uint32_t b = xs & 1u, sl = xs % n_slices;
      if (xs >= 2 && !mbar_wait_bounded(sbase + P.xfree + b * 8, ((xs >> 1) - 1u) & 1u)) {
        if (lane == 0) atomicOr(status, QK_DEV_TIMEOUT);
        return;
      }
      const uint32_t ncol = min(KS, Kp - sl * KS);  // columns of this slice
      const uint32_t bytes = ncol * 2u;
      const uint32_t bar = sbase + P.xfull + b * 8;
      if (lane == 0) mbar_expect_tx(bar, bytes * MPAD);
      __syncwarp();
      if (lane < (uint32_t)MPAD)
        bulk_g2s(sbase + P.xbuf + b * P.xbuf_bytes + lane * P.xstride, x16 + (uint64_t)lane * Kp + (uint64_t)sl * KS, bytes, bar);
    }
    return;
  }

  // ================= compute warps =================
  // 16 / GW groups of GW warps.  Group q takes the stages of chunks j = q and q + 16 / GW of a
  // pass; its warps split a stage's 64-column groups between them and keep their f32 sums in
  // registers across all slices, so nothing is added into shared memory until the pass ends
  // (shared-memory float atomics are compare-and-swap loops, and warps adding into the same
  // sums serialise on them: measured 4 us per stage).  A warp that gives up on a wait (dead)
  // skips the rest of its work but still meets the others at the pass-end barriers.
  const uint32_t g = lane >> 2, tig = lane & 3;
  const uint32_t grp_id = warp >> P.gw_log2, wig = warp & (GW - 1u);
  const uint32_t gpw = (KS / 64u) >> P.gw_log2;  // 64-column groups of a stage per warp: 16, 8, 4 or 2
  float4 *part = reinterpret_cast<float4 *>(smem + P.acc);  // [CW][CPG][32]: the sums of warps 1 .. GW - 1 at pass end
  // ldmatrix row address of this lane inside an activation slice: matrices 0..3 = (tokens 0-7,
  // k 0-7), (tokens 8-15, k 0-7), (tokens 0-7, k 8-15), (tokens 8-15, k 8-15)
  const uint32_t lm_row = (lane & 7u) + ((lane >> 3) & 1u) * 8u, lm_koff = (lane >> 4) * 16u;
  const uint32_t xlane = lm_row * P.xstride + lm_koff;
  const __half2 k_lo = __float2half2_rn(1024.f), k_hi = __float2half2_rn(64.f);
  bool dead = false;
  uint32_t it_base = 0, sc = 0;  // first stage of the current slice and slice counter, in the producer's order

  for (uint32_t pass = 0; pass < n_pass; pass++) {
    const uint32_t c0 = pass * pass_chunks, nc = min(pass_chunks, my_chunks - c0);
    float c[CPG][4][4];  // four interleaved accumulation chains per chunk (one per MMA step of a group)
#pragma unroll
    for (int jj = 0; jj < CPG; jj++)
#pragma unroll
      for (int k = 0; k < 4; k++) c[jj][k][0] = c[jj][k][1] = c[jj][k][2] = c[jj][k][3] = 0.f;
    for (uint32_t sl = 0; sl < n_slices && !dead; sl++, sc++, it_base += nc) {
      const uint32_t ncol = min(KS, Kp - sl * KS), ngrp = ncol / 64u;  // 64-column groups in this slice
      const uint32_t b = sc & 1u;
      if (!mbar_wait_bounded(sbase + P.xfull + b * 8, (sc >> 1) & 1u)) {
        dead = true;
        break;
      }
      const uint32_t xb = sbase + P.xbuf + b * P.xbuf_bytes + xlane;
      const uint32_t g0 = min(wig * gpw, ngrp), g1 = min(g0 + gpw, ngrp);  // this warp's groups of every stage
#pragma unroll
      for (int jj = 0; jj < CPG; jj++) {
        const uint32_t j = (uint32_t)jj * NG + grp_id;
        if (j >= nc || dead) continue;  // warp-uniform
        const uint32_t it = it_base + j, st = it % nst;
        if (!mbar_wait_bounded(sbase + P.full + st * 8, (it / nst) & 1u)) {
          dead = true;
          continue;
        }
        const uint32_t tile = sbase + P.ring + st * P.stage_bytes;
        // Two groups (a "pair": 128 columns, half a span) at a time: they share the span's
        // header and one word of its packed 6-bit scales.  Every shared-memory load of the pair
        // is issued before the first use (the loads are volatile asm, which the compiler keeps
        // in source order: written load -> use -> load -> use, each step waited out the previous
        // one's latency).  The kernel is bound by the integer pipe, so the pair is written for
        // few instructions: scales and mins converted two at a time in half2 arithmetic
        // (1024 + byte is an fp16 bit pattern), the moves of one half to both halves left to the
        // operand selectors of the multiply-adds.  (Written out in the loop on purpose: the
        // same body as a lambda, or a span-level loop with both pairs unrolled, measured 5 %
        // slower.)
        for (uint32_t gi = g0; gi < g1; gi += 2) {
          const uint32_t span = gi >> 2, hi_pair = (gi >> 1) & 1u;
          const uint32_t sp = tile + span * COLB;
          // row g's header: d, dmin and the 6-bit scales / mins of the span's eight sub-blocks
          // (reference/q4_k.rs:27-49); this pair uses sub-blocks 4 hi_pair .. 4 hi_pair + 3
          const uint4 h = lds128(sp + g * 16);
          // the lane's 8 bytes of each group (row g, bytes 8 tig .. + 7)
          const uint32_t qa = sp + 128u + hi_pair * 512u + g * 32u + tig * 8u;
          uint2 wq[2];
          wq[0] = lds64(qa), wq[1] = lds64(qa + 256u);
          const uint32_t xg = xb + gi * 128u;  // the pair's activations: 2 groups x 4 steps x 32 bytes
          uint32_t a[8][4];
#pragma unroll
          for (int q = 0; q < 8; q++) ldmatrix_x4(a[q], xg + (uint32_t)q * 32u);
          const __half2 d2 = __low2half2(bits_h2(h.x));
          const __half2 nm2 = __hneg2(__high2half2(bits_h2(h.x)));  // -dmin
          const uint32_t scw = hi_pair ? ((h.w & 0x0F0F0F0Fu) | ((h.y >> 2) & 0x30303030u)) : (h.y & 0x3F3F3F3Fu);
          const uint32_t mnw = hi_pair ? (((h.w >> 4) & 0x0F0F0F0Fu) | ((h.z >> 2) & 0x30303030u)) : (h.z & 0x3F3F3F3Fu);
#pragma unroll
          for (int u = 0; u < 2; u++) {
            // bytes 2 u and 2 u + 1 of the words -> fp16 (1024 + byte, exact), -1024, times d:
            // the scales of the group's low-nibble and high-nibble sub-block in one half2
            const uint32_t sel = u ? 0x4342u : 0x4140u;
            const __half2 s2 = __hmul2(__hsub2(bits_h2(prmt(scw, 0x64646464u, sel)), k_lo), d2);
            const __half2 m2 = __hmul2(__hsub2(bits_h2(prmt(mnw, 0x64646464u, sel)), k_lo), nm2);
            const __half2 s_lo = __low2half2(s2), s_hi = __high2half2(s2);
            const __half2 m_lo = __low2half2(m2), m_hi = __high2half2(m2);
#pragma unroll
            for (int hf = 0; hf < 2; hf++) {
              const uint32_t w = hf ? wq[u].y : wq[u].x, wj = w >> 8;
              // nibble -> fp16 by dropping it into the mantissa of 1024 (low) or 64 (high); q
              // exact after the subtraction, then one fused q * scale - min
              const uint32_t e0 = (w & 0x000F000Fu) | 0x64006400u, e1 = (wj & 0x000F000Fu) | 0x64006400u;
              const uint32_t e2 = (w & 0x00F000F0u) | 0x54005400u, e3 = (wj & 0x00F000F0u) | 0x54005400u;
              const uint32_t bl0 = h2_bits(__hfma2(__hsub2(bits_h2(e0), k_lo), s_lo, m_lo));
              const uint32_t bl1 = h2_bits(__hfma2(__hsub2(bits_h2(e1), k_lo), s_lo, m_lo));
              const uint32_t bh0 = h2_bits(__hfma2(__hsub2(bits_h2(e2), k_hi), s_hi, m_hi));
              const uint32_t bh1 = h2_bits(__hfma2(__hsub2(bits_h2(e3), k_hi), s_hi, m_hi));
              mma_f16(c[jj][2 * hf], a[4 * u + 2 * hf], bl0, bl1);          // step (hf, low)
              mma_f16(c[jj][2 * hf + 1], a[4 * u + 2 * hf + 1], bh0, bh1);  // step (hf, high)
            }
          }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(sbase + P.empty + st * 8);
      }
      if (dead) break;
      __syncwarp();
      if (lane == 0) mbar_arrive(sbase + P.xfree + b * 8);  // this warp is done with the slice's activations
    }
    // End of the pass: warps 1 .. GW - 1 of a group leave their sums in shared memory, the
    // first adds them to its own, scales each token back and writes y (a chunk's eight rows
    // are 32 contiguous bytes of a token's output row).
    if (GW > 1) {
      if (wig != 0) {
#pragma unroll
        for (int jj = 0; jj < CPG; jj++)
          part[(warp * CPG + jj) * 32 + lane] =
              make_float4((c[jj][0][0] + c[jj][1][0]) + (c[jj][2][0] + c[jj][3][0]), (c[jj][0][1] + c[jj][1][1]) + (c[jj][2][1] + c[jj][3][1]),
                          (c[jj][0][2] + c[jj][1][2]) + (c[jj][2][2] + c[jj][3][2]), (c[jj][0][3] + c[jj][1][3]) + (c[jj][2][3] + c[jj][3][3]));
      }
      asm volatile("bar.sync 1, %0;" ::"n"(CW * 32) : "memory");
    }
    if (pass == 0) pdl_wait();  // y may still be read by the kernel before this one
    if (wig == 0 && !dead) {
#pragma unroll
      for (int jj = 0; jj < CPG; jj++) {
        const uint32_t j = (uint32_t)jj * NG + grp_id;
        if (j >= nc) continue;
        float v[4];
#pragma unroll
        for (int q = 0; q < 4; q++) v[q] = (c[jj][0][q] + c[jj][1][q]) + (c[jj][2][q] + c[jj][3][q]);
        for (uint32_t w2 = 1; w2 < GW; w2++) {
          const float4 p = part[((warp + w2) * CPG + jj) * 32 + lane];
          v[0] += p.x, v[1] += p.y, v[2] += p.z, v[3] += p.w;
        }
        const uint32_t row = (chunk0 + c0 + j) * 8 + 2 * tig;
        const uint32_t t0 = g, t1 = g + 8;
        if (t0 < m_tokens) {
          const float sc0 = __ldg(xscale + t0);
          if (row < L.rows) y[(uint64_t)t0 * ldy + row] = v[0] * sc0;
          if (row + 1 < L.rows) y[(uint64_t)t0 * ldy + row + 1] = v[1] * sc0;
        }
        if (t1 < m_tokens) {
          const float sc1 = __ldg(xscale + t1);
          if (row < L.rows) y[(uint64_t)t1 * ldy + row] = v[2] * sc1;
          if (row + 1 < L.rows) y[(uint64_t)t1 * ldy + row + 1] = v[3] * sc1;
        }
      }
    }
    if (GW > 1 && pass + 1 < n_pass)
      asm volatile("bar.sync 1, %0;" ::"n"(CW * 32) : "memory");  // before the next pass reuses the exchange buffer
  }
  if (dead && lane == 0) atomicOr(status, QK_DEV_TIMEOUT);
}

bool make_sb_plan(const QkLayout &L, uint32_t m, int sm_count, SbPlan *P) {
  if (L.type != QK_T_Q4_K || L.nb == 0 || L.chunks == 0 || m < 1 || m > (uint32_t)MPAD || sm_count < 1) return false;
  SbPlan p;
  uint32_t off = 0;
  p.full = off, off += MAX_STAGES * 8;
  p.empty = off, off += MAX_STAGES * 8;
  p.xfull = off, off += 16;
  p.xfree = off, off += 16;
  off = (off + 127u) & ~127u;
  p.acc = off, off += CW * CPG * 32 * 16;
  p.xstride = KS * 2u + 16u;  // 16 bytes of padding: eight consecutive rows fall into eight different 16-byte bank groups
  p.xbuf_bytes = (MPAD * p.xstride + 127u) & ~127u;
  p.xbuf = off, off += 2 * p.xbuf_bytes;
  p.stage_bytes = (KS / 256u) * COLB;  // a multiple of 128
  p.ring = off;
  const uint32_t budget = 227u * 1024u - 1024u;
  int nst = (int)((budget - off) / p.stage_bytes);
  if (nst > MAX_STAGES) nst = MAX_STAGES;  // one ring slot per lane of the weight producer
  p.nst = nst;
  p.total = off + (uint32_t)nst * p.stage_bytes;
  // warps per stage: as few as still let one pass (16 / GW groups x CPG chunks) cover a CTA's chunks
  const uint32_t grid = (uint32_t)sm_count < L.chunks ? (uint32_t)sm_count : L.chunks;
  const uint32_t cpc = (L.chunks + grid - 1) / grid;
  p.gw_log2 = cpc <= 4 ? 3u : cpc <= 8 ? 2u : cpc <= 16 ? 1u : 0u;
  *P = p;
  return true;
}

}  // namespace


bool qk_gemm_sb_supported(const QkLayout &L, uint32_t m) {
  SbPlan P;
  return make_sb_plan(L, m, 1, &P);
}

bool qk_gemm_sb_preferred(const QkLayout &L, uint32_t m, int sm_count) {
  return m > QK_GEMV_MAX_M && m <= (uint32_t)MPAD && sm_count > 0 && L.chunks >= 8u * (uint32_t)sm_count &&
         qk_gemm_sb_supported(L, m);
}

size_t qk_gemm_sb_scratch_bytes(const QkLayout &L, uint32_t m) {
  (void)m;
  const size_t Kp = (size_t)L.nb * 256u;
  return (((size_t)MPAD * Kp * 2 + 255) & ~(size_t)255) + MPAD * 4;
}

cudaError_t qk_launch_gemm_sb(const QkLayout &L, const uint8_t *tiled, const float *x, float *y, uint32_t m,
                              uint64_t ldy, unsigned *status, unsigned char *scratch, int sm_count, cudaStream_t s) {
  SbPlan P;
  if (!make_sb_plan(L, m, sm_count, &P)) return cudaErrorInvalidConfiguration;
  auto kern = qk_gemm_sb_q4k_kernel;
  static QkPerDevice attr_set;
  if (attr_set.first()) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
    if (e != cudaSuccess) return attr_set.reset(), e;
  }
  const uint32_t Kp = L.nb * 256u;
  __half *x16 = reinterpret_cast<__half *>(scratch);
  float *xscale = reinterpret_cast<float *>(scratch + (((size_t)MPAD * Kp * 2 + 255) & ~(size_t)255));
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[0].val.programmaticStreamSerializationAllowed = 1;
  cudaLaunchConfig_t c0 = {};
  c0.gridDim = dim3(MPAD), c0.blockDim = dim3(256), c0.stream = s, c0.attrs = at, c0.numAttrs = 1;
  cudaError_t e = cudaLaunchKernelEx(&c0, qk_x16_sb_kernel, x, m, L.cols, (uint32_t)MPAD, Kp, x16, xscale);
  if (e != cudaSuccess) return e;
  uint32_t grid = (uint32_t)sm_count;
  if (grid > L.chunks) grid = L.chunks;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid), cfg.blockDim = dim3((CW + 2) * 32), cfg.dynamicSmemBytes = P.total, cfg.stream = s;
  cfg.attrs = at, cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kern, L, tiled, (const __half *)x16, (const float *)xscale, y, ldy, m, Kp, status, P);
}
