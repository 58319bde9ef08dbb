// Batched dequant-matmul (prefill and larger decode batches) for Q4_K on the
// 5th-generation tensor cores: tcgen05.mma with the accumulator in tensor memory.
//
//   y[t][n] = sum_k  w(n, k) * x[t][k]          w = d sc q - dmin mn   (reference/q4_k.rs:79-93)
//
// A real dense contraction, so it goes to the tensor cores: the 128 weight rows
// of a tile are the MMA's M dimension, BN activation rows (tokens) its N
// dimension, fp16 operands with f32 accumulation in TMEM (kind::f16).
//
// One CTA per SM, persistent over (128-row block) x (BN-token block) tiles.
//   warp 0      producer: per 256-column step, 16 bulk copies (8 rows x 144 B
//               each, contiguous in the block-major tile layout) bring the packed
//               super-blocks of the 128 rows into a 2-stage ring; per 64-column
//               step one TMA tile load (128-byte swizzle, no multicast) brings
//               the fp16 activations of the BN tokens
//   warp 1      allocates TMEM, then one elected thread issues four
//               tcgen05.mma (K = 16 each) per 64-column stage and commits them to
//               the stage's "empty" mbarrier
//   warps 2-9   two threads per weight row: decode the 6-bit scales, turn 16
//               bytes of nibbles each into 32 fp16 weights (magic-number nibble ->
//               half2, one HFMA2 and one HSUB2 per pair) and store them as one
//               128-byte row of the swizzled K-major A tile; after a tile's last
//               stage the same warps read the accumulator with tcgen05.ld and
//               store y (lanes = consecutive weight rows = consecutive addresses)
//
// The activations are converted to fp16 once per call by qk_x16_kernel, with
// the columns of every 64-group permuted into the order in which a packed word
// yields its nibbles (both operands use the same order, so the sum is
// unchanged).  fp16 operands put the result at ~3e-4 of the output's inf-norm
// against the f32 reference (its stated tolerance is 1e-3).
//
// Every mbarrier wait is time-bounded; a wait that runs out raises
// QK_DEV_TIMEOUT and the CTA falls through to the common exit, which always
// frees its tensor memory.
#include <cuda.h>

#include <cstdlib>

#include "qk_kernels.h"
#include "qk_pipe.cuh"

using namespace qkpipe;

namespace {

constexpr int BM = 128;            // weight rows per tile (UMMA M)
constexpr int BK = 64;             // columns per stage: one 128-byte swizzle row of fp16
constexpr int NDW = 8;              // dequant / epilogue warps: two threads per weight row
constexpr int NTHREADS = 64 + NDW * 32;  // + producer warp + MMA warp
constexpr int MAX_PK_STAGES = 8;   // ring of packed super-block slabs (depth chosen per tile shape)
constexpr uint32_t PK_CHUNK = 1152 + 32;  // one chunk's super-block column, padded against bank aliasing
constexpr uint32_t PK_BYTES = 16 * PK_CHUNK;

struct GemmSmem {
  uint32_t ab_full, ab_empty, pk_full, pk_empty, acc_full, acc_empty, tmem_slot;
  uint32_t pk, a, b;  // ring bases (a, b 1024-byte aligned)
  uint32_t a_stage, b_stage;
  int stages, pk_stages;
};

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

// ---------------------------------------------------------------- activations -> fp16
// X16[t][64 g + 8 i + j] = x[t][64 g + 4 i + {0,2,1,3}[j & 3] + 32 (j >> 2)]; rows t >= m and
// columns >= cols are zero.  One thread per 8 output halves (one 16-byte store).
__global__ void __launch_bounds__(256)
    qk_x16_kernel(const float *__restrict__ x, uint32_t m, uint32_t cols, uint32_t m_pad,
                  uint32_t Kp, __half *__restrict__ out) {
  pdl_launch_dependents();
  pdl_wait();
  const uint32_t per_row = Kp / 8;
  const uint64_t total = (uint64_t)m_pad * per_row;
  for (uint64_t it = blockIdx.x * 256ull + threadIdx.x; it < total; it += (uint64_t)gridDim.x * 256) {
    const uint32_t t = (uint32_t)(it / per_row), c = (uint32_t)(it % per_row);
    const uint32_t g = c >> 3, i = c & 7u;
    __align__(16) __half h[8];
#pragma unroll
    for (int j = 0; j < 8; j++) {
      const uint32_t k = 64 * g + 4 * i + ((j & 3) == 1 ? 2 : (j & 3) == 2 ? 1 : (j & 3)) + 32 * (j >> 2);
      const float v = (t < m && k < cols) ? __ldg(x + (uint64_t)t * cols + k) : 0.f;
      h[j] = __float2half_rn(v);
    }
    *reinterpret_cast<uint4 *>(out + (uint64_t)t * Kp + 8ull * c) = *reinterpret_cast<const uint4 *>(h);
  }
}

// ---------------------------------------------------------------- main kernel
template <int BN>
__global__ void __launch_bounds__(NTHREADS, 1)
    qk_gemm_q4k_tc_kernel(QkLayout L, const uint8_t *__restrict__ W,
                          const __grid_constant__ CUtensorMap xmap, float *__restrict__ y,
                          uint64_t ldy, uint32_t m_tokens, uint32_t tok_blocks, uint32_t row_blocks,
                          unsigned *status, GemmSmem S) {
  extern __shared__ __align__(1024) unsigned char smem[];
  const uint32_t sbase = smem_u32(smem);
  const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int NS = S.stages;
  const uint32_t nsb = L.nb;            // super-blocks along K
  const uint32_t steps = nsb * 4;       // 64-column stages per tile
  const uint32_t n_tiles = tok_blocks * row_blocks;
  constexpr uint32_t IDESC = (1u << 4) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);

  pdl_launch_dependents();
  if (threadIdx.x == 0) {
    for (int s = 0; s < NS; s++) {
      mbar_init(sbase + S.ab_full + s * 8, NDW + 1);  // dequant warps + the producer's expect_tx
      mbar_init(sbase + S.ab_empty + s * 8, 1);  // tcgen05.commit
    }
    for (int s = 0; s < S.pk_stages; s++) {
      mbar_init(sbase + S.pk_full + s * 8, 1);
      mbar_init(sbase + S.pk_empty + s * 8, NDW);
    }
    mbar_init(sbase + S.acc_full, 1);
    mbar_init(sbase + S.acc_empty, NDW);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {  // tensor memory for the BN accumulator columns
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     sbase + S.tmem_slot),
                 "r"((uint32_t)(BN < 32 ? 32 : BN))
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t *>(smem + S.tmem_slot);
  pdl_wait();  // X16 and y belong to the previous kernel until it has finished

  bool dead = false;
  if (warp == 0) {
    // ======================= producer =======================
    if (lane == 0) {
      uint32_t st = 0, eph = 0, first_round = 1;  // A/B stage ring
      uint32_t ps = 0, pph = 0, pk_first = 1;     // packed ring
      for (uint32_t t = blockIdx.x; t < n_tiles && !dead; t += gridDim.x) {
        const uint32_t rb = t / tok_blocks, tb = t % tok_blocks;
        for (uint32_t sbk = 0; sbk < nsb && !dead; sbk++) {
          // ---- packed super-block slab of the tile's 16 row chunks
          if (!pk_first && !mbar_wait_bounded(sbase + S.pk_empty + ps * 8, pph ^ 1)) dead = true;
          if (dead) break;
          {
            const uint32_t kt = sbk / L.nbt, b = sbk % L.nbt;
            uint32_t nvalid = 0;
            for (uint32_t c = 0; c < 16; c++)
              if (rb * 16 + c < L.chunks) nvalid++;
            const uint32_t bar = sbase + S.pk_full + ps * 8;
            mbar_expect_tx(bar, nvalid * 1152);
            for (uint32_t c = 0; c < 16; c++) {
              const uint32_t chunk = rb * 16 + c;
              if (chunk >= L.chunks) break;
              bulk_g2s(sbase + S.pk + ps * PK_BYTES + c * PK_CHUNK,
                       W + qk_tile_offset(L, chunk, kt) + (uint64_t)b * 1152, 1152, bar);
            }
          }
          if (++ps == (uint32_t)S.pk_stages) ps = 0, pph ^= 1, pk_first = 0;
          // ---- four 64-column activation tiles
          for (uint32_t gq = 0; gq < 4; gq++) {
            if (!first_round && !mbar_wait_bounded(sbase + S.ab_empty + st * 8, eph ^ 1)) {
              dead = true;
              break;
            }
            const uint32_t bar = sbase + S.ab_full + st * 8;
            mbar_expect_tx(bar, BN * 128);
            tma_load_2d(sbase + S.b + st * S.b_stage, &xmap, (int)(sbk * 256 + gq * 64),
                        (int)(tb * BN), bar);
            if (++st == (uint32_t)NS) st = 0, eph ^= 1, first_round = 0;
          }
        }
      }
      if (dead) atomicOr(status, QK_DEV_TIMEOUT);
    }
  } else if (warp == 1) {
    // ======================= MMA issuer =======================
    if (lane == 0) {
      uint32_t st = 0, fph = 0, aph = 0, first_tile = 1;
      for (uint32_t t = blockIdx.x; t < n_tiles && !dead; t += gridDim.x) {
        // the epilogue of the previous tile must have drained the accumulator
        if (!first_tile && !mbar_wait_bounded(sbase + S.acc_empty, aph)) dead = true;
        if (!first_tile) aph ^= 1;
        first_tile = 0;
        if (dead) break;
        tc_fence_after();
        for (uint32_t step = 0; step < steps; step++) {
          if (!mbar_wait_bounded(sbase + S.ab_full + st * 8, fph)) {
            dead = true;
            break;
          }
          tc_fence_after();
          const uint32_t a0 = sbase + S.a + st * S.a_stage, b0 = sbase + S.b + st * S.b_stage;
#pragma unroll
          for (int k = 0; k < BK / 16; k++)
            umma_f16(tmem_base, umma_desc(a0 + k * 32), umma_desc(b0 + k * 32), IDESC,
                     (step | (uint32_t)k) ? 1u : 0u);
          umma_commit(sbase + S.ab_empty + st * 8);  // frees the stage when these MMAs retire
          if (++st == (uint32_t)NS) st = 0, fph ^= 1;
        }
        if (dead) break;
        umma_commit(sbase + S.acc_full);  // accumulator complete
      }
      if (dead) atomicOr(status, QK_DEV_TIMEOUT);
    }
  } else {
    // ======================= dequant + epilogue warps =======================
    const uint32_t r = (threadIdx.x - 64) & 127u;  // weight row inside the tile
    const uint32_t half = (threadIdx.x - 64) >> 7; // which 16 of the 32 group bytes this thread expands
    const uint32_t chunk_in_tile = r >> 3, rr = r & 7u;
    uint32_t st = 0, eph = 0, first_round = 1, ps = 0, pph = 0, accph = 0;
    for (uint32_t t = blockIdx.x; t < n_tiles && !dead; t += gridDim.x) {
      const uint32_t rb = t / tok_blocks, tb = t % tok_blocks;
      for (uint32_t sbk = 0; sbk < nsb && !dead; sbk++) {
        if (!__all_sync(0xffffffffu, mbar_wait_bounded(sbase + S.pk_full + ps * 8, pph))) {
          dead = true;  // warp-uniform: these warps execute .aligned tcgen05 instructions later
          break;
        }
        const uint32_t slab = sbase + S.pk + ps * PK_BYTES + chunk_in_tile * PK_CHUNK;
        // header of this row's super-block: d, dmin and the 6-bit fields (reference/q4_k.rs:27-49)
        const uint4 h = lds128(slab + rr * 16);
        const float d = h2f_bits(h.x), dmin = h2f_bits(h.x >> 16);
        const uint32_t sc[2] = {h.y & 0x3F3F3F3Fu, (h.w & 0x0F0F0F0Fu) | ((h.y >> 2) & 0x30303030u)};
        const uint32_t mn[2] = {h.z & 0x3F3F3F3Fu,
                                ((h.w >> 4) & 0x0F0F0F0Fu) | ((h.z >> 2) & 0x30303030u)};
#pragma unroll
        for (int gq = 0; gq < 4; gq++) {
          // sub-blocks 2 gq (low nibbles) and 2 gq + 1 (high nibbles)
          const uint32_t sh = (gq & 1) * 16;
          const float ds_lo = d * (float)((sc[gq >> 1] >> sh) & 0xFF);
          const float ds_hi = d * (float)((sc[gq >> 1] >> (sh + 8)) & 0xFF);
          const float dm_lo = dmin * (float)((mn[gq >> 1] >> sh) & 0xFF);
          const float dm_hi = dmin * (float)((mn[gq >> 1] >> (sh + 8)) & 0xFF);
          const __half2 s_lo = __float2half2_rn(ds_lo), s_hi = __float2half2_rn(ds_hi);
          // (1024 + q) * s - 1024 * s is exact in the FMA, so q * s is rounded once
          const __half2 c_lo = __hmul2(s_lo, __float2half2_rn(-1024.f));
          const __half2 c_hi = __hmul2(s_hi, __float2half2_rn(-1024.f));
          const __half2 m_lo = __float2half2_rn(dm_lo), m_hi = __float2half2_rn(dm_hi);
          const uint4 q0 = lds128(slab + 128 + gq * 256 + rr * 32 + half * 16);
          const uint32_t w[4] = {q0.x, q0.y, q0.z, q0.w};
          if (!first_round &&
              !__all_sync(0xffffffffu, mbar_wait_bounded(sbase + S.ab_empty + st * 8, eph ^ 1))) {
            dead = true;
            break;
          }
          const uint32_t arow = sbase + S.a + st * S.a_stage + r * 128;
#pragma unroll
          for (int i = 0; i < 4; i++) {
            // one packed word -> 8 fp16 weights = one 16-byte chunk of the row
            uint32_t e[4] = {(w[i] & 0x000F000Fu) | 0x64006400u, ((w[i] >> 8) & 0x000F000Fu) | 0x64006400u,
                             ((w[i] >> 4) & 0x000F000Fu) | 0x64006400u,
                             ((w[i] >> 12) & 0x000F000Fu) | 0x64006400u};
            uint32_t o[4];
#pragma unroll
            for (int p = 0; p < 4; p++) {
              const __half2 q = *reinterpret_cast<__half2 *>(&e[p]);
              const __half2 v = p < 2 ? __hsub2(__hfma2(q, s_lo, c_lo), m_lo)
                                      : __hsub2(__hfma2(q, s_hi, c_hi), m_hi);
              o[p] = *reinterpret_cast<const uint32_t *>(&v);
            }
            asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(arow + (((uint32_t)(i + 4 * half) ^ rr) << 4)),
                         "r"(o[0]), "r"(o[1]), "r"(o[2]), "r"(o[3])
                         : "memory");
          }
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // generic writes -> MMA reads
          __syncwarp();
          if (lane == 0) mbar_arrive(sbase + S.ab_full + st * 8);
          if (++st == (uint32_t)NS) st = 0, eph ^= 1, first_round = 0;
        }
        if (dead) break;
        __syncwarp();
        if (lane == 0) mbar_arrive(sbase + S.pk_empty + ps * 8);  // this warp is done with the slab
        if (++ps == (uint32_t)S.pk_stages) ps = 0, pph ^= 1;
      }
      if (dead) break;
      // ---- epilogue: accumulator row (32 * (warp % 4) + lane) of the tile, all BN tokens
      if (!__all_sync(0xffffffffu, mbar_wait_bounded(sbase + S.acc_full, accph))) {
        dead = true;
        break;
      }
      accph ^= 1;
      tc_fence_after();
      const uint32_t lane_row = 32 * (warp & 3u) + lane;
      const uint32_t row = rb * BM + lane_row;
      const uint32_t taddr = tmem_base + ((32 * (warp & 3u)) << 16);
      const int c_begin = BN >= 64 ? (int)half * (BN / 2) : 0;
      const int c_end = BN >= 64 ? c_begin + BN / 2 : (half == 0 ? BN : 0);
#pragma unroll 1
      for (int c0 = c_begin; c0 < c_end; c0 += 32) {
        uint32_t v[32];
        asm volatile(
            "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
            "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
            "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
            : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]),
              "=r"(v[7]), "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]),
              "=r"(v[14]), "=r"(v[15]), "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]),
              "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]),
              "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
            : "r"(taddr + (uint32_t)c0));
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        if (row < L.rows) {
#pragma unroll
          for (int j = 0; j < 32; j++) {
            const uint32_t tok = tb * BN + c0 + j;
            if (tok < m_tokens) y[(uint64_t)tok * ldy + row] = __uint_as_float(v[j]);
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(sbase + S.acc_empty);
    }
    if (dead && lane == 0) atomicOr(status, QK_DEV_TIMEOUT);
  }

  // common exit: the tensor memory is always returned
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (warp == 1)
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                 "r"((uint32_t)(BN < 32 ? 32 : BN))
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

bool plan_gemm(int bn, GemmSmem *S, uint32_t *total) {
  uint32_t off = 0;
  GemmSmem s;
  s.ab_full = off, off += 8 * 8;
  s.ab_empty = off, off += 8 * 8;
  s.pk_full = off, off += MAX_PK_STAGES * 8;
  s.pk_empty = off, off += MAX_PK_STAGES * 8;
  s.acc_full = off, off += 8;
  s.acc_empty = off, off += 8;
  s.tmem_slot = off, off += 16;
  off = (off + 127u) & ~127u;
  s.a_stage = BM * 128;
  s.b_stage = (uint32_t)bn * 128;
  // Shared memory is split between the fp16 operand ring (>= 3 stages) and the ring
  // of packed slabs, which is what hides HBM latency: as deep as fits, up to 8.
  const uint32_t budget = 227u * 1024u - 2048u;
  int stages = bn >= 256 ? 3 : 4;
  int pk_stages = (int)((budget - off - 1024u - stages * (s.a_stage + s.b_stage)) / PK_BYTES);
  if (pk_stages > MAX_PK_STAGES) pk_stages = MAX_PK_STAGES;
  if (pk_stages < 2) return false;
  s.stages = stages, s.pk_stages = pk_stages;
  s.pk = off, off += pk_stages * PK_BYTES;
  off = (off + 1023u) & ~1023u;
  s.a = off, off += stages * s.a_stage;
  s.b = off, off += stages * s.b_stage;
  *S = s, *total = off;
  return true;
}

template <int BN>
cudaError_t launch_gemm(const QkLayout &L, const uint8_t *W, const float *x, float *y, uint32_t m,
                        uint64_t ldy, unsigned *status, unsigned char *scratch, int sm_count,
                        cudaStream_t s) {
  GemmSmem S;
  uint32_t total;
  if (!plan_gemm(BN, &S, &total)) return cudaErrorInvalidConfiguration;
  auto kern = qk_gemm_q4k_tc_kernel<BN>;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
    if (e != cudaSuccess) return e;
    attr_set = true;
  }
  EncodeTiledFn enc = encode_fn();
  if (!enc) return cudaErrorNotSupported;
  const uint32_t Kp = L.nb * 256u;
  const uint32_t tok_blocks = (m + BN - 1) / BN, m_pad = tok_blocks * BN;
  const uint32_t row_blocks = (L.rows + BM - 1) / BM;
  __half *x16 = reinterpret_cast<__half *>(scratch);

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
  c0.gridDim = dim3((unsigned)((n8 + 255) / 256 > 148 * 8 ? 148 * 8 : (n8 + 255) / 256));
  c0.blockDim = dim3(256), c0.stream = s, c0.attrs = at, c0.numAttrs = 1;
  cudaError_t e = cudaLaunchKernelEx(&c0, qk_x16_kernel, x, m, L.cols, m_pad, Kp, x16);
  if (e != cudaSuccess) return e;

  uint32_t grid = tok_blocks * row_blocks;
  if (grid > (uint32_t)sm_count) grid = sm_count;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid), cfg.blockDim = dim3(NTHREADS), cfg.dynamicSmemBytes = total, cfg.stream = s;
  cfg.attrs = at, cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kern, L, W, map, y, ldy, m, tok_blocks, row_blocks, status, S);
}

int pick_bn(uint32_t m) { return m <= 32 ? 32 : m <= 64 ? 64 : m <= 128 ? 128 : 256; }

}  // namespace

bool qk_gemm_tc_supported(const QkLayout &L, uint32_t m) {
  return L.type == QK_T_Q4_K && m >= 1 && L.rows >= 1 && L.nb >= 1;
}

size_t qk_gemm_tc_scratch_bytes(const QkLayout &L, uint32_t m) {
  const int bn = pick_bn(m);
  const uint64_t m_pad = ((m + bn - 1) / bn) * (uint64_t)bn;
  return (size_t)(m_pad * L.nb * 256ull * 2ull);
}

cudaError_t qk_launch_gemm_tc(const QkLayout &L, const uint8_t *tiled, const float *x, float *y,
                              uint32_t m, uint64_t ldy, unsigned *status, unsigned char *scratch,
                              int sm_count, cudaStream_t s) {
  switch (pick_bn(m)) {
    case 32:
      return launch_gemm<32>(L, tiled, x, y, m, ldy, status, scratch, sm_count, s);
    case 64:
      return launch_gemm<64>(L, tiled, x, y, m, ldy, status, scratch, sm_count, s);
    case 128:
      return launch_gemm<128>(L, tiled, x, y, m, ldy, status, scratch, sm_count, s);
    default:
      return launch_gemm<256>(L, tiled, x, y, m, ldy, status, scratch, sm_count, s);
  }
}
