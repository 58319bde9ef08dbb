// Decode-path dequant-dot (M <= 4 activation rows): HBM-bound, so the kernel is
// built around keeping many bulk copies in flight and spending few issue slots
// per weight byte.
//
// Shape of the kernel
//  * Persistent: one CTA per SM slot, CTA i takes row-chunks i, i+grid, ...
//    (a chunk = 8 weight rows; its k-tiles are contiguous spans of HBM).
//  * One elected thread streams tiles into a ring of shared-memory stages with
//    cp.async.bulk (global -> shared, completion on an mbarrier); all waits on
//    those barriers are bounded and raise QK_DEV_TIMEOUT instead of spinning.
//  * While the first tiles are in flight every CTA splits the f32 activations
//    into base-254 signed 8-bit digits per 32-column block:
//        x ~= sx * (D0 + D1/254 + D2/254^2),  |x - x~| <= amax * 6.1e-8
//    (two digits: 1.5e-5) and keeps block sums of x for the min / zero-point
//    terms.  Weights are small integers, so the inner product becomes exact
//    integer dp4a work; the f32 rounding that remains is one scale multiply and
//    one add per 32 weights, well inside what f32 summation order costs anyway.
//  * A thread owns a 64-weight unit of a row for several rows of the chunk, so
//    the digit registers are reused across rows; partial sums are reduced with
//    warp shuffles, then across warps through shared memory.
//
// Result: y[m][row] = sum_c w(row,c) x[m][c] with w exactly the reference's
// dequantised weight (reference/q4_k.rs:133-181 and siblings), accumulated in
// a different order and with x carried to ~24 bits.
#include "qk_formats.cuh"
#include "qk_kernels.h"
#include "qk_pipe.cuh"

using namespace qkpipe;

namespace {

constexpr int NT = 256;          // threads per CTA
constexpr int NWARP = NT / 32;

// Position of column e's digit byte inside its 256-column span, per format:
// the order in which the format's packed words meet their activations.
template <int TYPE>
__device__ __forceinline__ uint32_t x_pos(uint32_t e) {
  uint32_t s = e & ~255u, o = e & 255u, p;
  if (TYPE == QK_T_Q4_0) {
    // byte i of a block holds elements 2i (low nibble) and 2i+1 (high):
    // evens first, then odds, inside every 32-block (reference/q4_0.rs:40-46)
    uint32_t b = o & ~31u, i = o & 31u;
    p = b + ((i & 1u) << 4) + (i >> 1);
  } else if (TYPE == QK_T_Q6_K) {
    // unit (G, is) gathers the four 16-column strips k = 0..3 it decodes
    // together (reference/q6_k.rs:51-70)
    uint32_t G = o >> 7, k = (o >> 5) & 3u, is = (o >> 4) & 1u, b = o & 15u;
    p = ((2u * G + is) << 6) + (k << 4) + b;
  } else {
    p = o;  // Q4_K, Q8_0: natural order
  }
  // 16-byte slots of a 64-byte unit are XOR-swizzled by the unit index so that
  // consecutive lanes (consecutive units) hit distinct banks.
  uint32_t u = (s + p) >> 6, j = (p >> 4) & 3u;
  return ((s + p) & ~48u) | ((j ^ ((u >> 1) & 3u)) << 4);
}

struct Smem {
  uint32_t bars;   // mbarriers, 8 B each
  uint32_t xd;     // digit planes  [M][D][Kp]
  uint32_t xs;     // per 32-block float4 (sx, S32, S16a, S16b)  [M][Kp/32]
  uint32_t dec;    // decoded per-unit scales of the current tile
  uint32_t red;    // cross-warp reduction  [NWARP][8]
  uint32_t flag;   // abort flag
  uint32_t stage;  // ring of tiles
};

// Fills the CTA's digit planes and block statistics from x (global, f32).
// `after_first_loads` runs once per thread, right after its first activation loads are issued.
template <int TYPE, int M, int D, typename F>
__device__ void prep_x(const QkLayout &L, const float *__restrict__ x, unsigned char *smem,
                       const Smem &S, uint32_t Kp, F &&after_first_loads) {
  const uint32_t quads = Kp / 4;
  for (uint32_t it = threadIdx.x; it < (uint32_t)M * quads; it += NT) {
    uint32_t m = M == 1 ? 0u : it / quads, q = M == 1 ? it : it % quads, e0 = q * 4;
    float v[4];
#pragma unroll
    for (int i = 0; i < 4; i++)
      v[i] = (e0 + i < L.cols) ? x[(uint64_t)m * L.cols + e0 + i] : 0.f;
    if (it == threadIdx.x) after_first_loads();
    float amax = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));
    float s4 = (v[0] + v[1]) + (v[2] + v[3]);
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 4));
    s4 += __shfl_xor_sync(0xffffffffu, s4, 1);
    s4 += __shfl_xor_sync(0xffffffffu, s4, 2);  // sum of this thread's 16-column half
    float other = __shfl_xor_sync(0xffffffffu, s4, 4);
    if (!(amax < 8.0e37f)) amax = 8.0e37f;  // inf/nan/huge x: keep the scale finite (__fdividef: y < 2^126)
    float inv = amax > 0.f ? __fdividef(127.f, amax) : 0.f;
    // Balanced base-254 digits by magic-number rounding: adding 1.5 * 2^23 rounds to the
    // nearest integer and leaves it, as two's complement, in the low mantissa byte; with
    // |v| <= amax every digit lies in [-127, 127] without a clamp.
    constexpr float MAGIC = 12582912.f;
#pragma unroll
    for (int i = 0; i < 4; i++) {
      const float t0 = fmaf(v[i], inv, MAGIC);
      const float r1 = fmaf(v[i], inv, -(t0 - MAGIC));  // exact residual of the first digit
      const float t1 = fmaf(r1, 254.f, MAGIC);
      const float r2 = fmaf(r1, 254.f, -(t1 - MAGIC));
      const float t2 = fmaf(r2, 254.f, MAGIC);
      uint32_t pos = x_pos<TYPE>(e0 + i);
      unsigned char *base = smem + S.xd + (size_t)m * D * Kp + pos;
      base[0] = (unsigned char)__float_as_uint(t0);
      base[Kp] = (unsigned char)__float_as_uint(t1);
      if (D == 3) base[2 * Kp] = (unsigned char)__float_as_uint(t2);
    }
    if ((threadIdx.x & 7) == 0) {
      float4 st = make_float4(amax * (1.f / 127.f), s4 + other, s4, other);
      *reinterpret_cast<float4 *>(smem + S.xs + ((size_t)m * (Kp / 32) + e0 / 32) * 16) =
          st;
    }
  }
}

// Combines the integer digit dots into sx * (I0 + I1/254 + I2/254^2).
template <int D>
__device__ __forceinline__ float digits_to_f32(const int *I, float sx) {
  float p = (float)I[D - 1];
#pragma unroll
  for (int d = D - 2; d >= 0; d--) p = fmaf(p, 1.f / 254.f, (float)I[d]);
  return p * sx;
}

template <int TYPE, int M, int D, int RS>
__global__ void __launch_bounds__(NT)
    qk_gemv_kernel(QkLayout L, const uint8_t *__restrict__ W, const float *__restrict__ x,
                   float *__restrict__ y, uint64_t ldy, unsigned *status, int nstage,
                   uint32_t stage_bytes, Smem S, uint32_t Kp, int npre) {
  extern __shared__ __align__(128) unsigned char smem[];
  // Eight neighbouring lanes take the eight rows of a chunk and the same 64-weight unit:
  // their 16-byte weight reads are one 128-byte span of the block-major tile (no bank
  // conflict) and their activation reads one broadcast.
  static_assert(RS == 8, "one row per lane");
  constexpr int RPT = 1;                  // rows per thread
  constexpr int UL = NT / 8;              // units in flight per pass of the CTA
  const uint32_t sbase = smem_u32(smem);  // S.* are offsets from here (S.bars == 0)
  const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t split = lane & 7u, ulane = threadIdx.x >> 3;
  volatile int *abort_flag = reinterpret_cast<volatile int *>(smem + S.flag);

  const uint32_t my_chunks =
      blockIdx.x < L.chunks ? (L.chunks - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
  const uint32_t my_items = my_chunks * L.ktiles;

  auto issue = [&](uint32_t item) {  // thread 0 only
    uint32_t chunk = blockIdx.x + (item / L.ktiles) * gridDim.x, kt = item % L.ktiles;
    uint32_t bytes = QK_TILE_ROWS * qk_tile_nb(L, kt) * L.bb;
    uint32_t st = item % nstage;
    uint32_t bar = sbase + S.bars + st * 8;
    mbar_expect_tx(bar, bytes);
    bulk_g2s_stream(sbase + S.stage + st * stage_bytes, W + qk_tile_offset(L, chunk, kt), bytes, bar);
  };

  // Programmatic dependent launch: the next kernel in the stream may start its prologue
  // as this one's CTAs retire, and this one prefetches its (immutable) weights before it
  // waits for the previous kernel, whose output x may be.
  pdl_launch_dependents();
  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int s = 0; s < nstage; s++) mbar_init(sbase + S.bars + s * 8, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    for (uint32_t i = 0; i < (uint32_t)npre && i < my_items; i++) issue(i);
  }
  pdl_wait();  // x and y belong to the previous kernel until it has finished
  // The rest of the first ring fill goes out behind the activation loads, not ahead of
  // them: queued behind a whole ring of weight tiles from every CTA those loads take
  // about a microsecond longer.
  prep_x<TYPE, M, D>(L, x, smem, S, Kp, [&]() {
    if (threadIdx.x == 0)
      for (uint32_t i = (uint32_t)npre; i < (uint32_t)nstage && i < my_items; i++) issue(i);
  });
  __syncthreads();

  float acc[M][RPT];
#pragma unroll
  for (int m = 0; m < M; m++)
#pragma unroll
    for (int r = 0; r < RPT; r++) acc[m][r] = 0.f;

  for (uint32_t item = 0; item < my_items; item++) {
    const uint32_t chunk = blockIdx.x + (item / L.ktiles) * gridDim.x, kt = item % L.ktiles;
    const uint32_t st = item % nstage, nbt = qk_tile_nb(L, kt);
    const uint32_t tile = sbase + S.stage + st * stage_bytes;
    if (!mbar_wait_bounded(sbase + S.bars + st * 8, (item / nstage) & 1)) {
      *abort_flag = 1;
      atomicOr(status, QK_DEV_TIMEOUT);
    }

    // ---- per-tile scale decode into floats (one thread per block of the tile)
    if (TYPE == QK_T_Q6_K) {
      for (uint32_t i = threadIdx.x; i < 8 * nbt; i += NT) {  // i = r * nbt + sb
        const uint32_t blk = tile + (i % nbt) * 1680u, ri = i / nbt;  // block-major: ql+qh 1536 | scales 128 | d 16
        uint4 s = lds128(blk + 1536 + ri * 16);
        uint32_t dw = lds32(blk + 1664 + (ri & ~1u) * 2);
        float d = h2f_bits((ri & 1) ? (dw >> 16) : dw);
        uint32_t w[4] = {s.x, s.y, s.z, s.w};
#pragma unroll
        for (int u = 0; u < 4; u++) {  // unit u = 2G + is needs scales 8G + is + 2k
          int G = u >> 1, is = u & 1;
          float4 o;
          o.x = d * (float)(int8_t)(w[2 * G] >> (8 * is));
          o.y = d * (float)(int8_t)(w[2 * G] >> (8 * (is + 2)));
          o.z = d * (float)(int8_t)(w[2 * G + 1] >> (8 * is));
          o.w = d * (float)(int8_t)(w[2 * G + 1] >> (8 * (is + 2)));
          *reinterpret_cast<float4 *>(smem + S.dec + (((i % nbt) * 4 + u) * 8 + ri) * 16) = o;  // [sb][unit][row]
        }
      }
      __syncthreads();
    }

    // ---- main: units of 64 weights, RPT rows each
    const uint32_t units = nbt * (L.bs == 32 ? 1u : 8u) / 2u;  // 64-weight units per row in this tile
    const uint32_t kbase = kt * QK_TILE_ELEMS;                 // first column of the tile
    for (uint32_t u = ulane; u < units; u += UL) {
      // digit registers for this unit: 16 words per (m, d)
      uint32_t xw[M][D][16];
      const uint32_t xoff = kbase + u * 64, sw = ((xoff >> 6) >> 1) & 3u;
#pragma unroll
      for (int m = 0; m < M; m++)
#pragma unroll
        for (int d = 0; d < D; d++)
#pragma unroll
          for (int j = 0; j < 4; j++) {
            uint4 t = lds128(sbase + S.xd + (m * D + d) * Kp + xoff + ((j ^ sw) << 4));
            xw[m][d][4 * j] = t.x, xw[m][d][4 * j + 1] = t.y;
            xw[m][d][4 * j + 2] = t.z, xw[m][d][4 * j + 3] = t.w;
          }
#pragma unroll
      for (int rr = 0; rr < RPT; rr++) {
        const uint32_t r = split * RPT + rr;
        if (TYPE == QK_T_Q4_0 || TYPE == QK_T_Q8_0) {
          // block-major: a block's 8 rows are [nibbles or int8s, 16-byte granules x 8 rows][d, 8 x 2]
          const uint32_t bsz = TYPE == QK_T_Q4_0 ? 144u : 272u, doff = TYPE == QK_T_Q4_0 ? 128u : 256u;
          const uint32_t b0 = 2 * u;  // blocks 2u, 2u+1 of this row in the tile
#pragma unroll
          for (int j = 0; j < 2; j++) {
            if (b0 + j >= nbt) break;
            const uint32_t blk = tile + (b0 + j) * bsz;
            const uint32_t dw = lds32(blk + doff + (r & ~1u) * 2);
            float dj = h2f_bits((r & 1u) ? (dw >> 16) : dw);
            if (TYPE == QK_T_Q4_0) {
              uint4 q = lds128(blk + r * 16);
              uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
              for (int m = 0; m < M; m++) {
                int Ie[D], Io[D];
#pragma unroll
                for (int d = 0; d < D; d++) {
                  int ie = 0, io = 0;
#pragma unroll
                  for (int k = 0; k < 4; k++) {
                    ie = dp4a_us(w[k] & 0x0F0F0F0Fu, xw[m][d][8 * j + k], ie);
                    io = dp4a_us(w[k] & 0xF0F0F0F0u, xw[m][d][8 * j + 4 + k], io);
                  }
                  Ie[d] = ie, Io[d] = io;
                }
                float4 s = lds128f(sbase + S.xs + (m * (Kp / 32) + (xoff >> 5) + j) * 16);
                float p = fmaf(digits_to_f32<D>(Io, s.x), 1.f / 16.f, digits_to_f32<D>(Ie, s.x));
                acc[m][rr] = fmaf(dj, fmaf(-8.f, s.y, p), acc[m][rr]);  // (q - 8) zero point
              }
            } else {
              uint4 q0 = lds128(blk + r * 16);
              uint4 q1 = lds128(blk + 128 + r * 16);
              uint32_t w[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
#pragma unroll
              for (int m = 0; m < M; m++) {
                int I[D];
#pragma unroll
                for (int d = 0; d < D; d++) {
                  int i0 = 0;
#pragma unroll
                  for (int k = 0; k < 8; k++) i0 = dp4a_ss(w[k], xw[m][d][8 * j + k], i0);
                  I[d] = i0;
                }
                float4 s = lds128f(sbase + S.xs + (m * (Kp / 32) + (xoff >> 5) + j) * 16);
                acc[m][rr] = fmaf(dj, digits_to_f32<D>(I, s.x), acc[m][rr]);
              }
            }
          }
        } else {  // Q6_K: unit = (sb, G, is); strips k = 0..3 of 16 columns each
          const uint32_t sb = u >> 2, G = (u >> 1) & 1u, is = u & 1u;
          const uint32_t qb = tile + sb * 1680u + r * 16;  // byte o of ql+qh: granule o / 16 of the block
          uint4 a = lds128(qb + (4 * G + is) * 128), b = lds128(qb + (4 * G + 2 + is) * 128);
          uint4 h = lds128(qb + (8 + 2 * G + is) * 128);
          float4 sc = lds128f(sbase + S.dec + ((sb * 4 + (u & 3u)) * 8 + r) * 16);
          uint32_t aw[4] = {a.x, a.y, a.z, a.w}, bw[4] = {b.x, b.y, b.z, b.w};
          uint32_t hw[4] = {h.x, h.y, h.z, h.w};
          uint32_t q[4][4];  // [strip][word], reference/q6_k.rs:55-60
#pragma unroll
          for (int i = 0; i < 4; i++) {
            q[0][i] = (aw[i] & 0x0F0F0F0Fu) | ((hw[i] << 4) & 0x30303030u);
            q[1][i] = (bw[i] & 0x0F0F0F0Fu) | ((hw[i] << 2) & 0x30303030u);
            q[2][i] = ((aw[i] >> 4) & 0x0F0F0F0Fu) | (hw[i] & 0x30303030u);
            q[3][i] = ((bw[i] >> 4) & 0x0F0F0F0Fu) | ((hw[i] >> 2) & 0x30303030u);
          }
          const float scs[4] = {sc.x, sc.y, sc.z, sc.w};
#pragma unroll
          for (int m = 0; m < M; m++) {
            // the unit's four strips sit in x-blocks 4G .. 4G+3 of the super-block
            const uint32_t xsa =
                sbase + S.xs + (m * (Kp / 32) + ((kbase + sb * 256) >> 5) + 4 * G) * 16;
            float t = acc[m][rr];
#pragma unroll
            for (int k = 0; k < 4; k++) {
              int I[D];
#pragma unroll
              for (int d = 0; d < D; d++) {
                int i0 = 0;
#pragma unroll
                for (int i = 0; i < 4; i++) i0 = dp4a_us(q[k][i], xw[m][d][4 * k + i], i0);
                I[d] = i0;
              }
              float4 s = lds128f(xsa + 16 * k);
              float p = fmaf(-32.f, is ? s.w : s.z, digits_to_f32<D>(I, s.x));  // (q - 32)
              t = fmaf(scs[k], p, t);
            }
            acc[m][rr] = t;
          }
        }
      }
    }
    __syncthreads();  // everyone is done with this stage (and with `dec`)
    if (*abort_flag) break;
    if (threadIdx.x == 0 && item + nstage < my_items) issue(item + nstage);

    if (kt + 1 == L.ktiles) {  // chunk finished: reduce and write 8 rows x M
      const uint32_t red_parity = (item / L.ktiles) & 1;  // double-buffered
      float *red = reinterpret_cast<float *>(smem + S.red) + red_parity * (NWARP * M * 8);
#pragma unroll
      for (int m = 0; m < M; m++) {
        float v = acc[m][0];
        v += __shfl_xor_sync(0xffffffffu, v, 16);
        v += __shfl_xor_sync(0xffffffffu, v, 8);  // lanes 0..7: this warp's sum for rows 0..7
        if (lane < 8) red[warp * (M * 8) + m * 8 + lane] = v;
        acc[m][0] = 0.f;
      }
      __syncthreads();
      if (threadIdx.x < 8 * M) {
        uint32_t m = threadIdx.x / 8, r = threadIdx.x % 8;
        float v = 0.f;
#pragma unroll
        for (int wv = 0; wv < NWARP; wv++) v += red[wv * (M * 8) + m * 8 + r];
        uint32_t row = chunk * 8 + r;
        if (row < L.rows) y[(uint64_t)m * ldy + row] = v;
      }
    }
  }

  if (*abort_flag && threadIdx.x == 0) {
    // give copies already issued a bounded chance to land before the CTA exits
    for (int s = 0; s < nstage; s++) {
      mbar_wait_bounded(sbase + S.bars + s * 8, 0);
      mbar_wait_bounded(sbase + S.bars + s * 8, 1);
    }
  }
}

struct Plan {
  Smem S;
  uint32_t Kp, stage_bytes, total;
  int nstage, ctas_per_sm, D;
};

bool make_plan(const QkLayout &L, uint32_t m, int RS, Plan *P) {
  (void)RS;
  if (L.nb == 0 || L.chunks == 0) return false;  // nothing to stream: the callers handle empty shapes
  uint32_t Kp = L.nb * L.bs;
  Kp = (Kp + 255u) & ~255u;
  // Activation digits (base 254): three give f32-grade results (~2e-6 of the output's
  // inf-norm, the f32 reference's own distance from an f64 sum); two measured 5e-5 for 9 %
  // less time on the Q6_K LM head, so three are kept up to M = 2.  QK_DIGITS=2 is a
  // developer knob for M <= 2.
  int D = m <= 2 ? 3 : 2;
  if (m <= 2)
    if (const char *e = qk_knob("QK_DIGITS")) D = atoi(e) == 2 ? 2 : atoi(e) == 3 ? 3 : D;
  uint32_t nbt_max = L.nb < L.nbt ? L.nb : L.nbt;
  uint32_t stage_bytes = QK_TILE_ROWS * nbt_max * L.bb;
  stage_bytes = (stage_bytes + 127u) & ~127u;
  uint32_t dec_bytes = L.type == QK_T_Q6_K ? 8 * nbt_max * 64 : 0;
  uint32_t off = 0;
  Smem S;
  S.bars = off, off += 64;  // up to 8 stages
  S.flag = off, off += 16;
  S.red = off, off += 2 * NWARP * 4 * 8 * 4;
  off = (off + 127u) & ~127u;
  S.xd = off, off += m * D * Kp;
  S.xs = off, off += m * (Kp / 32) * 16;
  S.dec = off, off += dec_bytes;
  off = (off + 127u) & ~127u;
  S.stage = off;
  const uint32_t budget = 227u * 1024u;
  if (off + 2 * stage_bytes > budget) return false;
  // Prefer 2 CTAs per SM (barrier bubbles of one hide behind the other) when
  // each can still keep >= 3 tiles in flight.
  int ctas = 1, nstage;
  uint32_t per2 = (budget / 2) - 1024;
  if (off + 3 * stage_bytes <= per2) {
    ctas = 2;
    nstage = (int)((per2 - off) / stage_bytes);
  } else {
    nstage = (int)((budget - 1024 - off) / stage_bytes);
  }
  if (nstage > 8) nstage = 8;
  if (nstage < 2) return false;
  P->S = S, P->Kp = Kp, P->stage_bytes = stage_bytes, P->nstage = nstage;
  P->ctas_per_sm = ctas, P->D = D;
  P->total = off + nstage * stage_bytes;
  return true;
}

template <int TYPE, int M, int D, int RS>
cudaError_t launch_one(const QkLayout &L, const uint8_t *W, const float *x, float *y, uint64_t ldy,
                       unsigned *status, int sm_count, const Plan &P, cudaStream_t s) {
  auto kern = qk_gemv_kernel<TYPE, M, D, RS>;
  static QkPerDevice attr_set;
  if (attr_set.first()) {
    cudaError_t e =
        cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
    if (e != cudaSuccess) return attr_set.reset(), e;
  }
  // A persistent grid must be fully resident: size it from the real occupancy.
  static int occ_cached[2] = {0, 0};  // [0] smem it was computed for, [1] CTAs per SM
  if (occ_cached[0] != (int)P.total) {
    int occ = 0;
    cudaError_t e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, kern, NT, P.total);
    if (e != cudaSuccess) return e;
    if (occ < 1) return cudaErrorLaunchOutOfResources;
    occ_cached[0] = (int)P.total, occ_cached[1] = occ;
  }
  int ctas = occ_cached[1] < P.ctas_per_sm ? occ_cached[1] : P.ctas_per_sm;
  uint32_t grid = (uint32_t)sm_count * ctas;
  if (grid > L.chunks) grid = L.chunks;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[0].val.programmaticStreamSerializationAllowed = 1;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid), cfg.blockDim = dim3(NT), cfg.dynamicSmemBytes = P.total, cfg.stream = s;
  cfg.attrs = at, cfg.numAttrs = 1;
  static int npre_env = -1;  // developer knob: weight tiles issued before the wait on the previous kernel
  if (npre_env < 0) {
    const char *e = qk_knob("QK_PRE");
    npre_env = e ? atoi(e) : 0;
  }
  // Default: the whole ring.  Holding tiles back until the activation loads are out (what
  // the Q4_K kernel does) measured within 3 % either way here: Q8_0 4096^2 7.9 us with two
  // tiles first against 8.1 us, Q6_K 4096 x 14336 28.9 us against 28.2 us.
  int npre = npre_env > 0 ? npre_env : P.nstage;
  if (npre > P.nstage) npre = P.nstage;
  return cudaLaunchKernelEx(&cfg, kern, L, W, x, y, ldy, status, P.nstage, P.stage_bytes, P.S, P.Kp, npre);
}

// Row splits: as many rows per thread as still leave every warp a unit to work on.
int pick_rs(const QkLayout &L) {
  uint32_t nbt_max = L.nb < L.nbt ? L.nb : L.nbt;
  uint32_t units = nbt_max * (L.bs == 32 ? 1u : 8u) / 2u;
  if (units == 0) units = 1;
  (void)units;
  return 8;  // one row per lane
}

template <int TYPE, int M, int D>
cudaError_t launch_rs(int rs, const QkLayout &L, const uint8_t *W, const float *x, float *y,
                      uint64_t ldy, unsigned *status, int sm_count, const Plan &P, cudaStream_t s) {
  (void)rs;
  return launch_one<TYPE, M, D, 8>(L, W, x, y, ldy, status, sm_count, P, s);
}

template <int TYPE>
cudaError_t launch_m(uint32_t m, int rs, const QkLayout &L, const uint8_t *W, const float *x,
                     float *y, uint64_t ldy, unsigned *status, int sm_count, const Plan &P,
                     cudaStream_t s) {
  switch (m) {
    case 1:
      if (P.D == 2) return launch_rs<TYPE, 1, 2>(rs, L, W, x, y, ldy, status, sm_count, P, s);
      return launch_rs<TYPE, 1, 3>(rs, L, W, x, y, ldy, status, sm_count, P, s);
    case 2:
      if (P.D == 2) return launch_rs<TYPE, 2, 2>(rs, L, W, x, y, ldy, status, sm_count, P, s);
      return launch_rs<TYPE, 2, 3>(rs, L, W, x, y, ldy, status, sm_count, P, s);
    case 3:
      return launch_rs<TYPE, 3, 2>(rs, L, W, x, y, ldy, status, sm_count, P, s);
    default:
      return launch_rs<TYPE, 4, 2>(rs, L, W, x, y, ldy, status, sm_count, P, s);
  }
}

}  // namespace

bool qk_gemv_fast_supported(const QkLayout &L, uint32_t m) {
  if (m < 1 || m > QK_GEMV_MAX_M) return false;
  if (L.type == QK_T_Q4_K) return qk_gemv_mma_supported(L, m);
  if (L.type == QK_T_IQ4_XS) return false;
  if (L.bs == 32 && (L.nb & 1u)) return false;  // 64-weight units pair two 32-blocks
  Plan P;
  return make_plan(L, m, pick_rs(L), &P);
}

size_t qk_gemv_fast_scratch_bytes(const QkLayout &L, uint32_t m) {
  return L.type == QK_T_Q4_K ? qk_gemv_mma_scratch_bytes(L, m) : 0;
}

cudaError_t qk_launch_gemv_fast(const QkLayout &L, const uint8_t *tiled, const float *x, float *y,
                                uint32_t m, uint64_t ldy, unsigned *status, unsigned char *scratch,
                                int sm_count, cudaStream_t s) {
  if (L.type == QK_T_Q4_K)
    return qk_launch_gemv_mma(L, tiled, x, y, m, ldy, status, scratch, sm_count, s);
  Plan P;
  int rs = pick_rs(L);
  if (!make_plan(L, m, rs, &P)) return cudaErrorInvalidConfiguration;
  switch (L.type) {
    case QK_T_Q4_0:
      return launch_m<QK_T_Q4_0>(m, rs, L, tiled, x, y, ldy, status, sm_count, P, s);
    case QK_T_Q8_0:
      return launch_m<QK_T_Q8_0>(m, rs, L, tiled, x, y, ldy, status, sm_count, P, s);
    case QK_T_Q6_K:
      return launch_m<QK_T_Q6_K>(m, rs, L, tiled, x, y, ldy, status, sm_count, P, s);
    default:
      return cudaErrorInvalidValue;
  }
}

// ---- decode kernels with the output fan-out built in
bool qk_gemv_peer_supported(const QkLayout &L, uint32_t m) {
  return L.type == QK_T_Q4_K && qk_gemv_mma_supported(L, m);
}

size_t qk_gemv_peer_scratch_bytes(const QkLayout &L, uint32_t m) { return qk_gemv_mma_scratch_bytes(L, m); }

cudaError_t qk_launch_gemv_peer(const QkLayout &L, const uint8_t *tiled, const float *x, uint32_t m,
                                uint64_t ldy, unsigned *status, unsigned char *scratch, int sm_count,
                                cudaStream_t s, const QkPeers *peers) {
  if (L.type != QK_T_Q4_K) return cudaErrorNotSupported;
  return qk_launch_gemv_mma(L, tiled, x, nullptr, m, ldy, status, scratch, sm_count, s, peers);
}
