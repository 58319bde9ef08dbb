// Generic kernels: re-tiling at upload, bit-exact dequantisation, an any-shape
// f32 dequant-dot (the path for shapes the specialised kernels do not take),
// the Q8_0-activation fused matvec and the Q8_0 activation encoder.
#include "qk_formats.cuh"
#include "qk_kernels.h"

// ---------------------------------------------------------------- re-tile
// One thread moves one 16-bit unit (every field width and GGUF offset is even).
__global__ void qk_repack_kernel(QkLayout L, const uint8_t *__restrict__ raw,
                                 uint8_t *__restrict__ tiled) {
  uint64_t units_per_block = L.bb / 2;
  uint64_t total = (uint64_t)L.rows * L.nb * units_per_block;
  for (uint64_t u = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x; u < total;
       u += (uint64_t)gridDim.x * blockDim.x) {
    uint64_t gblk = u / units_per_block;
    uint32_t off = (uint32_t)(u % units_per_block) * 2;  // byte offset inside the GGUF block
    uint32_t row = (uint32_t)(gblk / L.nb), blk = (uint32_t)(gblk % L.nb);
    int p = 0;
    for (int i = 0; i < (int)L.nplanes; i++)
      if (off >= L.po[i] && off < L.po[i] + L.pw[i]) p = i;
    uint64_t dst = qk_byte_offset(L, row, blk, p, off - L.po[p]);
    *reinterpret_cast<uint16_t *>(tiled + dst) =
        *reinterpret_cast<const uint16_t *>(raw + gblk * L.bb + off);
  }
}

cudaError_t qk_launch_repack(const QkLayout &L, const uint8_t *raw_dev, uint8_t *tiled_dev,
                             cudaStream_t s) {
  uint64_t total = (uint64_t)L.rows * L.nb * (L.bb / 2);
  if (total == 0) return cudaSuccess;
  uint64_t blocks = (total + 255) / 256;
  if (blocks > 148ull * 64) blocks = 148ull * 64;
  qk_repack_kernel<<<(unsigned)blocks, 256, 0, s>>>(L, raw_dev, tiled_dev);
  return cudaGetLastError();
}

// ---------------------------------------------------------------- dequant
__global__ void qk_dequant_kernel(QkLayout L, const uint8_t *__restrict__ tiled,
                                  float *__restrict__ out) {
  uint64_t total = (uint64_t)L.rows * L.cols;
  for (uint64_t e = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x; e < total;
       e += (uint64_t)gridDim.x * blockDim.x) {
    uint32_t row = (uint32_t)(e / L.cols), col = (uint32_t)(e % L.cols);
    out[e] = qk_dequant_elem(L, tiled, row, col);
  }
}

cudaError_t qk_launch_dequant(const QkLayout &L, const uint8_t *tiled, float *out, cudaStream_t s) {
  uint64_t total = (uint64_t)L.rows * L.cols;
  if (total == 0) return cudaSuccess;
  uint64_t blocks = (total + 255) / 256;
  if (blocks > 148ull * 32) blocks = 148ull * 32;
  qk_dequant_kernel<<<(unsigned)blocks, 256, 0, s>>>(L, tiled, out);
  return cudaGetLastError();
}

// ---------------------------------------------------------------- generic dequant-dot
// One warp per weight row; lanes stride over columns; each weight is decoded
// once and multiplied into up to MT activation rows.  f32 FMA per lane, then a
// shuffle tree: the sum order differs from the reference's sequential sum (by
// ~1e-6 relative), the products do not.
#define QK_SIMPLE_MT 8
__global__ void __launch_bounds__(128)
    qk_gemm_simple_kernel(QkLayout L, const uint8_t *__restrict__ tiled,
                          const float *__restrict__ x, float *__restrict__ y, uint32_t m,
                          uint64_t ldy) {
  uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  uint32_t row = blockIdx.x * 4 + warp;
  if (row >= L.rows) return;
  for (uint32_t m0 = blockIdx.y * QK_SIMPLE_MT; m0 < m; m0 += gridDim.y * QK_SIMPLE_MT) {
    float acc[QK_SIMPLE_MT];
#pragma unroll
    for (int i = 0; i < QK_SIMPLE_MT; i++) acc[i] = 0.f;
    for (uint32_t c = lane; c < L.cols; c += 32) {
      float w = qk_dequant_elem(L, tiled, row, c);
#pragma unroll
      for (int i = 0; i < QK_SIMPLE_MT; i++)
        if (m0 + i < m) acc[i] = fmaf(w, x[(uint64_t)(m0 + i) * L.cols + c], acc[i]);
    }
#pragma unroll
    for (int i = 0; i < QK_SIMPLE_MT; i++) {
      float v = acc[i];
      for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
      if (lane == 0 && m0 + i < m) y[(uint64_t)(m0 + i) * ldy + row] = v;
    }
  }
}

cudaError_t qk_launch_gemm_simple(const QkLayout &L, const uint8_t *tiled, const float *x, float *y,
                                  uint32_t m, uint64_t ldy, cudaStream_t s) {
  if (L.rows == 0 || m == 0) return cudaSuccess;
  uint32_t mt = (m + QK_SIMPLE_MT - 1) / QK_SIMPLE_MT;
  if (mt > 64) mt = 64;
  dim3 grid((L.rows + 3) / 4, mt);
  qk_gemm_simple_kernel<<<grid, 128, 0, s>>>(L, tiled, x, y, m, ldy);
  return cudaGetLastError();
}

// ---------------------------------------------------------------- Q8_0-activation fused matvec
// out[row] += sum_c w(row,c) * (d_a * q_a)(c), with w the f32 dequantised weight
// and the activation taken from Q8_0 block c/32 (traits.rs:89-173; the K-quant
// overrides pair one super-block with eight Q8_0 blocks, reference/q4_k.rs:218-333,
// reference/q6_k.rs:212-354).  Algebraically the reference's per-format formulas;
// sum order differs.
__global__ void __launch_bounds__(128)
    qk_fused_simple_kernel(QkLayout L, const uint8_t *__restrict__ tiled,
                           const uint8_t *__restrict__ acts, float *__restrict__ out) {
  uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  uint32_t row = blockIdx.x * 4 + warp;
  if (row >= L.rows) return;
  float acc = 0.f;
  for (uint32_t c = lane; c < L.cols; c += 32) {
    const uint8_t *ab = acts + (uint64_t)(c >> 5) * 34;
    float a = __fmul_rn((float)(int8_t)ab[2 + (c & 31)], qk_h2f(ab));
    acc = fmaf(qk_dequant_elem(L, tiled, row, c), a, acc);
  }
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if (lane == 0) out[row] += acc;
}

cudaError_t qk_launch_fused_simple(const QkLayout &L, const uint8_t *tiled, const uint8_t *acts,
                                   float *out, cudaStream_t s) {
  if (L.rows == 0) return cudaSuccess;
  qk_fused_simple_kernel<<<(L.rows + 3) / 4, 128, 0, s>>>(L, tiled, acts, out);
  return cudaGetLastError();
}

// ---------------------------------------------------------------- Q8_0 encoder
// quantize.rs:190-210, bit for bit: amax, d = amax/127, id = 1/d (0 if d == 0),
// q = clamp(round_half_away(x*id)), stored scale = f16(d).  One warp per block.
__global__ void __launch_bounds__(128)
    qk_quantize_q8_0_kernel(const float *__restrict__ x, uint64_t nblocks,
                            uint8_t *__restrict__ out) {
  uint64_t b = (uint64_t)blockIdx.x * 4 + (threadIdx.x >> 5);
  uint32_t lane = threadIdx.x & 31;
  if (b >= nblocks) return;
  float v = x[b * 32 + lane];
  float a = fabsf(v);
  if (a != a) a = 0.f;  // f32::max ignores NaN operands
  for (int o = 16; o > 0; o >>= 1) a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, o));
  float d = __fdiv_rn(a, 127.0f);
  float id = d != 0.0f ? __fdiv_rn(1.0f, d) : 0.0f;
  float r = roundf(__fmul_rn(v, id));
  int q = (r != r) ? 0 : (r >= 127.f ? 127 : (r <= -128.f ? -128 : (int)r));
  uint8_t *o = out + b * 34;
  const unsigned h = __half_as_ushort(__float2half_rn(d));
  if (lane < 2) o[lane] = (uint8_t)((h >> (8 * lane)) & 0xFFu);  // f16 scale, little-endian
  o[2 + lane] = (uint8_t)(int8_t)q;
}

cudaError_t qk_launch_quantize_q8_0(const float *x, uint64_t n, uint8_t *out, cudaStream_t s) {
  uint64_t nblocks = n / 32;
  if (nblocks == 0) return cudaSuccess;
  qk_quantize_q8_0_kernel<<<(unsigned)((nblocks + 3) / 4), 128, 0, s>>>(x, nblocks, out);
  return cudaGetLastError();
}
