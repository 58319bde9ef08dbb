// Mixture-of-experts FFN around the quantized matmuls (crates/oxillama-arch/src/common/moe.rs:184-258):
// routing, the per-expert token lists, and the element-wise steps between the three
// matmuls of an expert (moe.rs:75-126).  The matmuls themselves are the ordinary
// dequant-matmul kernels: for decode-sized calls run once per expert on the tokens routed to
// it, for batches as one grouped launch per projection over all local experts (the _grouped
// kernels below work on arrays that reserve `cap` rows per expert, live below counts[e]).
#include <cfloat>

#include "qk_kernels.h"

namespace {

// One thread per token: softmax over all experts, the top_k largest in descending order
// (equal values keep ascending expert order, as a stable sort would), weights
// renormalised by the selected sum (moe.rs:200-248).
__global__ void __launch_bounds__(128)
    qk_moe_route_kernel(const float *__restrict__ logits, uint32_t tokens, uint32_t n_exp,
                        uint32_t top_k, int *__restrict__ ids, float *__restrict__ wts) {
  const uint32_t t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= tokens) return;
  const float *l = logits + (uint64_t)t * n_exp;
  const uint32_t ek = top_k < n_exp ? top_k : n_exp;
  float mx = -INFINITY;
  for (uint32_t i = 0; i < n_exp; i++) mx = fmaxf(mx, l[i]);
  float es = 0.f;
  for (uint32_t i = 0; i < n_exp; i++) es = __fadd_rn(es, expf(__fsub_rn(l[i], mx)));
  auto prob = [&](uint32_t i) {
    const float e = expf(__fsub_rn(l[i], mx));
    return es > 0.f ? __fdiv_rn(e, es) : __fdiv_rn(1.f, (float)n_exp);
  };
  float ssum = 0.f;
  for (uint32_t k = 0; k < ek; k++) {  // k-th largest not yet taken; ties to the lower index
    float best = -1.f;
    uint32_t bi = 0;
    for (uint32_t i = 0; i < n_exp; i++) {
      bool taken = false;
      for (uint32_t j = 0; j < k; j++) taken |= ids[(uint64_t)t * top_k + j] == (int)i;
      const float p = prob(i);
      if (!taken && p > best) best = p, bi = i;
    }
    ids[(uint64_t)t * top_k + k] = (int)bi;
    wts[(uint64_t)t * top_k + k] = best;
    ssum = __fadd_rn(ssum, best);
  }
  for (uint32_t k = 0; k < ek; k++) {
    float &w = wts[(uint64_t)t * top_k + k];
    w = ssum > 1e-9f ? __fdiv_rn(w, ssum) : __fdiv_rn(1.f, (float)ek);
  }
  for (uint32_t k = ek; k < top_k; k++) ids[(uint64_t)t * top_k + k] = -1, wts[(uint64_t)t * top_k + k] = 0.f;
}

// One warp per local expert: the (token, slot) pairs routed to it, in token order.
__global__ void __launch_bounds__(32)
    qk_moe_lists_kernel(const int *__restrict__ ids, uint32_t tokens, uint32_t top_k,
                        uint32_t expert_begin, int *__restrict__ counts, int *__restrict__ lists,
                        int *__restrict__ pos) {
  const uint32_t e = blockIdx.x, lane = threadIdx.x;
  const int want = (int)(expert_begin + e);
  const uint64_t n = (uint64_t)tokens * top_k;
  uint32_t count = 0;
  for (uint64_t base = 0; base < n; base += 32) {
    const uint64_t i = base + lane;
    const bool hit = i < n && ids[i] == want;
    const uint32_t mask = __ballot_sync(0xffffffffu, hit);
    if (hit) {
      const uint32_t p = count + __popc(mask & ((1u << lane) - 1u));
      lists[(uint64_t)e * n + p] = (int)i;
      if (pos) pos[i] = (int)p;  // where (token, slot) i sits in its expert's list
    }
    count += __popc(mask);
  }
  if (lane == 0) counts[e] = (int)count;
}

__global__ void __launch_bounds__(256)
    qk_moe_gather_kernel(const float *__restrict__ x, const int *__restrict__ list, uint32_t n,
                         uint32_t top_k, uint32_t hidden, float *__restrict__ xe) {
  const uint32_t i = blockIdx.x;
  if (i >= n) return;
  const float *src = x + (uint64_t)(list[i] / (int)top_k) * hidden;
  for (uint32_t c = threadIdx.x; c < hidden; c += blockDim.x) xe[(uint64_t)i * hidden + c] = src[c];
}

// u <- silu(g) * u  (moe.rs:96-112: g * sigmoid(g), then times up)
__global__ void __launch_bounds__(256)
    qk_moe_silu_mul_kernel(const float *__restrict__ g, float *__restrict__ u, uint64_t n) {
  for (uint64_t i = blockIdx.x * 256ull + threadIdx.x; i < n; i += (uint64_t)gridDim.x * 256) {
    const float v = g[i];
    const float sig = __fdiv_rn(1.f, __fadd_rn(1.f, expf(-v)));
    u[i] = __fmul_rn(u[i], __fmul_rn(v, sig));
  }
}

// g <- silu(g) * u: swiglu_inplace (crates/oxillama-arch/src/common/swiglu.rs:15-21), each step rounded
__global__ void __launch_bounds__(256)
    qk_swiglu_kernel(float *__restrict__ g, const float *__restrict__ u, uint64_t n) {
  for (uint64_t i = blockIdx.x * 256ull + threadIdx.x; i < n; i += (uint64_t)gridDim.x * 256) {
    const float v = g[i];
    const float sig = __fdiv_rn(1.f, __fadd_rn(1.f, expf(-v)));
    g[i] = __fmul_rn(__fmul_rn(v, sig), u[i]);
  }
}

// y[token] += w * o[i]; a token occurs at most once in one expert's list.
__global__ void __launch_bounds__(256)
    qk_moe_scatter_kernel(const float *__restrict__ o, const int *__restrict__ list,
                          const float *__restrict__ wts, uint32_t n, uint32_t top_k, uint32_t hidden,
                          float *__restrict__ y) {
  const uint32_t i = blockIdx.x;
  if (i >= n) return;
  const int slot = list[i];
  const float w = wts[slot];
  float *dst = y + (uint64_t)(slot / (int)top_k) * hidden;
  for (uint32_t c = threadIdx.x; c < hidden; c += blockDim.x)
    dst[c] = __fadd_rn(dst[c], __fmul_rn(w, o[(uint64_t)i * hidden + c]));
}


// Grouped form of the element-wise step: u[(e, i)] <- silu(g[(e, i)]) * u[(e, i)] for the live rows
// i < counts[e] of every local expert; rows are `cap` apart per expert (moe.rs:96-112).
__global__ void __launch_bounds__(256)
    qk_moe_silu_mul_grouped_kernel(const float *__restrict__ g, float *__restrict__ u, const int *__restrict__ counts,
                                   uint32_t cap, uint32_t inter) {
  const uint32_t e = blockIdx.y, i = blockIdx.x;
  if ((int)i >= counts[e]) return;
  const uint64_t base = ((uint64_t)e * cap + i) * inter;
  for (uint32_t c = threadIdx.x; c < inter; c += 256) {
    const float v = g[base + c];
    const float sig = __fdiv_rn(1.f, __fadd_rn(1.f, expf(-v)));
    u[base + c] = __fmul_rn(u[base + c], __fmul_rn(v, sig));
  }
}

// y[token] = sum over the token's slots, in slot order, of w[slot] * o[(expert, position)] for
// the slots whose expert is local (moe.rs:232-255 accumulates in that order); a token none of
// whose experts is local gets zeros.
__global__ void __launch_bounds__(256)
    qk_moe_combine_kernel(const float *__restrict__ o, const int *__restrict__ ids, const int *__restrict__ pos,
                          const float *__restrict__ wts, uint32_t top_k, uint32_t expert_begin, uint32_t n_local,
                          uint32_t cap, uint32_t hidden, float *__restrict__ y) {
  const uint32_t t = blockIdx.x;
  for (uint32_t c = threadIdx.x; c < hidden; c += 256) {
    float acc = 0.f;
    for (uint32_t k = 0; k < top_k; k++) {
      const int id = ids[(uint64_t)t * top_k + k];
      if (id < (int)expert_begin || id >= (int)(expert_begin + n_local)) continue;
      const uint64_t row = (uint64_t)(id - (int)expert_begin) * cap + (uint32_t)pos[(uint64_t)t * top_k + k];
      acc = __fadd_rn(acc, __fmul_rn(wts[(uint64_t)t * top_k + k], o[row * hidden + c]));
    }
    y[(uint64_t)t * hidden + c] = acc;
  }
}

// out[i][:] = x[idx[i]][:]: the rows a rank sends to another rank, in send order.
__global__ void __launch_bounds__(256)
    qk_moe_take_rows_kernel(const float *__restrict__ x, const int *__restrict__ idx, uint32_t width,
                            float *__restrict__ out) {
  const uint64_t src = (uint64_t)(uint32_t)idx[blockIdx.x] * width, dst = (uint64_t)blockIdx.x * width;
  for (uint32_t c = threadIdx.x; c < width; c += 256) out[dst + c] = x[src + c];
}

// y[t][:] = +0 + src[idx[t][0]] + src[idx[t][1]] + ... in that order, entries below zero skipped:
// the partial outputs that came back for token t, in the order of the ranks that made them.
__global__ void __launch_bounds__(256)
    qk_moe_sum_rows_kernel(const float *__restrict__ src, const int *__restrict__ idx, uint32_t per_row,
                           uint32_t width, float *__restrict__ y) {
  const uint32_t t = blockIdx.x;
  for (uint32_t c = threadIdx.x; c < width; c += 256) {
    float acc = 0.f;
    for (uint32_t j = 0; j < per_row; j++) {
      const int r = idx[(uint64_t)t * per_row + j];
      if (r >= 0) acc = __fadd_rn(acc, src[(uint64_t)r * width + c]);
    }
    y[(uint64_t)t * width + c] = acc;
  }
}

}  // namespace

cudaError_t qk_launch_moe_route(const float *logits, uint32_t tokens, uint32_t n_exp, uint32_t top_k,
                                int *ids, float *wts, cudaStream_t s) {
  if (tokens == 0) return cudaSuccess;
  qk_moe_route_kernel<<<(tokens + 127) / 128, 128, 0, s>>>(logits, tokens, n_exp, top_k, ids, wts);
  return cudaGetLastError();
}
cudaError_t qk_launch_moe_lists(const int *ids, uint32_t tokens, uint32_t top_k, uint32_t expert_begin,
                                uint32_t n_local, int *counts, int *lists, int *pos, cudaStream_t s) {
  if (n_local == 0) return cudaSuccess;
  qk_moe_lists_kernel<<<n_local, 32, 0, s>>>(ids, tokens, top_k, expert_begin, counts, lists, pos);
  return cudaGetLastError();
}
cudaError_t qk_launch_moe_silu_mul_grouped(const float *g, float *u, const int *counts, uint32_t n_local,
                                           uint32_t max_rows, uint32_t cap, uint32_t inter, cudaStream_t s) {
  if (n_local == 0 || max_rows == 0 || inter == 0) return cudaSuccess;
  qk_moe_silu_mul_grouped_kernel<<<dim3(max_rows, n_local), 256, 0, s>>>(g, u, counts, cap, inter);
  return cudaGetLastError();
}
cudaError_t qk_launch_moe_combine(const float *o, const int *ids, const int *pos, const float *wts, uint32_t tokens,
                                  uint32_t top_k, uint32_t expert_begin, uint32_t n_local, uint32_t cap,
                                  uint32_t hidden, float *y, cudaStream_t s) {
  if (tokens == 0 || hidden == 0) return cudaSuccess;
  qk_moe_combine_kernel<<<tokens, 256, 0, s>>>(o, ids, pos, wts, top_k, expert_begin, n_local, cap, hidden, y);
  return cudaGetLastError();
}
cudaError_t qk_launch_moe_gather(const float *x, const int *list, uint32_t n, uint32_t top_k,
                                 uint32_t hidden, float *xe, cudaStream_t s) {
  if (n == 0) return cudaSuccess;
  qk_moe_gather_kernel<<<n, 256, 0, s>>>(x, list, n, top_k, hidden, xe);
  return cudaGetLastError();
}
cudaError_t qk_launch_moe_silu_mul(const float *g, float *u, uint64_t n, cudaStream_t s) {
  if (n == 0) return cudaSuccess;
  const uint64_t blocks = (n + 255) / 256;
  qk_moe_silu_mul_kernel<<<(unsigned)(blocks > 148 * 16 ? 148 * 16 : blocks), 256, 0, s>>>(g, u, n);
  return cudaGetLastError();
}
cudaError_t qk_launch_swiglu(float *g, const float *u, uint64_t n, cudaStream_t s) {
  if (n == 0) return cudaSuccess;
  const uint64_t blocks = (n + 255) / 256;
  qk_swiglu_kernel<<<(unsigned)(blocks > 148 * 16 ? 148 * 16 : blocks), 256, 0, s>>>(g, u, n);
  return cudaGetLastError();
}

cudaError_t qk_launch_moe_scatter(const float *o, const int *list, const float *wts, uint32_t n,
                                  uint32_t top_k, uint32_t hidden, float *y, cudaStream_t s) {
  if (n == 0) return cudaSuccess;
  qk_moe_scatter_kernel<<<n, 256, 0, s>>>(o, list, wts, n, top_k, hidden, y);
  return cudaGetLastError();
}

cudaError_t qk_launch_moe_take_rows(const float *x, const int *idx, uint32_t n, uint32_t width, float *out,
                                    cudaStream_t s) {
  if (n == 0 || width == 0) return cudaSuccess;
  qk_moe_take_rows_kernel<<<n, 256, 0, s>>>(x, idx, width, out);
  return cudaGetLastError();
}
cudaError_t qk_launch_moe_sum_rows(const float *src, const int *idx, uint32_t tokens, uint32_t per_row,
                                   uint32_t width, float *y, cudaStream_t s) {
  if (tokens == 0 || width == 0) return cudaSuccess;
  qk_moe_sum_rows_kernel<<<tokens, 256, 0, s>>>(src, idx, per_row, width, y);
  return cudaGetLastError();
}
