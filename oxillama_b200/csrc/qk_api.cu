// C ABI of the backend (see include/qk_cuda.h): argument checking in the
// reference's order, the context (stream, scratch, weight cache), and the
// choice of kernel for each shape.  Nothing here computes on the CPU: a call
// that cannot reach the GPU returns QK_CUDA_ERROR.
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <mutex>
#include <string>
#include <tuple>

#include <vector>

#include "qk_internal.h"

#define CK(ctx, call)                                                                     \
  do {                                                                                    \
    cudaError_t e__ = (call);                                                             \
    if (e__ != cudaSuccess) {                                                             \
      (ctx)->err = std::string(#call) + ": " + cudaGetErrorString(e__);                   \
      return QK_CUDA_ERROR;                                                               \
    }                                                                                     \
  } while (0)

static bool type_ok(int t) {
  return t == QK_TYPE_Q4_0 || t == QK_TYPE_Q8_0 || t == QK_TYPE_Q4_K || t == QK_TYPE_Q5_K || t == QK_TYPE_Q6_K ||
         t == QK_TYPE_IQ4_XS || t == QK_TYPE_Q2_K || t == QK_TYPE_Q3_K || t == QK_TYPE_Q8_K;
}

extern "C" size_t qk_block_size(int type) {
  switch (type) {
    case QK_TYPE_Q4_0:
    case QK_TYPE_Q8_0:
      return 32;
    case QK_TYPE_Q2_K:
    case QK_TYPE_Q3_K:
    case QK_TYPE_Q4_K:
    case QK_TYPE_Q5_K:
    case QK_TYPE_Q6_K:
    case QK_TYPE_Q8_K:
    case QK_TYPE_IQ4_XS:
      return 256;
    default:
      return 0;
  }
}

extern "C" size_t qk_block_bytes(int type) {
  switch (type) {
    case QK_TYPE_Q4_0:
      return 18;
    case QK_TYPE_Q8_0:
      return 34;
    case QK_TYPE_Q4_K:
      return 144;
    case QK_TYPE_Q5_K:
      return 176;
    case QK_TYPE_Q2_K:
      return 84;
    case QK_TYPE_Q3_K:
      return 110;
    case QK_TYPE_Q8_K:
      return 292;
    case QK_TYPE_Q6_K:
      return 210;
    case QK_TYPE_IQ4_XS:
      return 136;
    default:
      return 0;
  }
}

extern "C" const char *qk_name(int type) {
  switch (type) {
    case QK_TYPE_Q4_0:
      return "Q4_0";
    case QK_TYPE_Q8_0:
      return "Q8_0";
    case QK_TYPE_Q4_K:
      return "Q4_K";
    case QK_TYPE_Q5_K:
      return "Q5_K";
    case QK_TYPE_Q2_K:
      return "Q2_K";
    case QK_TYPE_Q3_K:
      return "Q3_K";
    case QK_TYPE_Q8_K:
      return "Q8_K";
    case QK_TYPE_Q6_K:
      return "Q6_K";
    case QK_TYPE_IQ4_XS:
      return "IQ4_XS";
    default:
      return nullptr;
  }
}

extern "C" int qk_init(int device, qk_ctx **out) {
  if (!out) return QK_INVALID_ARGUMENT;
  *out = nullptr;
  int n = 0;
  if (cudaGetDeviceCount(&n) != cudaSuccess || device < 0 || device >= n) return QK_CUDA_ERROR;
  if (cudaSetDevice(device) != cudaSuccess) return QK_CUDA_ERROR;
  qk_ctx *c = new qk_ctx();
  c->device = device;
  cudaDeviceProp prop;
  if (cudaGetDeviceProperties(&prop, device) != cudaSuccess || prop.major != 10) {
    delete c;  // the kernels are sm_100a-only
    return QK_CUDA_ERROR;
  }
  c->sm_count = prop.multiProcessorCount;
  unsigned *sh = nullptr;
  if (cudaStreamCreateWithFlags(&c->stream, cudaStreamNonBlocking) != cudaSuccess ||
      cudaHostAlloc((void **)&sh, sizeof(unsigned), cudaHostAllocMapped | cudaHostAllocPortable) != cudaSuccess ||
      cudaHostGetDevicePointer((void **)&c->status_dev, sh, 0) != cudaSuccess ||
      cudaMalloc(&c->scratch, (size_t)1 << 20) != cudaSuccess) {
    if (sh) cudaFreeHost(sh);
    delete c;
    return QK_CUDA_ERROR;
  }
  *sh = 0;
  c->status_host = sh;
  c->scratch_cap = (size_t)1 << 20;
  const char *fs = qk_knob("QK_FORCE_SIMPLE");
  c->force_simple = fs && fs[0] == '1';
  *out = c;
  return QK_OK;
}

static void free_weights(qk_weights *h) {
  if (!h) return;
  if (h->dev) cudaFree(h->dev);
  delete h;
}

extern "C" int qk_shutdown(qk_ctx *c) {
  if (!c) return QK_INVALID_ARGUMENT;
  cudaSetDevice(c->device);
  cudaStreamSynchronize(c->stream);
  for (auto &kv : c->cache) free_weights(kv.second);
  if (c->sa) cudaFree(c->sa);
  if (c->sb) cudaFree(c->sb);
  cudaFreeHost((void *)c->status_host);
  if (c->scratch) cudaFree(c->scratch);
  if (c->moe) cudaFree(c->moe);
  if (c->ffn) cudaFree(c->ffn);
  cudaStreamDestroy(c->stream);
  delete c;
  return QK_OK;
}

extern "C" int qk_last_error(qk_ctx *c, char *buf, size_t buf_len) {
  if (!c || !buf || buf_len == 0) return QK_INVALID_ARGUMENT;
  snprintf(buf, buf_len, "%s", c->err.c_str());
  return QK_OK;
}

static int grow(qk_ctx *c, void **p, size_t *cap, size_t need) {
  if (need <= *cap) return QK_OK;
  if (*p) {
    CK(c, cudaStreamSynchronize(c->stream));
    cudaFree(*p);
    *p = nullptr;
    *cap = 0;
  }
  size_t want = need + need / 4 + 256;
  CK(c, cudaMalloc(p, want));
  *cap = want;
  return QK_OK;
}

static size_t need_bytes(int type, size_t n_rows, size_t n_cols) {
  size_t bs = qk_block_size(type), bb = qk_block_bytes(type);
  return n_rows * ((n_cols + bs - 1) / bs) * bb;
}

// ------------------------------------------------------------ upload
static int upload_impl(qk_ctx *c, int type, const uint8_t *w, size_t n_cols, size_t row_begin,
                       size_t row_end, qk_weights **out) {
  size_t rows = row_end - row_begin;
  qk_weights *h = new qk_weights();
  h->device = c->device;
  h->dev = nullptr;
  if (!qk_make_layout(type, rows, n_cols, &h->L)) {
    delete h;
    return QK_UNSUPPORTED_TYPE;
  }
  h->algo_bytes = need_bytes(type, rows, n_cols);
  size_t row_bytes = (size_t)h->L.nb * h->L.bb;
  size_t tiled = h->L.total_bytes ? h->L.total_bytes : 16;
  cudaError_t e = cudaMalloc(&h->dev, tiled);
  if (e != cudaSuccess) {
    c->err = std::string("cudaMalloc(weights): ") + cudaGetErrorString(e);
    delete h;
    return QK_CUDA_ERROR;
  }
  uint8_t *raw = nullptr;
  int st = QK_OK;
  do {
    if ((e = cudaMemsetAsync(h->dev, 0, tiled, c->stream)) != cudaSuccess) break;
    if (h->algo_bytes == 0) break;
    if ((e = cudaMalloc(&raw, h->algo_bytes)) != cudaSuccess) break;
    if ((e = cudaMemcpyAsync(raw, w + row_begin * row_bytes, h->algo_bytes, cudaMemcpyHostToDevice,
                             c->stream)) != cudaSuccess)
      break;
    if ((e = qk_launch_repack(h->L, raw, h->dev, c->stream)) != cudaSuccess) break;
  } while (0);
  if (e == cudaSuccess) e = cudaStreamSynchronize(c->stream);
  if (raw) cudaFree(raw);
  if (e != cudaSuccess) {
    c->err = std::string("weights upload: ") + cudaGetErrorString(e);
    free_weights(h);
    st = QK_CUDA_ERROR;
  } else {
    *out = h;
  }
  return st;
}

extern "C" int qk_weights_upload(qk_ctx *c, int type, const uint8_t *w, size_t w_len, size_t n_rows,
                                 size_t n_cols, size_t row_begin, size_t row_end,
                                 qk_weights **out) {
  if (!c || !out) return QK_INVALID_ARGUMENT;
  *out = nullptr;
  if (!type_ok(type)) return QK_UNSUPPORTED_TYPE;
  if (row_begin > row_end || row_end > n_rows) return QK_INVALID_ARGUMENT;
  if (n_rows >= (1ull << 31) || n_cols >= (1ull << 31)) return QK_INVALID_ARGUMENT;
  if (w_len < need_bytes(type, n_rows, n_cols)) return QK_BUFFER_TOO_SMALL;
  if (!w && need_bytes(type, n_rows, n_cols) > 0) return QK_INVALID_ARGUMENT;
  std::lock_guard<std::mutex> g(c->mu);
  CK(c, cudaSetDevice(c->device));
  return upload_impl(c, type, w, n_cols, row_begin, row_end, out);
}

extern "C" int qk_weights_free(qk_ctx *c, qk_weights *h) {
  if (!c || !h) return QK_INVALID_ARGUMENT;
  std::lock_guard<std::mutex> g(c->mu);
  cudaSetDevice(c->device);
  free_weights(h);
  return QK_OK;
}

extern "C" int qk_weights_info(const qk_weights *h, int *type, size_t *rows, size_t *cols,
                               size_t *bytes) {
  if (!h) return QK_INVALID_ARGUMENT;
  if (type) *type = h->L.type;
  if (rows) *rows = h->L.rows;
  if (cols) *cols = h->L.cols;
  if (bytes) *bytes = h->algo_bytes;
  return QK_OK;
}

// Cheap content fingerprint of a host weight buffer: every byte when it is small, else its
// first and last 256 bytes and 64 evenly spread 8-byte samples (about 70 cache lines: the
// check runs on every host-pointer call, and the 2048 samples it once took were a dozen
// microseconds of cache misses per call on weights that do not fit the host's caches).  It
// guards the pointer-keyed cache against a freed buffer's address being reused for other
// weights; it does not detect a few bytes edited in place (qk_weights_cache_evict).
static uint64_t fingerprint(const uint8_t *w, size_t n) {
  uint64_t h = 1469598103934665603ull ^ n;
  auto mix = [&](uint64_t v) { h = (h ^ v) * 1099511628211ull; h ^= h >> 29; };
  if (n <= 4096) {
    size_t i = 0;
    for (; i + 8 <= n; i += 8) { uint64_t v; memcpy(&v, w + i, 8); mix(v); }
    for (; i < n; i++) mix(w[i]);
    return h;
  }
  for (size_t i = 0; i < 256; i += 8) { uint64_t v; memcpy(&v, w + i, 8); mix(v); }
  for (size_t i = n - 256; i + 8 <= n; i += 8) { uint64_t v; memcpy(&v, w + i, 8); mix(v); }
  const size_t step = (n - 8) / 64;
  for (size_t k = 0; k < 64; k++) { uint64_t v; memcpy(&v, w + k * step, 8); mix(v); }
  return h;
}

// Cached device copy for the host-pointer entry points, keyed by (pointer, length, type,
// shape); a hit whose fingerprint no longer matches is uploaded again.
static int cached(qk_ctx *c, int type, const uint8_t *w, size_t w_len, size_t n_rows, size_t n_cols,
                  qk_weights **out) {
  const size_t need = need_bytes(type, n_rows, n_cols);
  const uint64_t fp = fingerprint(w, need);
  qk_ctx::Key k(w, w_len, type, n_rows, n_cols, 0);
  auto it = c->cache.find(k);
  if (it != c->cache.end()) {
    if (it->second->fp == fp) {
      *out = it->second;
      return QK_OK;
    }
    CK(c, cudaStreamSynchronize(c->stream));  // other contents behind the same address: drop the stale copy
    c->cache_bytes -= it->second->algo_bytes;
    free_weights(it->second);
    c->cache.erase(it);
  }
  if (c->cache_bytes + need > c->cache_cap) {  // simplest policy: start over
    CK(c, cudaStreamSynchronize(c->stream));
    for (auto &kv : c->cache) free_weights(kv.second);
    c->cache.clear();
    c->cache_bytes = 0;
  }
  int st = upload_impl(c, type, w, n_cols, 0, n_rows, out);
  if (st == QK_OK) {
    (*out)->fp = fp;
    c->cache[k] = *out;
    c->cache_bytes += need;
  }
  return st;
}

extern "C" int qk_weights_cache_evict(qk_ctx *c, const uint8_t *w) {
  if (!c) return QK_INVALID_ARGUMENT;
  std::lock_guard<std::mutex> g(c->mu);
  cudaSetDevice(c->device);
  cudaStreamSynchronize(c->stream);
  for (auto it = c->cache.begin(); it != c->cache.end();) {
    if (!w || std::get<0>(it->first) == (const void *)w) {
      c->cache_bytes -= it->second->algo_bytes;
      free_weights(it->second);
      it = c->cache.erase(it);
    } else {
      ++it;
    }
  }
  return QK_OK;
}

// ------------------------------------------------------------ device entry points
static int gemm_dispatch(qk_ctx *c, const qk_weights *h, const float *x, float *y, size_t m,
                         size_t ldy, cudaStream_t s) {
  if (h->L.rows == 0 || m == 0) return QK_OK;
  if (h->L.cols == 0) {  // empty dot products
    CK(c, cudaMemset2DAsync(y, ldy * sizeof(float), 0, h->L.rows * sizeof(float), m, s));
    return QK_OK;
  }
  auto ensure_scratch = [&](size_t need) -> int {
    if (need <= c->scratch_cap) return QK_OK;
    CK(c, cudaDeviceSynchronize());
    cudaFree(c->scratch);
    c->scratch = nullptr, c->scratch_cap = 0;
    CK(c, cudaMalloc(&c->scratch, need * 2));
    c->scratch_cap = need * 2;
    return QK_OK;
  };
  if (!c->force_simple && m <= QK_GEMV_MAX_M && qk_gemv_fast_supported(h->L, (uint32_t)m)) {
    int st = ensure_scratch(qk_gemv_fast_scratch_bytes(h->L, (uint32_t)m));
    if (st) return st;
    CK(c, qk_launch_gemv_fast(h->L, h->dev, x, y, (uint32_t)m, ldy, c->status_dev, c->scratch,
                              c->sm_count, s));
    return QK_OK;
  }
  // 5 .. 16 rows of a tall Q4_K matrix: the streaming fp16-MMA kernel (measured faster than
  // the tcgen05 kernel from eight 8-row chunks per SM up; below that it is not)
  if (!c->force_simple && !qk_knob("QK_NO_SB") && qk_gemm_sb_preferred(h->L, (uint32_t)m, c->sm_count)) {
    int st = ensure_scratch(qk_gemm_sb_scratch_bytes(h->L, (uint32_t)m));
    if (st) return st;
    CK(c, qk_launch_gemm_sb(h->L, h->dev, x, y, (uint32_t)m, ldy, c->status_dev, c->scratch, c->sm_count, s));
    return QK_OK;
  }
  // The tensor-core path rounds its operands to fp16; batches the decode kernels take keep
  // f32-grade activations.  Decode-sized calls the decode kernels cannot take (K not a
  // multiple of 256, activations too long for shared memory) go to the generic kernel below.
  // (Two to four rows of a format whose decode kernel stops below four rows for register
  // reasons also go to the tensor cores.)
  const bool tc_small = m <= QK_GEMV_MAX_M && m > 1 && qk_gemv_fast_supported(h->L, 1);
  if (!c->force_simple && (m > QK_GEMV_MAX_M || tc_small) && m < (1u << 30) &&
      qk_gemm_tc_supported(h->L, (uint32_t)m)) {
    int st = ensure_scratch(qk_gemm_tc_scratch_bytes(h->L, (uint32_t)m));
    if (st) return st;
    CK(c, qk_launch_gemm_tc(h->L, h->dev, x, y, (uint32_t)m, ldy, c->status_dev, c->scratch,
                            c->sm_count, s));
    return QK_OK;
  }
  CK(c, qk_launch_gemm_simple(h->L, h->dev, x, y, (uint32_t)m, ldy, s));
  return QK_OK;
}

extern "C" int qk_gemv_dev(qk_ctx *c, const qk_weights *h, const float *x_dev, float *y_dev,
                           void *stream) {
  if (!c || !h || !x_dev || !y_dev) return QK_INVALID_ARGUMENT;
  if (h->device != c->device) return QK_INVALID_ARGUMENT;
  return gemm_dispatch(c, h, x_dev, y_dev, 1, h->L.rows, (cudaStream_t)stream);
}

extern "C" int qk_gemm_dev(qk_ctx *c, const qk_weights *h, const float *x_dev, float *y_dev,
                           size_t m, size_t ldy, void *stream) {
  if (!c || !h || !x_dev || !y_dev) return QK_INVALID_ARGUMENT;
  if (h->device != c->device) return QK_INVALID_ARGUMENT;
  if (ldy < h->L.rows) return QK_DIMENSION_MISMATCH;
  return gemm_dispatch(c, h, x_dev, y_dev, m, ldy, (cudaStream_t)stream);
}

extern "C" int qk_moe_route_dev(qk_ctx *c, const float *logits_dev, size_t tokens, size_t n_exp,
                                size_t top_k, int *ids_dev, float *wts_dev, void *stream) {
  if (!c || !logits_dev || !ids_dev || !wts_dev) return QK_INVALID_ARGUMENT;
  if (n_exp == 0 || top_k == 0 || n_exp > 4096) return QK_INVALID_ARGUMENT;
  CK(c, qk_launch_moe_route(logits_dev, (uint32_t)tokens, (uint32_t)n_exp, (uint32_t)top_k, ids_dev, wts_dev,
                            (cudaStream_t)stream));
  return QK_OK;
}

extern "C" int qk_moe_take_rows_dev(qk_ctx *c, const float *x_dev, const int *idx_dev, size_t n, size_t width,
                                    float *out_dev, void *stream) {
  if (!c) return QK_INVALID_ARGUMENT;
  if (n == 0 || width == 0) return QK_OK;
  if (!x_dev || !idx_dev || !out_dev || n > 0x7fffffffu || width > 0x7fffffffu) return QK_INVALID_ARGUMENT;
  CK(c, qk_launch_moe_take_rows(x_dev, idx_dev, (uint32_t)n, (uint32_t)width, out_dev, (cudaStream_t)stream));
  return QK_OK;
}

extern "C" int qk_moe_sum_rows_dev(qk_ctx *c, const float *src_dev, const int *idx_dev, size_t tokens,
                                   size_t per_row, size_t width, float *y_dev, void *stream) {
  if (!c) return QK_INVALID_ARGUMENT;
  if (tokens == 0 || width == 0) return QK_OK;
  if (!y_dev || (per_row && (!src_dev || !idx_dev)) || tokens > 0x7fffffffu || per_row > 0x7fffffffu ||
      width > 0x7fffffffu)
    return QK_INVALID_ARGUMENT;
  CK(c, qk_launch_moe_sum_rows(src_dev, idx_dev, (uint32_t)tokens, (uint32_t)per_row, (uint32_t)width, y_dev,
                               (cudaStream_t)stream));
  return QK_OK;
}

extern "C" int qk_moe_ffn_dev(qk_ctx *c, const qk_weights *const *gate, const qk_weights *const *up,
                              const qk_weights *const *down, size_t n_local, size_t expert_begin,
                              size_t n_exp, const float *logits_dev, const float *x_dev, float *y_dev,
                              size_t tokens, size_t top_k, void *stream) {
  if (!c || !logits_dev || !x_dev || !y_dev || (n_local && (!gate || !up || !down))) return QK_INVALID_ARGUMENT;
  if (n_exp == 0 || top_k == 0 || n_exp > 4096 || expert_begin + n_local > n_exp) return QK_INVALID_ARGUMENT;
  cudaStream_t s = (cudaStream_t)stream;
  size_t hidden = 0, inter = 0;
  for (size_t e = 0; e < n_local; e++) {
    if (!gate[e] || !up[e] || !down[e]) return QK_INVALID_ARGUMENT;
    if (gate[e]->device != c->device || up[e]->device != c->device || down[e]->device != c->device)
      return QK_INVALID_ARGUMENT;
    if (e == 0) hidden = gate[e]->L.cols, inter = gate[e]->L.rows;
    if (gate[e]->L.cols != hidden || gate[e]->L.rows != inter || up[e]->L.cols != hidden ||
        up[e]->L.rows != inter || down[e]->L.cols != inter || down[e]->L.rows != hidden)
      return QK_DIMENSION_MISMATCH;
  }
  if (n_local == 0 || tokens == 0) return QK_OK;
  const size_t slots = tokens * top_k;
  auto al = [](size_t v) { return (v + 255) & ~(size_t)255; };
  auto grow_moe = [&](size_t need) -> int {
    if (need > c->moe_cap) {
      CK(c, cudaDeviceSynchronize());
      if (c->moe) cudaFree(c->moe);
      c->moe = nullptr, c->moe_cap = 0;
      CK(c, cudaMalloc(&c->moe, need));
      c->moe_cap = need;
    }
    return QK_OK;
  };

  // Grouped route: batches of more than a handful of tokens, experts of one format the
  // tensor-core kernel takes.  Every projection is one conversion launch (which also gathers
  // the routed rows) and one matmul launch over all local experts; the per-expert token
  // counts stay on the device and nothing is read back, so the whole call is a fixed
  // sequence of launches with no host synchronisation.  An expert may receive every token:
  // the activation arrays reserve `cap` rows per expert, of which only the live ones are
  // touched.
  bool grouped = !c->force_simple && !qk_knob("QK_NO_MOE_GROUPED") && tokens > 16 && n_local <= QK_MAX_GROUPS &&
                 hidden > 0 && inter > 0;
  for (size_t e = 0; e < n_local && grouped; e++)
    grouped = gate[e]->L.type == gate[0]->L.type && up[e]->L.type == gate[0]->L.type &&
              down[e]->L.type == down[0]->L.type && qk_gemm_tc_supported(gate[e]->L, 1) &&
              qk_gemm_tc_supported(down[e]->L, 1);
  if (grouped) {
    const size_t cap = qk_gemm_tc_group_cap((uint32_t)tokens), rows = n_local * cap;
    const size_t o_ids = 0, o_wts = o_ids + al(slots * 4), o_cnt = o_wts + al(slots * 4);
    const size_t o_lists = o_cnt + al(n_local * 4), o_pos = o_lists + al(n_local * slots * 4);
    const size_t o_g = o_pos + al(slots * 4), o_u = o_g + rows * inter * 4;  // u directly behind g
    const size_t o_o = al(o_u + rows * inter * 4), need = o_o + al(rows * hidden * 4);
    int st = grow_moe(need);
    if (st) return st;
    unsigned char *base = (unsigned char *)c->moe;
    int *ids = (int *)(base + o_ids), *cnt = (int *)(base + o_cnt), *lists = (int *)(base + o_lists);
    int *pos = (int *)(base + o_pos);
    float *wts = (float *)(base + o_wts), *g = (float *)(base + o_g), *u = (float *)(base + o_u);
    float *o = (float *)(base + o_o);
    size_t sneed = qk_gemm_tc_grouped_scratch_bytes(gate[0]->L, (uint32_t)n_local, (uint32_t)tokens);
    const size_t sdown = qk_gemm_tc_grouped_scratch_bytes(down[0]->L, (uint32_t)n_local, (uint32_t)tokens);
    if (sdown > sneed) sneed = sdown;
    if (sneed > c->scratch_cap) {
      CK(c, cudaDeviceSynchronize());
      cudaFree(c->scratch);
      c->scratch = nullptr, c->scratch_cap = 0;
      CK(c, cudaMalloc(&c->scratch, sneed));
      c->scratch_cap = sneed;
    }
    const uint8_t *wgu[QK_MAX_GROUPS], *wd[QK_MAX_GROUPS];
    const bool one_launch = 2 * n_local <= QK_MAX_GROUPS;  // gate and up as 2 n groups over n activation groups
    for (size_t e = 0; e < n_local; e++) wd[e] = down[e]->dev;
    CK(c, qk_launch_moe_route(logits_dev, (uint32_t)tokens, (uint32_t)n_exp, (uint32_t)top_k, ids, wts, s));
    CK(c, qk_launch_moe_lists(ids, (uint32_t)tokens, (uint32_t)top_k, (uint32_t)expert_begin, (uint32_t)n_local,
                              cnt, lists, pos, s));
    if (one_launch) {
      // u directly behind g: groups 0 .. n - 1 write g, groups n .. 2 n - 1 write u
      u = g + rows * inter;
      for (size_t e = 0; e < n_local; e++) wgu[e] = gate[e]->dev, wgu[n_local + e] = up[e]->dev;
      CK(c, qk_launch_gemm_tc_grouped(gate[0]->L, wgu, (uint32_t)(2 * n_local), (uint32_t)n_local, cnt,
                                      (uint32_t)tokens, x_dev, lists, (uint32_t)slots, (uint32_t)top_k, g, inter,
                                      c->status_dev, c->scratch, c->sm_count, s));
    } else {
      for (size_t e = 0; e < n_local; e++) wgu[e] = gate[e]->dev;
      CK(c, qk_launch_gemm_tc_grouped(gate[0]->L, wgu, (uint32_t)n_local, (uint32_t)n_local, cnt, (uint32_t)tokens,
                                      x_dev, lists, (uint32_t)slots, (uint32_t)top_k, g, inter, c->status_dev,
                                      c->scratch, c->sm_count, s));
      for (size_t e = 0; e < n_local; e++) wgu[e] = up[e]->dev;
      CK(c, qk_launch_gemm_tc_grouped(up[0]->L, wgu, (uint32_t)n_local, (uint32_t)n_local, cnt, (uint32_t)tokens,
                                      x_dev, lists, (uint32_t)slots, (uint32_t)top_k, u, inter, c->status_dev,
                                      c->scratch, c->sm_count, s));
    }
    CK(c, qk_launch_moe_silu_mul_grouped(g, u, cnt, (uint32_t)n_local, (uint32_t)tokens, (uint32_t)cap,
                                         (uint32_t)inter, s));
    CK(c, qk_launch_gemm_tc_grouped(down[0]->L, wd, (uint32_t)n_local, (uint32_t)n_local, cnt, (uint32_t)tokens, u, nullptr, 0, 1, o,
                                    hidden, c->status_dev, c->scratch, c->sm_count, s));
    CK(c, qk_launch_moe_combine(o, ids, pos, wts, (uint32_t)tokens, (uint32_t)top_k, (uint32_t)expert_begin,
                                (uint32_t)n_local, (uint32_t)cap, (uint32_t)hidden, y_dev, s));
    return QK_OK;
  }

  // Few tokens (decode): per expert, on the decode kernels, sized by the token counts read back.
  // scratch: ids, wts, counts, lists, then the per-expert activations (sized for every token)
  const size_t o_ids = 0, o_wts = o_ids + al(slots * 4), o_cnt = o_wts + al(slots * 4);
  const size_t o_lists = o_cnt + al(n_local * 4), o_xe = o_lists + al(n_local * slots * 4);
  const size_t o_g = o_xe + al(tokens * hidden * 4), o_u = o_g + al(tokens * inter * 4);
  const size_t o_o = o_u + al(tokens * inter * 4), need = o_o + al(tokens * hidden * 4);
  {
    int st = grow_moe(need);
    if (st) return st;
  }
  unsigned char *base = (unsigned char *)c->moe;
  int *ids = (int *)(base + o_ids), *cnt = (int *)(base + o_cnt), *lists = (int *)(base + o_lists);
  float *wts = (float *)(base + o_wts), *xe = (float *)(base + o_xe), *g = (float *)(base + o_g);
  float *u = (float *)(base + o_u), *o = (float *)(base + o_o);

  CK(c, cudaMemsetAsync(y_dev, 0, tokens * hidden * sizeof(float), s));
  CK(c, qk_launch_moe_route(logits_dev, (uint32_t)tokens, (uint32_t)n_exp, (uint32_t)top_k, ids, wts, s));
  CK(c, qk_launch_moe_lists(ids, (uint32_t)tokens, (uint32_t)top_k, (uint32_t)expert_begin, (uint32_t)n_local,
                            cnt, lists, nullptr, s));
  // the token counts size the per-expert matmuls: one small copy and a stream synchronise
  std::vector<int> counts(n_local);
  CK(c, cudaMemcpyAsync(counts.data(), cnt, n_local * sizeof(int), cudaMemcpyDeviceToHost, s));
  CK(c, cudaStreamSynchronize(s));
  for (size_t e = 0; e < n_local; e++) {
    const size_t m = (size_t)counts[e];
    if (m == 0) continue;
    const int *list = lists + e * slots;
    CK(c, qk_launch_moe_gather(x_dev, list, (uint32_t)m, (uint32_t)top_k, (uint32_t)hidden, xe, s));
    int st = gemm_dispatch(c, gate[e], xe, g, m, inter, s);
    if (st) return st;
    st = gemm_dispatch(c, up[e], xe, u, m, inter, s);
    if (st) return st;
    CK(c, qk_launch_moe_silu_mul(g, u, (uint64_t)m * inter, s));
    st = gemm_dispatch(c, down[e], u, o, m, hidden, s);
    if (st) return st;
    CK(c, qk_launch_moe_scatter(o, list, wts, (uint32_t)m, (uint32_t)top_k, (uint32_t)hidden, y_dev, s));
  }
  return QK_OK;
}

// ------------------------------------------------------------ feed-forward block
// FFN(x) = down(silu(gate x) * up x): the dense branch of feed_forward
// (crates/oxillama-arch/src/llama/model.rs:281-310) with swiglu_inplace
// (crates/oxillama-arch/src/common/swiglu.rs:15-21).
extern "C" int qk_ffn_dev(qk_ctx *c, const qk_weights *gate, const qk_weights *up, const qk_weights *down,
                          const float *x_dev, float *y_dev, size_t m, void *stream) {
  if (!c || !gate || !up || !down || !x_dev || !y_dev) return QK_INVALID_ARGUMENT;
  if (gate->device != c->device || up->device != c->device || down->device != c->device) return QK_INVALID_ARGUMENT;
  const size_t hidden = gate->L.cols, inter = gate->L.rows;
  if (up->L.cols != hidden || up->L.rows != inter || down->L.cols != inter) return QK_DIMENSION_MISMATCH;
  if (m == 0 || down->L.rows == 0) return QK_OK;
  cudaStream_t s = (cudaStream_t)stream;
  // scratch: h (and, on the unfused route, the up projection) [m x inter] each
  const size_t need = 2 * m * (inter ? inter : 1) * sizeof(float);
  if (need > c->ffn_cap) {
    CK(c, cudaDeviceSynchronize());
    if (c->ffn) cudaFree(c->ffn);
    c->ffn = nullptr, c->ffn_cap = 0;
    CK(c, cudaMalloc(&c->ffn, need));
    c->ffn_cap = need;
  }
  float *h = (float *)c->ffn, *u = h + m * inter;
  const bool fused = !c->force_simple && gate->L.type == QK_T_Q4_K && up->L.type == QK_T_Q4_K && hidden > 0 &&
                     inter > 0 && m <= QK_GEMV_MAX_M && qk_gemv_dual_supported(gate->L, (uint32_t)m);
  if (fused) {
    // gate and up in one launch (they share the split activations), silu(g) * u in its reducer
    const size_t sneed = qk_gemv_mma_scratch_bytes(gate->L, (uint32_t)m);
    if (sneed > c->scratch_cap) {
      CK(c, cudaDeviceSynchronize());
      cudaFree(c->scratch);
      c->scratch = nullptr, c->scratch_cap = 0;
      CK(c, cudaMalloc(&c->scratch, sneed * 2));
      c->scratch_cap = sneed * 2;
    }
    CK(c, qk_launch_gemv_dual(gate->L, gate->dev, up->dev, x_dev, h, (uint32_t)m, inter, c->status_dev, c->scratch,
                              c->sm_count, s));
  } else {
    int st = gemm_dispatch(c, gate, x_dev, h, m, inter, s);
    if (st) return st;
    if ((st = gemm_dispatch(c, up, x_dev, u, m, inter, s))) return st;
    CK(c, qk_launch_swiglu(h, u, (uint64_t)m * inter, s));
  }
  return gemm_dispatch(c, down, h, y_dev, m, down->L.rows, s);
}

extern "C" int qk_dequant_dev(qk_ctx *c, const qk_weights *h, float *out_dev, void *stream) {
  if (!c || !h || !out_dev) return QK_INVALID_ARGUMENT;
  CK(c, qk_launch_dequant(h->L, h->dev, out_dev, (cudaStream_t)stream));
  return QK_OK;
}

extern "C" int qk_matvec_q8_fused_dev(qk_ctx *c, const qk_weights *h, const uint8_t *acts_q8_dev,
                                      float *out_dev, void *stream) {
  if (!c || !h || !acts_q8_dev || !out_dev) return QK_INVALID_ARGUMENT;
  CK(c, qk_launch_fused_simple(h->L, h->dev, acts_q8_dev, out_dev, (cudaStream_t)stream));
  return QK_OK;
}

extern "C" int qk_quantize_q8_0_dev(qk_ctx *c, const float *x_dev, size_t n, uint8_t *out_dev,
                                    void *stream) {
  if (!c || (n && (!x_dev || !out_dev))) return QK_INVALID_ARGUMENT;
  if (n % 32 != 0) return QK_DIMENSION_MISMATCH;
  CK(c, qk_launch_quantize_q8_0(x_dev, n, out_dev, (cudaStream_t)stream));
  return QK_OK;
}

// Reads and clears the status word; the stream that ran the kernels must have been synchronised.
static int take_device_status(qk_ctx *c) {
  const unsigned v = *c->status_host;
  if (!v) return QK_OK;
  *c->status_host = 0;
  c->err = (v & QK_DEV_TIMEOUT) ? "device-side wait ran out" : "device-side range check tripped";
  return (v & QK_DEV_TIMEOUT) ? QK_TIMEOUT : QK_KERNEL_ERROR;
}

extern "C" int qk_check_device_status(qk_ctx *c, void *stream) {
  if (!c) return QK_INVALID_ARGUMENT;
  CK(c, cudaStreamSynchronize((cudaStream_t)stream));
  return take_device_status(c);
}

// ------------------------------------------------------------ host-pointer entry points
extern "C" int qk_dequant_block(qk_ctx *c, int type, const uint8_t *block, size_t block_len,
                                float *out, size_t out_len) {
  if (!c) return QK_INVALID_ARGUMENT;
  if (!type_ok(type)) return QK_UNSUPPORTED_TYPE;
  size_t bs = qk_block_size(type), bb = qk_block_bytes(type);
  if (block_len < bb) return QK_BUFFER_TOO_SMALL;
  if (out_len < bs) return QK_BUFFER_TOO_SMALL;
  if (!block || !out) return QK_INVALID_ARGUMENT;
  return qk_dequant_matrix(c, type, block, bb, 1, bs, out, bs);
}

extern "C" int qk_dequant_matrix(qk_ctx *c, int type, const uint8_t *w, size_t w_len, size_t n_rows,
                                 size_t n_cols, float *out, size_t out_len) {
  if (!c) return QK_INVALID_ARGUMENT;
  if (!type_ok(type)) return QK_UNSUPPORTED_TYPE;
  if (w_len < need_bytes(type, n_rows, n_cols)) return QK_BUFFER_TOO_SMALL;
  if (out_len < n_rows * n_cols) return QK_BUFFER_TOO_SMALL;
  if (n_rows * n_cols == 0) return QK_OK;
  if (!w || !out) return QK_INVALID_ARGUMENT;
  std::lock_guard<std::mutex> g(c->mu);
  CK(c, cudaSetDevice(c->device));
  qk_weights *h = nullptr;
  int st = upload_impl(c, type, w, n_cols, 0, n_rows, &h);  // not cached: one-shot
  if (st) return st;
  size_t nbytes = n_rows * n_cols * sizeof(float);
  st = grow(c, &c->sb, &c->sb_cap, nbytes);
  if (st == QK_OK) {
    cudaError_t e = qk_launch_dequant(h->L, h->dev, (float *)c->sb, c->stream);
    if (e == cudaSuccess) e = cudaMemcpyAsync(out, c->sb, nbytes, cudaMemcpyDeviceToHost, c->stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(c->stream);
    if (e != cudaSuccess) {
      c->err = std::string("dequant: ") + cudaGetErrorString(e);
      st = QK_CUDA_ERROR;
    }
  }
  free_weights(h);
  return st;
}

static int host_gemm(qk_ctx *c, int type, const uint8_t *w, size_t w_len, size_t n, size_t k,
                     const float *x, float *y, size_t m) {
  std::lock_guard<std::mutex> g(c->mu);
  CK(c, cudaSetDevice(c->device));
  qk_weights *h = nullptr;
  int st = cached(c, type, w, w_len, n, k, &h);
  if (st) return st;
  size_t xb = m * k * sizeof(float), yb = m * n * sizeof(float);
  if ((st = grow(c, &c->sa, &c->sa_cap, xb ? xb : 4))) return st;
  if ((st = grow(c, &c->sb, &c->sb_cap, yb ? yb : 4))) return st;
  if (xb) CK(c, cudaMemcpyAsync(c->sa, x, xb, cudaMemcpyHostToDevice, c->stream));
  // Decode-sized calls into pinned host memory: the kernels that serve M <= 4 only store y
  // (a few KB, 32 contiguous bytes per 8-row chunk), so they write it straight through the
  // mapping and the device-to-host copy with its launch drops out.
  float *ydev = (float *)c->sb;
  bool mapped = false;
  if (yb && m <= QK_GEMV_MAX_M && !c->force_simple && qk_gemv_fast_supported(h->L, (uint32_t)m)) {
    cudaPointerAttributes pa;
    if (cudaPointerGetAttributes(&pa, y) == cudaSuccess && pa.type == cudaMemoryTypeHost &&
        pa.devicePointer)
      ydev = (float *)pa.devicePointer, mapped = true;
    else
      (void)cudaGetLastError();
  }
  if ((st = gemm_dispatch(c, h, (const float *)c->sa, ydev, m, n, c->stream))) return st;
  if (yb && !mapped) CK(c, cudaMemcpyAsync(y, c->sb, yb, cudaMemcpyDeviceToHost, c->stream));
  CK(c, cudaStreamSynchronize(c->stream));
  return take_device_status(c);  // a bounded wait that ran out leaves y invalid: say so
}

extern "C" int qk_gemv(qk_ctx *c, int type, const uint8_t *w, size_t w_len, size_t n_rows,
                       size_t n_cols, const float *x, size_t x_len, float *y, size_t y_len) {
  if (!c) return QK_INVALID_ARGUMENT;
  if (!type_ok(type)) return QK_UNSUPPORTED_TYPE;
  if (x_len < n_cols) return QK_DIMENSION_MISMATCH;  // order as reference/q4_k.rs:117-128
  if (y_len < n_rows) return QK_DIMENSION_MISMATCH;
  if (w_len < need_bytes(type, n_rows, n_cols)) return QK_BUFFER_TOO_SMALL;
  if (n_rows == 0) return QK_OK;
  if (!w || !y || (n_cols && !x)) return QK_INVALID_ARGUMENT;
  return host_gemm(c, type, w, w_len, n_rows, n_cols, x, y, 1);
}

extern "C" int qk_gemm(qk_ctx *c, int type, const uint8_t *w, size_t w_len, const float *x,
                       size_t x_len, float *y, size_t y_len, size_t m, size_t n, size_t k) {
  if (!c) return QK_INVALID_ARGUMENT;
  if (!type_ok(type)) return QK_UNSUPPORTED_TYPE;
  if (x_len < m * k) return QK_DIMENSION_MISMATCH;
  if (y_len < m * n) return QK_DIMENSION_MISMATCH;
  if (w_len < need_bytes(type, n, k)) return QK_BUFFER_TOO_SMALL;
  if (m == 0 || n == 0) return QK_OK;
  if (!w || !y || (k && !x)) return QK_INVALID_ARGUMENT;
  return host_gemm(c, type, w, w_len, n, k, x, y, m);
}

// ------------------------------------------------------------ GpuKernel-shaped entry points
// crates/oxillama-gpu/src/kernels/mod.rs:91-106 (e.g. kernels/q4_k.rs:170-195): raw weight
// bytes and dimensions instead of a QuantTensor; checks in that implementation's order, every
// failed size check being its GpuError::BufferSize { expected, got } (text in qk_last_error).
static int buffer_size(qk_ctx *c, size_t expected, size_t got) {
  c->err = "Buffer size mismatch: expected " + std::to_string(expected) + ", got " + std::to_string(got);
  return QK_BUFFER_TOO_SMALL;
}

extern "C" int qk_gpu_gemv(qk_ctx *c, int type, const uint8_t *weight_bytes, size_t weight_len,
                           const float *input, size_t input_len, float *output, size_t output_len,
                           size_t rows, size_t cols) {
  if (!c) return QK_INVALID_ARGUMENT;
  if (!type_ok(type)) {
    c->err = "Unsupported quant type for GPU: type id " + std::to_string(type);
    return QK_UNSUPPORTED_TYPE;
  }
  if (output_len < rows) return buffer_size(c, rows, output_len);
  if (input_len < cols) return buffer_size(c, cols, input_len);
  if (weight_len < need_bytes(type, rows, cols)) return buffer_size(c, need_bytes(type, rows, cols), weight_len);
  if (rows == 0) return QK_OK;
  if (!weight_bytes && need_bytes(type, rows, cols)) return QK_INVALID_ARGUMENT;
  if (!output || (cols && !input)) return QK_INVALID_ARGUMENT;
  return host_gemm(c, type, weight_bytes, weight_len, rows, cols, input, output, 1);
}

// Y[b][r] = sum_c A[r][c] X[b][c]: kernels/batched_gemv.rs:36-50 with the matrix still
// quantised (that function takes it dequantised to f32; its callers dequantise first).
extern "C" int qk_gpu_gemv_batched(qk_ctx *c, int type, const uint8_t *weight_bytes, size_t weight_len,
                                   const float *vectors, size_t vectors_len, float *output, size_t output_len,
                                   size_t rows, size_t cols, size_t batch_size) {
  if (!c) return QK_INVALID_ARGUMENT;
  if (!type_ok(type)) {
    c->err = "Unsupported quant type for GPU: type id " + std::to_string(type);
    return QK_UNSUPPORTED_TYPE;
  }
  if (weight_len < need_bytes(type, rows, cols)) return buffer_size(c, need_bytes(type, rows, cols), weight_len);
  if (vectors_len != batch_size * cols) return buffer_size(c, batch_size * cols, vectors_len);  // exact, as there
  if (output_len < batch_size * rows) return buffer_size(c, batch_size * rows, output_len);
  if (rows == 0 || batch_size == 0) return QK_OK;
  if (!output) return QK_INVALID_ARGUMENT;
  if (cols == 0) {  // batched_gemv.rs:88-90: zeros
    memset(output, 0, batch_size * rows * sizeof(float));
    return QK_OK;
  }
  if (!weight_bytes || !vectors) return QK_INVALID_ARGUMENT;
  return host_gemm(c, type, weight_bytes, weight_len, rows, cols, vectors, output, batch_size);
}

extern "C" int qk_matvec_q8_fused(qk_ctx *c, int type, const uint8_t *w, size_t w_len,
                                  const uint8_t *acts_q8, size_t acts_len, float *out,
                                  size_t out_len, size_t n_rows, size_t n_cols) {
  if (!c) return QK_INVALID_ARGUMENT;
  if (!type_ok(type)) return QK_UNSUPPORTED_TYPE;
  if (out_len < n_rows) return QK_DIMENSION_MISMATCH;  // order as reference/q4_k.rs:226-250
  size_t bs = qk_block_size(type);
  size_t acts_needed = ((n_cols + bs - 1) / bs) * (bs / 32) * 34;
  if (w_len < need_bytes(type, n_rows, n_cols)) return QK_BUFFER_TOO_SMALL;
  if (acts_len < acts_needed) return QK_BUFFER_TOO_SMALL;
  if (n_rows == 0 || n_cols == 0) return QK_OK;
  if (!w || !acts_q8 || !out) return QK_INVALID_ARGUMENT;
  std::lock_guard<std::mutex> g(c->mu);
  CK(c, cudaSetDevice(c->device));
  qk_weights *h = nullptr;
  int st = cached(c, type, w, w_len, n_rows, n_cols, &h);
  if (st) return st;
  if ((st = grow(c, &c->sa, &c->sa_cap, acts_needed))) return st;
  if ((st = grow(c, &c->sb, &c->sb_cap, n_rows * sizeof(float)))) return st;
  CK(c, cudaMemcpyAsync(c->sa, acts_q8, acts_needed, cudaMemcpyHostToDevice, c->stream));
  CK(c, cudaMemcpyAsync(c->sb, out, n_rows * sizeof(float), cudaMemcpyHostToDevice, c->stream));
  CK(c, qk_launch_fused_simple(h->L, h->dev, (const uint8_t *)c->sa, (float *)c->sb, c->stream));
  CK(c, cudaMemcpyAsync(out, c->sb, n_rows * sizeof(float), cudaMemcpyDeviceToHost, c->stream));
  CK(c, cudaStreamSynchronize(c->stream));
  return QK_OK;
}

extern "C" int qk_quantize_q8_0(qk_ctx *c, const float *x, size_t n, uint8_t *out, size_t out_len) {
  if (!c) return QK_INVALID_ARGUMENT;
  if (n % 32 != 0) return QK_DIMENSION_MISMATCH;  // quantize.rs:59-64
  if (out_len < n / 32 * 34) return QK_BUFFER_TOO_SMALL;
  if (n == 0) return QK_OK;
  if (!x || !out) return QK_INVALID_ARGUMENT;
  std::lock_guard<std::mutex> g(c->mu);
  CK(c, cudaSetDevice(c->device));
  int st;
  if ((st = grow(c, &c->sa, &c->sa_cap, n * sizeof(float)))) return st;
  if ((st = grow(c, &c->sb, &c->sb_cap, n / 32 * 34))) return st;
  CK(c, cudaMemcpyAsync(c->sa, x, n * sizeof(float), cudaMemcpyHostToDevice, c->stream));
  CK(c, qk_launch_quantize_q8_0((const float *)c->sa, n, (uint8_t *)c->sb, c->stream));
  CK(c, cudaMemcpyAsync(out, c->sb, n / 32 * 34, cudaMemcpyDeviceToHost, c->stream));
  CK(c, cudaStreamSynchronize(c->stream));
  return QK_OK;
}
