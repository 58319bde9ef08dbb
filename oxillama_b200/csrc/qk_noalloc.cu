// qk_gemm_dev_noalloc: the Q4_K decode matvec for callers that must not allocate.
//
// Some users of this library run where device allocation is off the table once
// they are up: an inference server that reserved all of HBM for its own pools at
// start-up, code running under a memory budget enforced by a supervisor, or a
// latency-critical loop that may not take the driver's allocator lock.  The
// regular entry points keep their scratch (the split activations that travel
// between the two kernels of the matvec) in a buffer the context allocates and,
// for large activations, re-allocates.  This entry point instead keeps that
// scratch in a fixed array that is part of the library image: every GPU that
// loads the library holds QK_NOALLOC_SCRATCH_BYTES of it until the process exits,
// and nothing is allocated or freed by the call.
#include "qk_internal.h"

#define QK_NOALLOC_SCRATCH_BYTES (96u * 1024u)

// The scratch itself.  In host code this name is only a stand-in for the symbol;
// the device address is looked up once per device below and handed to the kernels.
static __device__ __align__(256) unsigned char qk_noalloc_scratch[QK_NOALLOC_SCRATCH_BYTES];

namespace {
constexpr int MAX_DEVICES = 64;
std::mutex g_mu;
unsigned char *g_scratch_ptr[MAX_DEVICES] = {};  // device address of the array, per device
}  // namespace

// y_dev[i * ldy + j] = dot(W_shard row j, x_dev row i) for a Q4_K shard and m <= 4,
// like qk_gemm_dev, without allocating.
//
// The first call on a device looks up the address of the built-in scratch array
// (cudaGetSymbolAddress, with that device current); make that first call before
// capturing a stream into a CUDA graph.  The split activations of the call must
// fit QK_NOALLOC_SCRATCH_BYTES (96 KiB: e.g. m = 3 rows of 8 192 columns);
// larger requests are refused with QK_INVALID_ARGUMENT and a message in
// qk_last_error.  All calls on a device share the one array and it keeps the
// previous call's contents: the call rewrites every byte it later reads, so
// nothing needs clearing, but two calls that overlap on the GPU (different
// streams, or graphs replayed concurrently) race on it — issue them in order.
extern "C" int qk_gemm_dev_noalloc(qk_ctx *c, const qk_weights *h, const float *x_dev, float *y_dev,
                                   size_t m, size_t ldy, void *stream) {
  if (!c || !h || !x_dev || !y_dev) return QK_INVALID_ARGUMENT;
  if (h->device != c->device || c->device < 0 || c->device >= MAX_DEVICES) return QK_INVALID_ARGUMENT;
  if (h->L.type != QK_TYPE_Q4_K) {
    c->err = "qk_gemm_dev_noalloc: only Q4_K weights are served by this entry point";
    return QK_UNSUPPORTED_TYPE;
  }
  if (ldy < h->L.rows) return QK_DIMENSION_MISMATCH;
  if (m == 0 || h->L.rows == 0) return QK_OK;  // nothing to write
  if (h->L.cols == 0) {  // empty dot products: y = 0, as qk_gemm_dev gives (a memset allocates nothing)
    cudaError_t e = cudaMemset2DAsync(y_dev, ldy * sizeof(float), 0, h->L.rows * sizeof(float), m,
                                      (cudaStream_t)stream);
    if (e != cudaSuccess) {
      c->err = std::string("qk_gemm_dev_noalloc: memset: ") + cudaGetErrorString(e);
      return QK_CUDA_ERROR;
    }
    return QK_OK;
  }
  if (m > 4 || !qk_gemv_mma_supported(h->L, (uint32_t)m)) {
    c->err = "qk_gemm_dev_noalloc: needs 1 <= m <= 4 and a shape the Q4_K decode kernel takes";
    return QK_INVALID_ARGUMENT;
  }
  const size_t need = qk_gemv_mma_scratch_bytes(h->L, (uint32_t)m);
  if (need > QK_NOALLOC_SCRATCH_BYTES) {
    c->err = "qk_gemm_dev_noalloc: split activations need " + std::to_string(need) +
             " bytes, the built-in scratch holds " + std::to_string(QK_NOALLOC_SCRATCH_BYTES);
    return QK_INVALID_ARGUMENT;
  }
  unsigned char *ptr;
  {
    std::lock_guard<std::mutex> g(g_mu);
    ptr = g_scratch_ptr[c->device];
    if (!ptr) {  // set-up, once per device, with that device current (the caller's own
                 // current device is put back afterwards)
      int prev = -1;
      cudaError_t e = cudaGetDevice(&prev);
      if (e == cudaSuccess) e = cudaSetDevice(c->device);
      if (e == cudaSuccess) e = cudaGetSymbolAddress((void **)&ptr, qk_noalloc_scratch);
      if (prev >= 0 && prev != c->device) cudaSetDevice(prev);
      if (e != cudaSuccess || !ptr) {
        c->err = std::string("qk_gemm_dev_noalloc: cudaGetSymbolAddress: ") + cudaGetErrorString(e);
        return QK_CUDA_ERROR;
      }
      g_scratch_ptr[c->device] = ptr;
    }
  }
  cudaError_t e = qk_launch_gemv_mma_split(h->L, h->dev, x_dev, y_dev, (uint32_t)m, ldy, c->status_dev,
                                           ptr, c->sm_count, (cudaStream_t)stream);
  if (e != cudaSuccess) {
    c->err = std::string("qk_gemm_dev_noalloc: launch: ") + cudaGetErrorString(e);
    return QK_CUDA_ERROR;
  }
  return QK_OK;
}
