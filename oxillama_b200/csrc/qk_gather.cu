// Row-sharded outputs gathered over NVLink without a collective library: every rank of a
// node owns a [m_cap x world * rows] f32 buffer; a sharded matvec stores its column
// block into the buffer of every rank (peer stores, from inside the matvec kernel where
// that kernel supports it, else from a small push kernel) and publishes an epoch flag
// in every rank; a consumer waits (bounded) until all ranks' flags have reached its own
// epoch.  Buffers and flags are plain cudaMalloc memory shared through CUDA IPC handles,
// which the ranks exchange by whatever host channel they have.
//
// Replaces, for a sharded layer, the NCCL all-gather that follows the matvec in the
// reference-shaped design (one all-gather of y per linear).  No multicast loads, no
// waits without a time limit.
#include <cstring>

#include "qk_internal.h"
#include "qk_pipe.cuh"

struct qk_gather {
  int world, rank, device;
  size_t rows, m_cap;          // rows per rank, most activation rows a call may carry
  float *local;                // [m_cap][world * rows]
  unsigned *ctl;               // flags[world], counter, epoch
  float *peer_y[QK_MAX_PEERS];
  unsigned *peer_ctl[QK_MAX_PEERS];
  bool opened[QK_MAX_PEERS];
};

namespace {

// Copies this rank's column block of the local buffer into every other rank's buffer,
// then the last CTA publishes the epoch (same protocol as the fused matvec).
__global__ void __launch_bounds__(256)
    qk_gather_push_kernel(QkPeers peers, const float *__restrict__ src, uint32_t m, uint32_t rows,
                          uint64_t ldy) {
  const uint64_t n = (uint64_t)m * rows;
  for (uint64_t i = blockIdx.x * 256ull + threadIdx.x; i < n; i += (uint64_t)gridDim.x * 256) {
    const uint64_t off = (i / rows) * ldy + (i % rows);
    const float v = src[off];
    for (uint32_t p = 0; p < peers.n; p++)
      if (p != peers.rank) peers.y[p][off] = v;
  }
  __threadfence();  // every thread orders its own peer stores before the count below (read on this GPU)
  __syncthreads();
  if (threadIdx.x == 0) {
    if (atomicAdd(peers.counter, 1u) == gridDim.x - 1) {
      __threadfence();
      *peers.counter = 0;
      const unsigned e = *peers.epoch + 1;
      *peers.epoch = e;
      __threadfence_system();
      for (uint32_t p = 0; p < peers.n; p++)
        asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(peers.flags[p] + peers.rank), "r"(e) : "memory");
    }
  }
}

// One thread per rank: waits until that rank's flag has reached the local epoch, for at
// most a quarter of a second.
__global__ void __launch_bounds__(32)
    qk_gather_wait_kernel(const unsigned *flags, const unsigned *epoch, uint32_t n, unsigned *status) {
  if (threadIdx.x >= n) return;
  const unsigned want = *epoch;
  unsigned long long t0;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
  for (;;) {
    unsigned v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(flags + threadIdx.x) : "memory");
    if ((int)(v - want) >= 0) return;
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    if (t - t0 > 250000000ull) {
      atomicOr(status, QK_DEV_TIMEOUT);
      return;
    }
  }
}

// First touch of every peer mapping from this GPU (one zero into this rank's block of
// each peer's freshly cleared buffer), so that the first real call meets established
// translations.
__global__ void qk_gather_touch_kernel(QkPeers peers) {
  if (threadIdx.x < peers.n) {
    peers.y[threadIdx.x][0] = 0.f;
    __threadfence_system();
  }
}

int fail(qk_ctx *c, cudaError_t e, const char *what) {
  c->err = std::string(what) + ": " + cudaGetErrorString(e);
  return QK_CUDA_ERROR;
}

QkPeers peers_of(const qk_gather *g) {
  QkPeers p = {};
  p.n = (uint32_t)g->world, p.rank = (uint32_t)g->rank;
  for (int r = 0; r < g->world; r++) {
    p.y[r] = g->peer_y[r] + (size_t)g->rank * g->rows;
    p.flags[r] = g->peer_ctl[r];
  }
  p.counter = g->ctl + QK_MAX_PEERS, p.epoch = g->ctl + QK_MAX_PEERS + 1;
  return p;
}

}  // namespace

extern "C" int qk_gather_create(qk_ctx *c, size_t rows_per_rank, size_t m_cap, int world, int rank,
                                qk_gather **out) {
  if (!c || !out || world < 1 || world > QK_MAX_PEERS || rank < 0 || rank >= world || rows_per_rank == 0 ||
      m_cap == 0)
    return QK_INVALID_ARGUMENT;
  std::lock_guard<std::mutex> lk(c->mu);
  cudaSetDevice(c->device);
  qk_gather *g = new qk_gather();
  g->world = world, g->rank = rank, g->device = c->device, g->rows = rows_per_rank, g->m_cap = m_cap;
  cudaError_t e = cudaMalloc(&g->local, m_cap * world * rows_per_rank * sizeof(float));
  if (e == cudaSuccess) e = cudaMalloc(&g->ctl, (QK_MAX_PEERS + 2) * sizeof(unsigned));
  if (e == cudaSuccess) e = cudaMemset(g->ctl, 0, (QK_MAX_PEERS + 2) * sizeof(unsigned));
  if (e == cudaSuccess) e = cudaMemset(g->local, 0, m_cap * world * rows_per_rank * sizeof(float));
  if (e == cudaSuccess) e = cudaDeviceSynchronize();  // the clears must have run before a peer can store here
  if (e != cudaSuccess) {
    if (g->local) cudaFree(g->local);
    if (g->ctl) cudaFree(g->ctl);
    delete g;
    return fail(c, e, "qk_gather_create");
  }
  g->peer_y[rank] = g->local, g->peer_ctl[rank] = g->ctl, g->opened[rank] = false;
  *out = g;
  return QK_OK;
}

// handle: 128 bytes = the IPC handles of the buffer and of the control words.
extern "C" int qk_gather_export(qk_ctx *c, qk_gather *g, unsigned char *handle, size_t len) {
  if (!c || !g || !handle || len < 128) return QK_INVALID_ARGUMENT;
  cudaSetDevice(c->device);
  cudaIpcMemHandle_t h0, h1;
  cudaError_t e = cudaIpcGetMemHandle(&h0, g->local);
  if (e == cudaSuccess) e = cudaIpcGetMemHandle(&h1, g->ctl);
  if (e != cudaSuccess) return fail(c, e, "qk_gather_export");
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
  memcpy(handle, &h0, 64), memcpy(handle + 64, &h1, 64);
  return QK_OK;
}

extern "C" int qk_gather_import(qk_ctx *c, qk_gather *g, int peer_rank, const unsigned char *handle, size_t len) {
  if (!c || !g || !handle || len < 128 || peer_rank < 0 || peer_rank >= g->world || peer_rank == g->rank)
    return QK_INVALID_ARGUMENT;
  cudaSetDevice(c->device);
  cudaIpcMemHandle_t h0, h1;
  memcpy(&h0, handle, 64), memcpy(&h1, handle + 64, 64);
  void *p0 = nullptr, *p1 = nullptr;
  cudaError_t e = cudaIpcOpenMemHandle(&p0, h0, cudaIpcMemLazyEnablePeerAccess);
  if (e == cudaSuccess) e = cudaIpcOpenMemHandle(&p1, h1, cudaIpcMemLazyEnablePeerAccess);
  if (e != cudaSuccess) {
    if (p0) cudaIpcCloseMemHandle(p0);
    return fail(c, e, "qk_gather_import");
  }
  g->peer_y[peer_rank] = (float *)p0, g->peer_ctl[peer_rank] = (unsigned *)p1, g->opened[peer_rank] = true;
  return QK_OK;
}

// After every import: touches all peer mappings once and waits for it.  Call it on every
// rank, then synchronise the ranks on the host, before the first qk_gemm_gather_dev.
extern "C" int qk_gather_ready(qk_ctx *c, qk_gather *g) {
  if (!c || !g) return QK_INVALID_ARGUMENT;
  for (int r = 0; r < g->world; r++)
    if (!g->peer_y[r]) return QK_INVALID_ARGUMENT;
  cudaSetDevice(c->device);
  qk_gather_touch_kernel<<<1, 32>>>(peers_of(g));
  cudaError_t e = cudaGetLastError();
  if (e == cudaSuccess) e = cudaDeviceSynchronize();
  return e == cudaSuccess ? QK_OK : fail(c, e, "qk_gather_ready");
}

extern "C" int qk_gather_destroy(qk_ctx *c, qk_gather *g) {
  if (!c || !g) return QK_INVALID_ARGUMENT;
  cudaSetDevice(c->device);
  cudaDeviceSynchronize();
  for (int r = 0; r < g->world; r++)
    if (g->opened[r]) cudaIpcCloseMemHandle(g->peer_y[r]), cudaIpcCloseMemHandle(g->peer_ctl[r]);
  cudaFree(g->local), cudaFree(g->ctl);
  delete g;
  return QK_OK;
}

extern "C" float *qk_gather_buffer(qk_gather *g) { return g ? g->local : nullptr; }

extern "C" int qk_gather_wait_dev(qk_ctx *c, qk_gather *g, void *stream);

extern "C" int qk_gemm_gather_after_dev(qk_ctx *c, const qk_weights *h, const float *x_dev, size_t m, qk_gather *g,
                                        qk_gather *after, void *stream) {
  if (!c || !h || !x_dev || !g) return QK_INVALID_ARGUMENT;
  if (after && after->device != c->device) return QK_INVALID_ARGUMENT;
  if (h->device != c->device || g->device != c->device) return QK_INVALID_ARGUMENT;
  if (h->L.rows != g->rows || m == 0 || m > g->m_cap) return QK_DIMENSION_MISMATCH;
  for (int r = 0; r < g->world; r++)
    if (!g->peer_y[r]) {
      c->err = "qk_gemm_gather_dev: a rank's buffer has not been imported";
      return QK_INVALID_ARGUMENT;
    }
  cudaStream_t s = (cudaStream_t)stream;
  const uint64_t ldy = (uint64_t)g->world * g->rows;
  QkPeers peers = peers_of(g);
  float *mine = g->local + (size_t)g->rank * g->rows;
  const bool fused = !c->force_simple && m <= QK_GEMV_MAX_M && h->L.type == QK_T_Q4_K &&
                     qk_gemv_mma_supported(h->L, (uint32_t)m);
  if (after) {
    if (fused) {  // the matvec kernels wait themselves, under their own prologue
      peers.wait_flags = after->ctl, peers.wait_epoch = after->ctl + QK_MAX_PEERS + 1;
      peers.wait_n = (uint32_t)after->world;
    } else {
      int st = qk_gather_wait_dev(c, after, stream);
      if (st) return st;
    }
  }
  if (!c->force_simple && m <= QK_GEMV_MAX_M && h->L.type == QK_T_Q4_K && qk_gemv_mma_supported(h->L, (uint32_t)m)) {
    // fused: the matvec kernel itself stores into every rank and signals
    const size_t need = qk_gemv_mma_scratch_bytes(h->L, (uint32_t)m);
    if (need > c->scratch_cap) {
      cudaError_t e = cudaDeviceSynchronize();
      if (e != cudaSuccess) return fail(c, e, "qk_gemm_gather_dev");
      cudaFree(c->scratch);
      c->scratch = nullptr, c->scratch_cap = 0;
      e = cudaMalloc(&c->scratch, need * 2);
      if (e != cudaSuccess) return fail(c, e, "qk_gemm_gather_dev");
      c->scratch_cap = need * 2;
    }
    cudaError_t e = qk_launch_gemv_mma(h->L, h->dev, x_dev, mine, (uint32_t)m, ldy, c->status_dev, c->scratch,
                                       c->sm_count, s, &peers);
    return e == cudaSuccess ? QK_OK : fail(c, e, "qk_gemm_gather_dev");
  }
  // any other shape or format: the ordinary kernels write this rank's block of the local
  // buffer, then a push kernel copies it to the other ranks and signals
  int st = qk_gemm_dev(c, h, x_dev, mine, m, ldy, stream);
  if (st) return st;
  const uint64_t n = (uint64_t)m * g->rows;
  unsigned blocks = (unsigned)((n + 255) / 256);
  if (blocks > 296) blocks = 296;
  qk_gather_push_kernel<<<blocks, 256, 0, s>>>(peers, mine, (uint32_t)m, (uint32_t)g->rows, ldy);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? QK_OK : fail(c, e, "qk_gemm_gather_dev");
}

extern "C" int qk_gemm_gather_dev(qk_ctx *c, const qk_weights *h, const float *x_dev, size_t m, qk_gather *g,
                                  void *stream) {
  return qk_gemm_gather_after_dev(c, h, x_dev, m, g, nullptr, stream);
}

extern "C" int qk_gather_wait_dev(qk_ctx *c, qk_gather *g, void *stream) {
  if (!c || !g) return QK_INVALID_ARGUMENT;
  qk_gather_wait_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(g->ctl, g->ctl + QK_MAX_PEERS + 1, (uint32_t)g->world,
                                                           c->status_dev);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? QK_OK : fail(c, e, "qk_gather_wait_dev");
}
