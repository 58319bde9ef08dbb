// Row-sharded outputs gathered over NVLink without a collective library.
//
// Every rank of a node owns, per gather object, an array of 8-byte slots, one per element
// of the gathered [m_cap x world * rows] result: (f32 value, tag), the tag being the
// ordinal of the sharded call that produced the value.  A sharded matvec stores each of
// its results, as one 64-bit word, into the slot of every rank (peer stores issued from
// inside the matvec kernel where that kernel supports it, else from a small push kernel
// behind the ordinary one).  A consumer polls a slot until it carries the tag of the call
// it wants (bounded: a quarter of a second, then QK_TIMEOUT): either the next matvec
// kernel itself, which reads its activations straight out of the slots, or
// qk_gather_wait_dev, which unpacks them into a plain f32 buffer.  Because value and tag
// travel in one single-copy-atomic store there is no flag behind the data, hence no fence
// that waits for a peer's acknowledgement and no last-CTA publish on the producer's
// critical path.  Slot arrays are plain cudaMalloc memory shared through CUDA IPC handles,
// which the ranks exchange by whatever host channel they have.
//
// Replaces, for a sharded layer, the all-gather that follows the matvec in the
// reference-shaped design (one all-gather of y per linear,
// crates/oxillama-arch/src/common/linear.rs:77-98).  No multicast loads, no waits without
// a time limit.
#include <cstring>

#include "qk_internal.h"
#include "qk_peer.cuh"
#include "qk_pipe.cuh"

struct qk_gather {
  int world, rank, device;
  size_t rows, m_cap;          // rows per rank, most activation rows a call may carry
  size_t last_m;               // activation rows of the latest call
  float *local;                // [m_cap][world * rows] plain result, filled by qk_gather_wait_dev
  unsigned long long *slots;   // [m_cap][world * rows] tagged slots, written by every rank
  unsigned *ctl;               // [0] CTAs of the running launch counted in, [1] calls issued (the latest tag)
  unsigned long long *peer_slots[QK_MAX_PEERS];
  bool opened[QK_MAX_PEERS];   // peer_slots[r] came from cudaIpcOpenMemHandle
};

namespace {

using namespace qkpeer;

// Stores this rank's column block (already computed into the plain buffer) into the slots
// of every rank, tagged with this call's ordinal; the last CTA records the call.
__global__ void __launch_bounds__(256)
    qk_gather_push_kernel(QkPeers peers, const float *__restrict__ src, uint32_t m, uint32_t rows,
                          uint64_t ldy) {
  qkpipe::pdl_launch_dependents();  // the next kernel may start its prologue
  qkpipe::pdl_wait();               // src and the call count belong to the kernels before this one
  // this call's tag = the object's call count + 1; the CTA that is counted in last knows that
  // every CTA has read the count and moves it on
  __shared__ unsigned tag_s;
  if (threadIdx.x == 0) {
    unsigned e;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(e) : "l"(peers.epoch) : "memory");
    if (atomicAdd(peers.counter, 1u) == gridDim.x - 1) {
      *reinterpret_cast<volatile unsigned *>(peers.counter) = 0;
      *reinterpret_cast<volatile unsigned *>(peers.epoch) = e + 1u;
    }
    tag_s = e + 1u;
  }
  __syncthreads();
  const unsigned tag = tag_s;
  const uint64_t n = (uint64_t)m * rows;
  for (uint64_t i = blockIdx.x * 256ull + threadIdx.x; i < n; i += (uint64_t)gridDim.x * 256) {
    const uint64_t off = (i / rows) * ldy + (i % rows);
    const float v = src[off];
    for (uint32_t p = 0; p < peers.n; p++) slot_store(peers.slots[p] + off, v, tag);
  }
}

// Unpacks the latest call: every slot of the [m x ld] result is polled until it carries
// the call's tag (each thread gives up after a quarter of a second) and its value goes
// into the plain buffer.
__global__ void __launch_bounds__(256)
    qk_gather_unpack_kernel(const unsigned long long *slots, const unsigned *epoch, float *__restrict__ out,
                            uint64_t n, unsigned *status) {
  // Programmatic dependent launch on both sides: the kernel after this one (usually the next
  // matvec) becomes resident and prefetches its weights while the slots are polled, and this
  // kernel was itself resident before the matvec in front of it had drained.
  qkpipe::pdl_launch_dependents();
  qkpipe::pdl_wait();  // the call count is written by the last CTA of the producing kernel
  const unsigned want = *reinterpret_cast<const volatile unsigned *>(epoch);
  bool arrived = true;
  for (uint64_t i = blockIdx.x * 256ull + threadIdx.x; i < n; i += (uint64_t)gridDim.x * 256) {
    float v = 0.f;
    if (arrived && !slot_wait(slots + i, want, v)) {
      arrived = false;
      atomicOr(status, QK_DEV_TIMEOUT);
    }
    out[i] = v;
  }
}

// First touch of every peer mapping from this GPU (slot 0 of this rank's block in each
// peer's freshly cleared array is written with its initial contents, value 0 and tag 0), so
// that the first real call meets established translations.
__global__ void qk_gather_touch_kernel(QkPeers peers) {
  if (threadIdx.x < peers.n) {
    slot_store(peers.slots[threadIdx.x], 0.f, 0u);
    __threadfence_system();
  }
}

// Launch with programmatic stream serialization allowed (the kernels above order themselves
// with griddepcontrol.wait).
template <typename... KArgs, typename... Args>
cudaError_t launch_pdl(void (*kern)(KArgs...), unsigned blocks, unsigned threads, cudaStream_t s, Args... args) {
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[0].val.programmaticStreamSerializationAllowed = 1;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(blocks), cfg.blockDim = dim3(threads), cfg.stream = s;
  cfg.attrs = at, cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kern, KArgs(args)...);
}

int fail(qk_ctx *c, cudaError_t e, const char *what) {
  c->err = std::string(what) + ": " + cudaGetErrorString(e);
  return QK_CUDA_ERROR;
}

QkPeers peers_of(const qk_gather *g) {
  QkPeers p = {};
  p.n = (uint32_t)g->world, p.rank = (uint32_t)g->rank;
  for (int r = 0; r < g->world; r++) p.slots[r] = g->peer_slots[r] + (size_t)g->rank * g->rows;
  p.counter = g->ctl, p.epoch = g->ctl + 1;
  return p;
}

size_t elems(const qk_gather *g) { return g->m_cap * (size_t)g->world * g->rows; }

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
  g->last_m = m_cap;
  const size_t n = elems(g);
  cudaError_t e = cudaMalloc(&g->local, n * sizeof(float));
  if (e == cudaSuccess) e = cudaMalloc(&g->slots, n * sizeof(unsigned long long));
  if (e == cudaSuccess) e = cudaMalloc(&g->ctl, 2 * sizeof(unsigned));
  if (e == cudaSuccess) e = cudaMemset(g->ctl, 0, 2 * sizeof(unsigned));
  if (e == cudaSuccess) e = cudaMemset(g->local, 0, n * sizeof(float));
  if (e == cudaSuccess) e = cudaMemset(g->slots, 0, n * sizeof(unsigned long long));  // tag 0: nothing arrived
  if (e == cudaSuccess) e = cudaDeviceSynchronize();  // the clears must have run before a peer can store here
  if (e != cudaSuccess) {
    if (g->local) cudaFree(g->local);
    if (g->slots) cudaFree(g->slots);
    if (g->ctl) cudaFree(g->ctl);
    delete g;
    return fail(c, e, "qk_gather_create");
  }
  g->peer_slots[rank] = g->slots;
  *out = g;
  return QK_OK;
}

// handle: 128 bytes; the first 64 are the IPC handle of the slot array, the rest is reserved.
extern "C" int qk_gather_export(qk_ctx *c, qk_gather *g, unsigned char *handle, size_t len) {
  if (!c || !g || !handle || len < 128) return QK_INVALID_ARGUMENT;
  cudaSetDevice(c->device);
  cudaIpcMemHandle_t h0;
  cudaError_t e = cudaIpcGetMemHandle(&h0, g->slots);
  if (e != cudaSuccess) return fail(c, e, "qk_gather_export");
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
  memset(handle, 0, 128);
  memcpy(handle, &h0, 64);
  return QK_OK;
}

extern "C" int qk_gather_import(qk_ctx *c, qk_gather *g, int peer_rank, const unsigned char *handle, size_t len) {
  if (!c || !g || !handle || len < 128 || peer_rank < 0 || peer_rank >= g->world || peer_rank == g->rank ||
      g->peer_slots[peer_rank])
    return QK_INVALID_ARGUMENT;
  cudaSetDevice(c->device);
  cudaIpcMemHandle_t h0;
  memcpy(&h0, handle, 64);
  void *p0 = nullptr;
  cudaError_t e = cudaIpcOpenMemHandle(&p0, h0, cudaIpcMemLazyEnablePeerAccess);
  if (e != cudaSuccess) return fail(c, e, "qk_gather_import");
  g->peer_slots[peer_rank] = (unsigned long long *)p0, g->opened[peer_rank] = true;
  return QK_OK;
}

// The same wiring for a peer that lives in this process (several contexts driven by one
// host thread, or several "ranks" on one GPU in a test): no IPC handle, the peer's slot
// array is used directly.  With the peer on another GPU, access to it is enabled first.
extern "C" int qk_gather_import_local(qk_ctx *c, qk_gather *g, int peer_rank, qk_gather *peer) {
  if (!c || !g || !peer || peer_rank < 0 || peer_rank >= g->world || peer_rank == g->rank ||
      g->peer_slots[peer_rank] || peer->world != g->world || peer->rank != peer_rank || peer->rows != g->rows ||
      peer->m_cap != g->m_cap)
    return QK_INVALID_ARGUMENT;
  if (peer->device != g->device) {
    cudaSetDevice(c->device);
    cudaError_t e = cudaDeviceEnablePeerAccess(peer->device, 0);
    if (e == cudaErrorPeerAccessAlreadyEnabled) (void)cudaGetLastError(), e = cudaSuccess;
    if (e != cudaSuccess) return fail(c, e, "qk_gather_import_local");
  }
  g->peer_slots[peer_rank] = peer->slots, g->opened[peer_rank] = false;
  return QK_OK;
}

// After every import: touches all peer mappings once and waits for it.  Call it on every
// rank, then synchronise the ranks on the host, before the first qk_gemm_gather_dev.
extern "C" int qk_gather_ready(qk_ctx *c, qk_gather *g) {
  if (!c || !g) return QK_INVALID_ARGUMENT;
  for (int r = 0; r < g->world; r++)
    if (!g->peer_slots[r]) return QK_INVALID_ARGUMENT;
  cudaSetDevice(c->device);
  qk_gather_touch_kernel<<<1, 32>>>(peers_of(g));
  cudaError_t e = cudaGetLastError();
  if (e == cudaSuccess) e = cudaDeviceSynchronize();
  return e == cudaSuccess ? QK_OK : fail(c, e, "qk_gather_ready");
}

// Teardown is two steps with a host synchronisation of the ranks between them: freeing
// memory that another process still has open through an IPC handle is undefined, so
// every rank first closes what it imported, and only when all have done so does anyone
// free its own arrays.
extern "C" int qk_gather_close_peers(qk_ctx *c, qk_gather *g) {
  if (!c || !g) return QK_INVALID_ARGUMENT;
  cudaSetDevice(c->device);
  cudaDeviceSynchronize();  // none of this rank's kernels may still be storing into a peer
  for (int r = 0; r < g->world; r++) {
    if (r == g->rank) continue;
    if (g->opened[r]) cudaIpcCloseMemHandle(g->peer_slots[r]);
    g->peer_slots[r] = nullptr, g->opened[r] = false;
  }
  return QK_OK;
}

extern "C" int qk_gather_destroy(qk_ctx *c, qk_gather *g) {
  if (!c || !g) return QK_INVALID_ARGUMENT;
  qk_gather_close_peers(c, g);
  cudaFree(g->local), cudaFree(g->slots), cudaFree(g->ctl);
  delete g;
  return QK_OK;
}

extern "C" float *qk_gather_buffer(qk_gather *g) { return g ? g->local : nullptr; }

extern "C" int qk_gather_wait_dev(qk_ctx *c, qk_gather *g, void *stream) {
  if (!c || !g) return QK_INVALID_ARGUMENT;
  // rows of the result are ld apart and the call filled m of them: one contiguous run
  const uint64_t n = (uint64_t)g->last_m * g->world * g->rows;
  unsigned blocks = (unsigned)((n + 255) / 256);
  const unsigned cap = (unsigned)c->sm_count * 2u;
  if (blocks > cap) blocks = cap;
  cudaError_t e = launch_pdl(qk_gather_unpack_kernel, blocks, 256, (cudaStream_t)stream,
                             (const unsigned long long *)g->slots, (const unsigned *)(g->ctl + 1), g->local, n,
                             c->status_dev);
  return e == cudaSuccess ? QK_OK : fail(c, e, "qk_gather_wait_dev");
}

extern "C" int qk_gemm_gather_after_dev(qk_ctx *c, const qk_weights *h, const float *x_dev, size_t m, qk_gather *g,
                                        qk_gather *after, void *stream) {
  return qk_gemm_gather_unpack_dev(c, h, x_dev, m, g, after, nullptr, stream);
}

extern "C" int qk_gemm_gather_unpack_dev(qk_ctx *c, const qk_weights *h, const float *x_dev, size_t m, qk_gather *g,
                                         qk_gather *after, qk_gather *unpack, void *stream) {
  if (!c || !h || !x_dev || !g) return QK_INVALID_ARGUMENT;
  if (after && after->device != c->device) return QK_INVALID_ARGUMENT;
  if (unpack && (unpack->device != c->device || unpack == g)) return QK_INVALID_ARGUMENT;
  if (h->device != c->device || g->device != c->device) return QK_INVALID_ARGUMENT;
  if (h->L.rows != g->rows || m == 0 || m > g->m_cap) return QK_DIMENSION_MISMATCH;
  for (int r = 0; r < g->world; r++)
    if (!g->peer_slots[r]) {
      c->err = "qk_gemm_gather_dev: a rank's buffer has not been imported";
      return QK_INVALID_ARGUMENT;
    }
  cudaStream_t s = (cudaStream_t)stream;
  const uint64_t ldy = (uint64_t)g->world * g->rows;
  QkPeers peers = peers_of(g);
  float *mine = g->local + (size_t)g->rank * g->rows;
  const bool fused = !c->force_simple && m <= QK_GEMV_MAX_M && h->L.cols > 0 &&
                     qk_gemv_peer_supported(h->L, (uint32_t)m);
  if (after) {
    // Activations that are the gathered output of the latest call on `after`.  Where the
    // matvec kernel can, it reads them straight from `after`'s slots (x_dev must then lie
    // inside after's buffer, rows one buffer row apart); otherwise `after` is unpacked
    // first and the kernels read the plain buffer.
    const uint64_t ld_a = (uint64_t)after->world * after->rows, n_a = after->m_cap * ld_a;
    const ptrdiff_t off = x_dev - after->local;
    const bool inside = x_dev >= after->local && (uint64_t)off + (m - 1) * ld_a + h->L.cols <= n_a;
    const bool rows_ok = m == 1 || h->L.cols == ld_a;  // the plain kernels take rows `cols` apart
    if (inside && !rows_ok) {
      c->err = "qk_gemm_gather_after_dev: several activation rows inside a gathered buffer need cols == world * rows";
      return QK_DIMENSION_MISMATCH;
    }
    if (fused && inside && (off & 1) == 0 && (ld_a & 1) == 0) {
      peers.wait_slots = after->slots + off, peers.wait_epoch = after->ctl + 1, peers.wait_ld = ld_a;
    } else {
      int st = qk_gather_wait_dev(c, after, stream);
      if (st) return st;
    }
  }
  if (unpack) {
    if (fused) {  // the matvec kernel unpacks it while its first weight tiles are in flight
      peers.unpack_slots = unpack->slots, peers.unpack_epoch = unpack->ctl + 1, peers.unpack_out = unpack->local;
      peers.unpack_n = (uint64_t)unpack->last_m * unpack->world * unpack->rows;
    } else {
      int st = qk_gather_wait_dev(c, unpack, stream);
      if (st) return st;
    }
  }
  g->last_m = m;
  if (fused) {  // the matvec kernel itself stores into every rank
    const size_t need = qk_gemv_peer_scratch_bytes(h->L, (uint32_t)m);
    if (need > c->scratch_cap) {
      cudaError_t e = cudaDeviceSynchronize();
      if (e != cudaSuccess) return fail(c, e, "qk_gemm_gather_dev");
      cudaFree(c->scratch);
      c->scratch = nullptr, c->scratch_cap = 0;
      e = cudaMalloc(&c->scratch, need * 2);
      if (e != cudaSuccess) return fail(c, e, "qk_gemm_gather_dev");
      c->scratch_cap = need * 2;
    }
    cudaError_t e = qk_launch_gemv_peer(h->L, h->dev, x_dev, (uint32_t)m, ldy, c->status_dev, c->scratch,
                                        c->sm_count, s, &peers);
    return e == cudaSuccess ? QK_OK : fail(c, e, "qk_gemm_gather_dev");
  }
  // any other shape or format (an empty K included: zeros): the ordinary kernels write this
  // rank's block of the local plain buffer, then a push kernel stores it into every rank's slots
  int st = qk_gemm_dev(c, h, x_dev, mine, m, ldy, stream);
  if (st) return st;
  const uint64_t n = (uint64_t)m * g->rows;
  unsigned blocks = (unsigned)((n + 255) / 256);
  const unsigned cap = (unsigned)c->sm_count * 2u;
  if (blocks > cap) blocks = cap;
  cudaError_t e = launch_pdl(qk_gather_push_kernel, blocks, 256, s, peers, (const float *)mine, (uint32_t)m,
                             (uint32_t)g->rows, ldy);
  return e == cudaSuccess ? QK_OK : fail(c, e, "qk_gemm_gather_dev");
}

extern "C" int qk_gemm_gather_dev(qk_ctx *c, const qk_weights *h, const float *x_dev, size_t m, qk_gather *g,
                                  void *stream) {
  return qk_gemm_gather_after_dev(c, h, x_dev, m, g, nullptr, stream);
}
