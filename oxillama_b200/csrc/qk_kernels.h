// Internal launch interface between the C-ABI layer and the kernel translation units.
#pragma once
#include <cstdlib>

#include "qk_layout.cuh"

// Developer knobs (environment variables that change ring depths, warp counts and the like)
// exist only in builds made with -DQK_DEV_KNOBS; the default build never reads the
// environment, so nothing outside the caller's arguments changes what a call computes.
static inline const char *qk_knob(const char *name) {
#ifdef QK_DEV_KNOBS
  return getenv(name);
#else
  (void)name;
  return nullptr;
#endif
}

// A flag per CUDA device: function attributes (e.g. the dynamic shared-memory limit) and
// occupancy figures belong to a device, and one process may drive several.
struct QkPerDevice {
  bool done[64] = {};
  // true the first time it is asked on the current device
  bool first() {
    int d = 0;
    if (cudaGetDevice(&d) != cudaSuccess || d < 0 || d >= 64) return true;
    if (done[d]) return false;
    done[d] = true;
    return true;
  }
  void reset() {  // the first-time work failed: try again on the next call
    int d = 0;
    if (cudaGetDevice(&d) == cudaSuccess && d >= 0 && d < 64) done[d] = false;
  }
};

// Device status word bits (read back by qk_check_device_status).
#define QK_DEV_TIMEOUT 1u
#define QK_DEV_BOUNDS 2u

// raw_dev: GGUF-layout bytes of rows [0, L.rows) of the shard; tiled_dev: L.total_bytes, zeroed.
cudaError_t qk_launch_repack(const QkLayout &L, const uint8_t *raw_dev, uint8_t *tiled_dev,
                             cudaStream_t s);
cudaError_t qk_launch_dequant(const QkLayout &L, const uint8_t *tiled, float *out, cudaStream_t s);
// Generic any-shape path: f32 dequant in registers, f32 FMA, one warp per weight row.
cudaError_t qk_launch_gemm_simple(const QkLayout &L, const uint8_t *tiled, const float *x, float *y,
                                  uint32_t m, uint64_t ldy, cudaStream_t s);
cudaError_t qk_launch_fused_simple(const QkLayout &L, const uint8_t *tiled, const uint8_t *acts,
                                   float *out, cudaStream_t s);
cudaError_t qk_launch_quantize_q8_0(const float *x, uint64_t n, uint8_t *out, cudaStream_t s);

// Output fan-out of a row-sharded matvec.  Every rank of the node owns a buffer of 8-byte
// slots, one per output element of the gathered [m x world * rows] result: the f32 value in
// the low half, the call's tag (its ordinal on that buffer, from 1) in the high half.  The
// kernel that computes a result stores the pair, as one 64-bit word, into the slot of every
// rank (plain peer stores over NVLink; entry `rank` is the local buffer).  A naturally
// aligned 64-bit store is single-copy atomic, so a reader that sees the tag it expects has
// the value that belongs to it: no fence, flag or counter stands between the data and its
// consumer, and nothing waits for a peer's acknowledgement.  n == 0: ordinary local output.
#define QK_MAX_PEERS 8
struct QkPeers {
  unsigned long long *slots[QK_MAX_PEERS];  // each rank's slot array, already offset to this rank's columns
  unsigned *counter;                        // local: CTAs of this launch counted in (returns to 0)
  unsigned *epoch;                          // local: calls issued so far on this buffer (the latest tag)
  uint32_t n, rank;
  // optional: the activations are the gathered output of an earlier sharded call and are
  // read straight from its slots, each read waiting (bounded) for the tag *wait_epoch
  const unsigned long long *wait_slots;     // slot of x[0][0]; row stride = wait_ld slots
  const unsigned *wait_epoch;
  uint64_t wait_ld;
  // optional: while its first weight tiles are on their way the kernel also unpacks the
  // latest call of another gather object (unpack_n slots, each waited for with a bound, tag
  // *unpack_epoch) into that object's plain buffer: the gather's completion costs no kernel
  // of its own and no gap between two matvecs
  const unsigned long long *unpack_slots;
  const unsigned *unpack_epoch;
  float *unpack_out;
  uint64_t unpack_n;
};

// Bandwidth-bound decode path (m <= QK_GEMV_MAX_M): bulk-copied tiles, integer dot.
#define QK_GEMV_MAX_M 4
bool qk_gemv_fast_supported(const QkLayout &L, uint32_t m);
// Q4_K decode path on the integer tensor-core MMA (m16n8k32 u8 x s8).  `scratch`
// is device memory of at least qk_gemv_mma_scratch_bytes(L, m) bytes, 16-byte
// aligned, that the call may overwrite (the split activations live there
// between its two kernels).
bool qk_gemv_mma_supported(const QkLayout &L, uint32_t m);
size_t qk_gemv_mma_scratch_bytes(const QkLayout &L, uint32_t m);
cudaError_t qk_launch_gemv_mma(const QkLayout &L, const uint8_t *tiled, const float *x, float *y,
                               uint32_t m, uint64_t ldy, unsigned *status, unsigned char *scratch,
                               int sm_count, cudaStream_t s, const QkPeers *peers = nullptr);
cudaError_t qk_launch_gemv_mma_split(const QkLayout &L, const uint8_t *tiled, const float *x,
                                     float *y, uint32_t m, uint64_t ldy, unsigned *status,
                                     unsigned char *scratch, int sm_count, cudaStream_t s);
// Decode kernels that can store their results into every rank's tagged slots themselves
// (and read gathered activations out of slots): `peers` as described at QkPeers.
bool qk_gemv_peer_supported(const QkLayout &L, uint32_t m);
size_t qk_gemv_peer_scratch_bytes(const QkLayout &L, uint32_t m);
cudaError_t qk_launch_gemv_peer(const QkLayout &L, const uint8_t *tiled, const float *x, uint32_t m,
                                uint64_t ldy, unsigned *status, unsigned char *scratch, int sm_count,
                                cudaStream_t s, const QkPeers *peers);
// Gate and up projection of a feed-forward block in one launch (two matrices of the same
// shape and format, Q4_K): h[i * ldh + j] = silu(gate_j . x_i) * (up_j . x_i).  Scratch as
// qk_gemv_mma_scratch_bytes.
bool qk_gemv_dual_supported(const QkLayout &L, uint32_t m);
cudaError_t qk_launch_gemv_dual(const QkLayout &L, const uint8_t *gate_tiled, const uint8_t *up_tiled, const float *x,
                                float *h, uint32_t m, uint64_t ldh, unsigned *status, unsigned char *scratch,
                                int sm_count, cudaStream_t s);
size_t qk_gemv_fast_scratch_bytes(const QkLayout &L, uint32_t m);
cudaError_t qk_launch_gemv_fast(const QkLayout &L, const uint8_t *tiled, const float *x, float *y,
                                uint32_t m, uint64_t ldy, unsigned *status, unsigned char *scratch,
                                int sm_count, cudaStream_t s);

// Small batches (1 .. 16 rows) of Q4_K on the fp16 mma.sync with the decode path's streaming
// structure.  `scratch`: qk_gemm_sb_scratch_bytes(L, m) bytes.  _preferred: the shapes where
// it was measured faster than the tcgen05 kernel (5 .. 16 rows, at least eight chunks per SM).
bool qk_gemm_sb_supported(const QkLayout &L, uint32_t m);
bool qk_gemm_sb_preferred(const QkLayout &L, uint32_t m, int sm_count);
size_t qk_gemm_sb_scratch_bytes(const QkLayout &L, uint32_t m);
cudaError_t qk_launch_gemm_sb(const QkLayout &L, const uint8_t *tiled, const float *x, float *y, uint32_t m,
                              uint64_t ldy, unsigned *status, unsigned char *scratch, int sm_count, cudaStream_t s);

// Q4_K batched matmul on tcgen05 / TMEM (any m; used for m > QK_GEMV_MAX_M).  `scratch`
// holds the fp16 copy of the activations: qk_gemm_tc_scratch_bytes(L, m) bytes.
bool qk_gemm_tc_supported(const QkLayout &L, uint32_t m);

// Grouped form (mixture-of-experts projections): `n` weight matrices of one shape and format,
// group e multiplying its own activation rows [e * cap, e * cap + counts[e]) (counts on the
// device: no host round trip sizes the launch) into output rows of the same numbers.
// Optionally the activation rows are gathered on the fly: row (e, i) = x[lists[e * list_stride
// + i] / list_div].  One conversion launch and one matmul launch for all groups.
#define QK_MAX_GROUPS 16
struct QkGroups {
  uint32_t n;                        // 0: one matrix (the ordinary call)
  uint32_t n_act;                    // groups e and e + n_act read the same activation rows (gate and up of an expert)
  uint32_t rbpg, tbpg;               // 128-row blocks and token blocks per group
  const int *counts;                 // device: valid activation rows per group
  const uint8_t *w[QK_MAX_GROUPS];   // each group's tiled weights
};
uint32_t qk_gemm_tc_group_cap(uint32_t max_rows_per_group);  // activation rows reserved per group
size_t qk_gemm_tc_grouped_scratch_bytes(const QkLayout &L, uint32_t n_groups, uint32_t max_rows_per_group);
// n_act: number of distinct activation groups (n_groups a multiple of it; counts_dev, x and the
// lists describe n_act groups, y holds n_groups * cap rows: group e + k n_act multiplies the
// activations of group e).
cudaError_t qk_launch_gemm_tc_grouped(const QkLayout &L, const uint8_t *const *tiled, uint32_t n_groups, uint32_t n_act,
                                      const int *counts_dev, uint32_t max_rows_per_group, const float *x,
                                      const int *lists, uint32_t list_stride, uint32_t list_div, float *y,
                                      uint64_t ldy, unsigned *status, unsigned char *scratch, int sm_count,
                                      cudaStream_t s);
size_t qk_gemm_tc_scratch_bytes(const QkLayout &L, uint32_t m);
cudaError_t qk_launch_gemm_tc(const QkLayout &L, const uint8_t *tiled, const float *x, float *y,
                              uint32_t m, uint64_t ldy, unsigned *status, unsigned char *scratch,
                              int sm_count, cudaStream_t s);

// Mixture-of-experts glue (routing, token lists, gather, silu * up, weighted scatter-add).
cudaError_t qk_launch_moe_route(const float *logits, uint32_t tokens, uint32_t n_exp, uint32_t top_k,
                                int *ids, float *wts, cudaStream_t s);
cudaError_t qk_launch_moe_lists(const int *ids, uint32_t tokens, uint32_t top_k, uint32_t expert_begin,
                                uint32_t n_local, int *counts, int *lists, int *pos, cudaStream_t s);
cudaError_t qk_launch_moe_silu_mul_grouped(const float *g, float *u, const int *counts, uint32_t n_local,
                                           uint32_t max_rows, uint32_t cap, uint32_t inter, cudaStream_t s);
cudaError_t qk_launch_moe_combine(const float *o, const int *ids, const int *pos, const float *wts, uint32_t tokens,
                                  uint32_t top_k, uint32_t expert_begin, uint32_t n_local, uint32_t cap,
                                  uint32_t hidden, float *y, cudaStream_t s);
cudaError_t qk_launch_moe_gather(const float *x, const int *list, uint32_t n, uint32_t top_k,
                                 uint32_t hidden, float *xe, cudaStream_t s);
cudaError_t qk_launch_moe_silu_mul(const float *g, float *u, uint64_t n, cudaStream_t s);
// g <- silu(g) * u (swiglu_inplace of the dense feed-forward block)
cudaError_t qk_launch_swiglu(float *g, const float *u, uint64_t n, cudaStream_t s);
cudaError_t qk_launch_moe_scatter(const float *o, const int *list, const float *wts, uint32_t n,
                                  uint32_t top_k, uint32_t hidden, float *y, cudaStream_t s);
cudaError_t qk_launch_moe_take_rows(const float *x, const int *idx, uint32_t n, uint32_t width, float *out,
                                    cudaStream_t s);
cudaError_t qk_launch_moe_sum_rows(const float *src, const int *idx, uint32_t tokens, uint32_t per_row,
                                   uint32_t width, float *y, cudaStream_t s);
