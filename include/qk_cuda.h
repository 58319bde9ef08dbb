/*
 * qk_cuda.h — C ABI of the B200 (sm_100a) quantized dequant-dot backend.
 *
 * This is the boundary a binding for OxiLLaMa's `QuantKernel` trait links
 * against (crates/oxillama-quant/src/traits.rs:21-183 of the reference): the
 * first group of entry points takes plain host pointers and sizes exactly as
 * the trait methods take slices; the second group keeps weights resident on
 * the GPU and takes device pointers, for callers that own device memory.
 *
 * Conventions
 *  - Every function returns a qk_status; nothing throws or aborts.
 *  - The caller owns every buffer; the library keeps only what it allocated
 *    itself (contexts, uploaded weights, its own scratch).
 *  - `type` is the GGUF tensor type id (crates/oxillama-gguf/src/types.rs:70-125):
 *    Q4_0 = 2, Q8_0 = 8, Q2_K = 10, Q3_K = 11, Q4_K = 12, Q5_K = 13, Q6_K = 14, Q8_K = 15, IQ4_XS = 23.
 *  - A weight matrix is [n_rows = out_features][n_cols = in_features], stored as
 *    n_rows consecutive rows of ceil(n_cols / block_size) blocks in GGUF byte
 *    layout (reference/q4_k.rs:110-131).  A partial last block is legal; the
 *    columns past n_cols contribute nothing.
 *  - One context drives one GPU (one process per GPU); a context may be used
 *    from any thread, one call at a time.
 *  - There is no CPU fallback: without a usable CUDA device every compute
 *    entry point fails with QK_CUDA_ERROR.
 */
#ifndef QK_CUDA_H
#define QK_CUDA_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Status codes.  0..7 map one to one onto the variants of the reference's
 * QuantError (crates/oxillama-quant/src/error.rs:10-71); the rest are new. */
typedef enum qk_status {
  QK_OK = 0,
  QK_UNSUPPORTED_TYPE = 1,     /* QuantError::UnsupportedType */
  QK_BLOCK_SIZE_MISMATCH = 2,  /* QuantError::BlockSizeMismatch */
  QK_DIMENSION_MISMATCH = 3,   /* QuantError::DimensionMismatch */
  QK_KERNEL_ERROR = 4,         /* QuantError::KernelError */
  QK_BLOCK_COUNT_MISMATCH = 5, /* QuantError::BlockCountMismatch */
  QK_BUFFER_TOO_SMALL = 6,     /* QuantError::BufferTooSmall */
  QK_INTERNAL = 7,             /* QuantError::Internal */
  QK_CUDA_ERROR = 100,         /* a CUDA runtime call failed; see qk_last_error */
  QK_TIMEOUT = 101,            /* a bounded device-side wait ran out */
  QK_INVALID_ARGUMENT = 102    /* null pointer, bad handle, bad range */
} qk_status;

#define QK_TYPE_Q4_0 2
#define QK_TYPE_Q8_0 8
#define QK_TYPE_Q4_K 12
#define QK_TYPE_Q5_K 13 /* Q5_K, Q2_K, Q3_K, Q8_K: generic kernels only so far (exact, not tuned) */
#define QK_TYPE_Q2_K 10
#define QK_TYPE_Q3_K 11
#define QK_TYPE_Q8_K 15
#define QK_TYPE_Q6_K 14
#define QK_TYPE_IQ4_XS 23

typedef struct qk_ctx qk_ctx;         /* one GPU + its stream and scratch */
typedef struct qk_weights qk_weights; /* one weight matrix (or row shard) resident in HBM */

/* ---- context: stands where KernelDispatcher::new() stands (dispatch.rs:128-131) ---- */
int qk_init(int device, qk_ctx **out);
int qk_shutdown(qk_ctx *ctx);
/* Copies the text of the last error raised on this context (empty if none). */
int qk_last_error(qk_ctx *ctx, char *buf, size_t buf_len);

/* ---- trait getters: QuantKernel::{block_size, block_bytes, name} (traits.rs:175-182) ---- */
size_t qk_block_size(int type);   /* 0 for an unsupported type */
size_t qk_block_bytes(int type);  /* 0 for an unsupported type */
const char *qk_name(int type);    /* "Q4_0", "Q8_0", "Q2_K" .. "Q6_K", "Q8_K", "IQ4_XS", or NULL */

/* ================= host-pointer entry points (the trait methods) ================= */

/* QuantKernel::dequant_block (traits.rs:28; e.g. reference/q4_k.rs:52-102).
 * One block -> block_size f32 values, bit-identical to the scalar reference.
 * block_len < block_bytes or out_len < block_size -> QK_BUFFER_TOO_SMALL. */
int qk_dequant_block(qk_ctx *ctx, int type, const uint8_t *block, size_t block_len, float *out,
                     size_t out_len);

/* Whole-matrix form of the same arithmetic, block by block in order, padding
 * columns dropped: what the reference's MoE loader does with dequant_block
 * (crates/oxillama-arch/src/llama/model.rs:843-886).  out is [n_rows x n_cols]. */
int qk_dequant_matrix(qk_ctx *ctx, int type, const uint8_t *w, size_t w_len, size_t n_rows,
                      size_t n_cols, float *out, size_t out_len);

/* QuantKernel::gemv (traits.rs:40-45; e.g. reference/q4_k.rs:104-184).
 * y[0..n_rows) = W x; y is overwritten.  x_len < n_cols or y_len < n_rows ->
 * QK_DIMENSION_MISMATCH; w_len short -> QK_BUFFER_TOO_SMALL. */
int qk_gemv(qk_ctx *ctx, int type, const uint8_t *w, size_t w_len, size_t n_rows, size_t n_cols,
            const float *x, size_t x_len, float *y, size_t y_len);

/* QuantKernel::gemm (traits.rs:59-67; e.g. reference/q4_k.rs:186-201): m
 * independent gemvs.  x is [m x k] row-major, y is [m x n] row-major and is
 * overwritten; n = weight rows, k = weight columns. */
int qk_gemm(qk_ctx *ctx, int type, const uint8_t *w, size_t w_len, const float *x, size_t x_len,
            float *y, size_t y_len, size_t m, size_t n, size_t k);

/* QuantKernel::matvec_q8_fused (traits.rs:89-173; overrides reference/q4_k.rs:218-333,
 * reference/q6_k.rs:212-354; free function reference/q4_0.rs:159-232).
 * acts_q8 holds ceil(n_cols/32) Q8_0 blocks (34 bytes each, already quantized
 * by the caller); out[row] += dot.  ACCUMULATES. */
int qk_matvec_q8_fused(qk_ctx *ctx, int type, const uint8_t *w, size_t w_len,
                       const uint8_t *acts_q8, size_t acts_len, float *out, size_t out_len,
                       size_t n_rows, size_t n_cols);

/* quantize_f32_to_q8_0 (crates/oxillama-quant/src/quantize.rs:58-75,190-210).
 * n must be a multiple of 32 (else QK_DIMENSION_MISMATCH); out needs n/32*34 bytes. */
int qk_quantize_q8_0(qk_ctx *ctx, const float *x, size_t n, uint8_t *out, size_t out_len);

/* ---- the reference's second operator surface: GpuKernel (crates/oxillama-gpu) ---- */

/* GpuKernel::gemv(ctx, weight_bytes, input, output, rows, cols)
 * (crates/oxillama-gpu/src/kernels/mod.rs:91-106; per type e.g. kernels/q4_k.rs:170-195):
 * output[i] = sum_j weight[i][j] input[j], output overwritten.  Same arithmetic and element
 * order as qk_gemv, i.e. the CPU crate's (that crate's own host-side Q4_K / Q6_K dequant
 * orders elements differently, kernels/q4_k.rs:138-157, kernels/q6_k.rs:94-121; it is not
 * followed).  Checks in that implementation's order: output_len < rows, input_len < cols,
 * weight_len short: each is its GpuError::BufferSize { expected, got }, returned here as
 * QK_BUFFER_TOO_SMALL with "Buffer size mismatch: expected E, got G" in qk_last_error;
 * GpuError::UnsupportedType is QK_UNSUPPORTED_TYPE. */
int qk_gpu_gemv(qk_ctx *ctx, int type, const uint8_t *weight_bytes, size_t weight_len, const float *input,
                size_t input_len, float *output, size_t output_len, size_t rows, size_t cols);

/* Batched form, Y[b][r] = sum_c A[r][c] X[b][c] (kernels/batched_gemv.rs:36-50), with A
 * still quantised.  vectors_len must equal batch_size * cols exactly, as there. */
int qk_gpu_gemv_batched(qk_ctx *ctx, int type, const uint8_t *weight_bytes, size_t weight_len,
                        const float *vectors, size_t vectors_len, float *output, size_t output_len,
                        size_t rows, size_t cols, size_t batch_size);

/* The host-pointer calls above keep the device copy of a weight matrix they
 * have seen, keyed by (pointer, length, type, shape) — weights are immutable
 * after load in the reference (llama/model.rs:805-822).  Call this before
 * reusing or rewriting that host memory.  w == NULL drops everything. */
int qk_weights_cache_evict(qk_ctx *ctx, const uint8_t *w);

/* ================= device-resident entry points (new; no reference counterpart) ================= */

/* Uploads rows [row_begin, row_end) of a [n_rows x n_cols] matrix (a row shard;
 * pass 0, n_rows for the whole matrix) and re-tiles them for the kernels. */
int qk_weights_upload(qk_ctx *ctx, int type, const uint8_t *w, size_t w_len, size_t n_rows,
                      size_t n_cols, size_t row_begin, size_t row_end, qk_weights **out);
int qk_weights_free(qk_ctx *ctx, qk_weights *h);
/* Shard shape: rows held, columns, and the algorithmic bytes of the shard
 * (rows * ceil(cols/block_size) * block_bytes). */
int qk_weights_info(const qk_weights *h, int *type, size_t *rows, size_t *cols, size_t *bytes);

/* ---- GGUF file -> device (new; stands where load_quant_linear copies tensor_data(name) into a
 * QuantTensor, crates/oxillama-arch/src/llama/model.rs:805-822) ---- */
typedef struct qk_gguf qk_gguf;
/* Parses header, metadata (only general.alignment is kept) and tensor infos of a GGUF v1-v3
 * file (crates/oxillama-gguf/src/parser.rs:34-60, 166-212); tensor data is not read.  *out is
 * set even when parsing fails, so that qk_gguf_last_error can say why: close it either way. */
int qk_gguf_open(const char *path, qk_gguf **out);
int qk_gguf_close(qk_gguf *g);
int qk_gguf_last_error(const qk_gguf *g, char *buf, size_t buf_len);
int qk_gguf_tensor_count(const qk_gguf *g, size_t *n);
int qk_gguf_tensor_name(const qk_gguf *g, size_t index, char *buf, size_t buf_len);
/* type = GGUF type id; dims in file order, unused ones 1; file_offset absolute; nbytes =
 * TensorInfo::data_size (tensor_info.rs:47-56), 0 for a type this library does not serve. */
int qk_gguf_tensor_info(const qk_gguf *g, const char *name, int *type, size_t *n_dims, uint64_t dims[4],
                        uint64_t *file_offset, uint64_t *nbytes);
/* qk_weights_upload of rows [row_begin, row_end) of the named tensor, rows = dimensions[0] and
 * columns = dimensions[1] as the reference reads them, straight from the file: the row range
 * is one contiguous byte range, read through pinned staging buffers, never copied into
 * pageable memory.  Unknown name: QK_INVALID_ARGUMENT; a type this library does not
 * serve: QK_UNSUPPORTED_TYPE; data past the end of the file: QK_BUFFER_TOO_SMALL. */
int qk_weights_upload_gguf(qk_ctx *ctx, const qk_gguf *g, const char *name, size_t row_begin, size_t row_end,
                           qk_weights **out);

/* y_dev[0..rows) = W_shard x_dev.  Device pointers; enqueued on `stream`
 * (a cudaStream_t; NULL is the legacy default stream); returns without waiting. */
int qk_gemv_dev(qk_ctx *ctx, const qk_weights *h, const float *x_dev, float *y_dev, void *stream);

/* y_dev[i*ldy + j] = dot(W_shard row j, x_dev row i), i < m, j < rows.  x_dev is
 * [m x cols] row-major.  ldy >= rows lets a row shard write its column block of
 * a wider [m x n] output in place. */
int qk_gemm_dev(qk_ctx *ctx, const qk_weights *h, const float *x_dev, float *y_dev, size_t m,
                size_t ldy, void *stream);

/* The dense feed-forward block around the path (new as one call; the reference's
 * feed_forward does it as three QuantLinear::forward calls and swiglu_inplace,
 * crates/oxillama-arch/src/llama/model.rs:281-310, crates/oxillama-arch/src/common/swiglu.rs:15-21):
 *   y_dev[i][:] = down( silu(gate x_i) * (up x_i) ),  i < m,  x_dev [m x hidden], y_dev [m x down rows].
 * gate and up are [inter x hidden], down is [rows x inter].  For Q4_K gate / up and m <= 4 the
 * two projections run as one launch over both matrices (they share the split activations) and
 * silu(g) * u is formed where the dot products are reduced, so neither g nor u is ever
 * written out; otherwise the three matmuls and an element-wise pass are enqueued in turn.
 * Keeps its own scratch for the hidden activations, grown on first use. */
int qk_ffn_dev(qk_ctx *ctx, const qk_weights *gate, const qk_weights *up, const qk_weights *down,
               const float *x_dev, float *y_dev, size_t m, void *stream);

/* out_dev[rows x cols] f32 = dequantised shard, bit-identical to dequant_block. */
int qk_dequant_dev(qk_ctx *ctx, const qk_weights *h, float *out_dev, void *stream);

/* out_dev[row] += dot with already-quantised Q8_0 activations on the device. */
int qk_matvec_q8_fused_dev(qk_ctx *ctx, const qk_weights *h, const uint8_t *acts_q8_dev,
                           float *out_dev, void *stream);

/* Q8_0 activation encoder on device memory; n a multiple of 32. */
int qk_quantize_q8_0_dev(qk_ctx *ctx, const float *x_dev, size_t n, uint8_t *out_dev, void *stream);

/* ---- mixture-of-experts FFN: MoeFfn::forward (crates/oxillama-arch/src/common/moe.rs:184-258) ---- */

/* Routing alone (moe.rs:200-248): per token the softmax over all n_exp logits, the
 * top_k experts in descending order of probability (ties to the lower expert id) and
 * their weights renormalised by the selected sum.  ids_dev / wts_dev are
 * [tokens x top_k]; with top_k > n_exp the extra slots get id -1 and weight 0. */
int qk_moe_route_dev(qk_ctx *ctx, const float *logits_dev, size_t tokens, size_t n_exp, size_t top_k,
                     int *ids_dev, float *wts_dev, void *stream);

/* y_dev[tokens x hidden] = sum over the n_local experts held here (global ids
 * expert_begin .. expert_begin + n_local) of  w(token, e) * down_e(silu(gate_e x) * up_e x)
 * for the tokens routed to them (Expert::forward, moe.rs:75-126); y_dev is overwritten.
 * gate[e], up[e] are [inter x hidden] shards, down[e] is [hidden x inter].  With every
 * expert local this is MoeFfn::forward given the router's logits; an expert-sharded
 * layer sums the y of its ranks.  logits_dev is [tokens x n_exp], x_dev [tokens x hidden].
 * More than 16 tokens, at most 16 local experts of one format: every projection is one
 * grouped matmul launch over all local experts, the per-expert token counts stay on the
 * device and the call does not synchronise (a fixed sequence of launches on `stream`).
 * Otherwise (decode-sized calls) the experts run one after the other on the decode kernels
 * and the call synchronises `stream` once to read the counts that size them.  The context
 * keeps the device scratch, grown (with a device synchronise) on first use of a larger size. */
int qk_moe_ffn_dev(qk_ctx *ctx, const qk_weights *const *gate, const qk_weights *const *up,
                   const qk_weights *const *down, size_t n_local, size_t expert_begin, size_t n_exp,
                   const float *logits_dev, const float *x_dev, float *y_dev, size_t tokens,
                   size_t top_k, void *stream);

/* ---- token exchange for an expert-sharded layer whose ranks each own their own tokens ---- */
/* (new; stands where a multi-process port of MoeFfn::forward, moe.rs:184-258, would send each
 * token's row to the ranks that hold its selected experts and take their partial outputs back) */

/* out_dev[i][:] = x_dev[idx_dev[i]][:] for i < n: rows of `width` floats, packed in send order. */
int qk_moe_take_rows_dev(qk_ctx *ctx, const float *x_dev, const int *idx_dev, size_t n, size_t width,
                         float *out_dev, void *stream);

/* y_dev[t][:] = +0 + src_dev[idx_dev[t][0]][:] + src_dev[idx_dev[t][1]][:] + ..., added in that
 * order, negative entries skipped; idx_dev is [tokens x per_row].  The partial outputs that came
 * back for a token are summed in the order of the ranks that computed them, the same on every run. */
int qk_moe_sum_rows_dev(qk_ctx *ctx, const float *src_dev, const int *idx_dev, size_t tokens, size_t per_row,
                        size_t width, float *y_dev, void *stream);

/* ---- row-sharded layers on the GPUs of one node: outputs gathered by peer stores ---- */
/* (new; stands where a sharded port of QuantLinear::forward would call an all-gather,
 * crates/oxillama-arch/src/common/linear.rs:77-132) */
typedef struct qk_gather qk_gather;

/* This rank's gathered [m_cap x world * rows_per_rank] f32 result and, behind it, an array
 * of 8-byte (value, tag) slots of the same shape that every rank stores into.  world <= 8.
 * The ranks then exchange qk_gather_export handles (128 bytes each) over any host channel
 * and qk_gather_import each other's (ranks that live in one process: qk_gather_import_local). */
int qk_gather_create(qk_ctx *ctx, size_t rows_per_rank, size_t m_cap, int world, int rank, qk_gather **out);
int qk_gather_export(qk_ctx *ctx, qk_gather *g, unsigned char *handle, size_t handle_len);
int qk_gather_import(qk_ctx *ctx, qk_gather *g, int peer_rank, const unsigned char *handle, size_t handle_len);
int qk_gather_import_local(qk_ctx *ctx, qk_gather *g, int peer_rank, qk_gather *peer);
/* Once every rank's handle is imported: touches each peer mapping and waits.  Every rank
 * calls it, then the ranks synchronise on the host, before the first sharded call. */
int qk_gather_ready(qk_ctx *ctx, qk_gather *g);
/* Teardown, in two steps: every rank calls qk_gather_close_peers (waits for this GPU's
 * work, closes what it imported), the ranks synchronise on the host, then every rank
 * calls qk_gather_destroy.  Freeing memory that a peer still has open is undefined. */
int qk_gather_close_peers(qk_ctx *ctx, qk_gather *g);
int qk_gather_destroy(qk_ctx *ctx, qk_gather *g);
/* Device pointer of the plain result: y_full[i * world * rows_per_rank + r * rows_per_rank + j],
 * valid once a qk_gather_wait_dev enqueued after the call has run. */
float *qk_gather_buffer(qk_gather *g);

/* qk_gemm_dev of this rank's shard (rows == rows_per_rank), with the [m x rows] result
 * stored into the slots of every rank, tagged with the call's ordinal on this qk_gather.
 * Where the decode kernel supports it (Q4_K, m <= 4) the kernel itself does the peer
 * stores; otherwise a push kernel follows the ordinary one.  Every rank must make the same
 * sequence of calls on a given qk_gather.  A call overwrites the slots of the previous
 * call on the same object in every rank, so a rank may start call k + 1 on an object only
 * when every rank has finished reading call k from it.  Two objects used alternately, each
 * call waiting (qk_gather_wait_dev, or `after` below) for the previous call before it
 * starts, satisfy this: a rank that has seen every block of call k knows that all ranks
 * have finished reading call k - 1.  Ranks that let a call run ahead of the wait for the
 * previous one (waiting one call later) need four objects in rotation. */
int qk_gemm_gather_dev(qk_ctx *ctx, const qk_weights *h, const float *x_dev, size_t m, qk_gather *g, void *stream);
/* The same, for activations that are themselves gathered: x_dev points into
 * qk_gather_buffer(after) (activation rows one buffer row apart) and stands for the result
 * of the latest call on `after`.  Where the matvec kernel does the peer stores it also reads
 * x straight from `after`'s slots, each read waiting until the slot carries that call's tag
 * (no unpacking pass, no kernel boundary between the arrival of the data and its use);
 * otherwise qk_gather_wait_dev(after) is enqueued first.  after == NULL: plain x_dev. */
int qk_gemm_gather_after_dev(qk_ctx *ctx, const qk_weights *h, const float *x_dev, size_t m, qk_gather *g,
                             qk_gather *after, void *stream);
/* The same, and in passing the latest call on `unpack` (another object, not g) is unpacked
 * into its plain buffer as qk_gather_wait_dev would do, by the matvec kernel itself while
 * its first weight tiles are on their way (where the matvec kernel does the peer stores;
 * otherwise qk_gather_wait_dev(unpack) is enqueued first).  A decode loop that wants every
 * gathered result in plain memory passes the previous call's object here and pays neither
 * a kernel nor a gap between two matvecs for it.  after and unpack may be NULL. */
int qk_gemm_gather_unpack_dev(qk_ctx *ctx, const qk_weights *h, const float *x_dev, size_t m, qk_gather *g,
                              qk_gather *after, qk_gather *unpack, void *stream);
/* Enqueues the unpacking of the latest call into the plain buffer: every slot is waited
 * for (at most 0.25 s per thread, then QK_TIMEOUT through qk_check_device_status and
 * zeros in the places that did not arrive). */
int qk_gather_wait_dev(qk_ctx *ctx, qk_gather *g, void *stream);

/* No counterpart in the reference.  qk_gemm_dev for Q4_K shards and m <= 4 that
 * allocates nothing: for callers that cannot allocate device memory once running
 * (a server that handed all of HBM to its own pools, a process under a fixed
 * memory budget, a loop that must not take the allocator lock).  Its scratch is
 * a 96 KiB array built into the library (held on every GPU that loads it), so
 * the split activations of a call (about 3.1 bytes per activation) must fit
 * 96 KiB, else QK_INVALID_ARGUMENT.  Like every *_dev entry point it launches on the
 * calling thread's current device, which must be the context's.
 * The first call on a device resolves the array's address: make it before any
 * stream capture.  Calls on one device share the array; overlapping calls race. */
int qk_gemm_dev_noalloc(qk_ctx *ctx, const qk_weights *h, const float *x_dev, float *y_dev,
                        size_t m, size_t ldy, void *stream);

/* Reads and clears the device-side status word of the context (bounded waits
 * that ran out, range checks that tripped).  Synchronises `stream`. */
int qk_check_device_status(qk_ctx *ctx, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* QK_CUDA_H */
