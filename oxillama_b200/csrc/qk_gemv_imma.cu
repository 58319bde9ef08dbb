// Decode matvec (1..4 activation rows) for Q8_0, Q4_0, IQ4_XS and Q6_K: the instantiations
// of the integer-MMA decode kernel (qk_gemv_skel.cuh) with the policies of qk_dec_fmts.cuh
// live in qk_dec_<format>.cu; this is the per-type dispatch of the decode path.
#include "qk_kernels.h"

// per-format entry points (qk_dec_<format>.cu)
#define QK_DEC_DECLARE(NAME)                                                                                    \
  bool qk_dec_##NAME##_supported(const QkLayout &L, uint32_t m);                                                \
  size_t qk_dec_##NAME##_scratch(const QkLayout &L, uint32_t m);                                                \
  cudaError_t qk_dec_##NAME##_launch(const QkLayout &L, const uint8_t *tiled, const float *x, float *y,         \
                                     uint32_t m, uint64_t ldy, unsigned *status, unsigned char *scratch,        \
                                     int sm_count, cudaStream_t s, const QkPeers *peers);
QK_DEC_DECLARE(q80)
QK_DEC_DECLARE(q40)
QK_DEC_DECLARE(iq4xs)
QK_DEC_DECLARE(q6k)

#define QK_BY_TYPE(L, call_q4k, call)            \
  switch ((L).type) {                            \
    case QK_T_Q4_K:                              \
      return call_q4k;                           \
    case QK_T_Q8_0:                              \
      return call(q80);                          \
    case QK_T_Q4_0:                              \
      return call(q40);                          \
    case QK_T_IQ4_XS:                            \
      return call(iq4xs);                        \
    case QK_T_Q6_K:                              \
      return call(q6k);                          \
    default:                                     \
      break;                                     \
  }

bool qk_gemv_fast_supported(const QkLayout &L, uint32_t m) {
  if (m < 1 || m > QK_GEMV_MAX_M) return false;
#define CALL(F) qk_dec_##F##_supported(L, m)
  QK_BY_TYPE(L, qk_gemv_mma_supported(L, m), CALL)
#undef CALL
  return false;
}

size_t qk_gemv_fast_scratch_bytes(const QkLayout &L, uint32_t m) {
#define CALL(F) qk_dec_##F##_scratch(L, m)
  QK_BY_TYPE(L, qk_gemv_mma_scratch_bytes(L, m), CALL)
#undef CALL
  return 0;
}

cudaError_t qk_launch_gemv_fast(const QkLayout &L, const uint8_t *tiled, const float *x, float *y,
                                uint32_t m, uint64_t ldy, unsigned *status, unsigned char *scratch,
                                int sm_count, cudaStream_t s) {
#define CALL(F) qk_dec_##F##_launch(L, tiled, x, y, m, ldy, status, scratch, sm_count, s, nullptr)
  QK_BY_TYPE(L, qk_launch_gemv_mma(L, tiled, x, y, m, ldy, status, scratch, sm_count, s), CALL)
#undef CALL
  return cudaErrorNotSupported;
}

// ---- the same kernels with the output fan-out of a row-sharded layer built in
bool qk_gemv_peer_supported(const QkLayout &L, uint32_t m) { return qk_gemv_fast_supported(L, m); }

size_t qk_gemv_peer_scratch_bytes(const QkLayout &L, uint32_t m) { return qk_gemv_fast_scratch_bytes(L, m); }

cudaError_t qk_launch_gemv_peer(const QkLayout &L, const uint8_t *tiled, const float *x, uint32_t m,
                                uint64_t ldy, unsigned *status, unsigned char *scratch, int sm_count,
                                cudaStream_t s, const QkPeers *peers) {
#define CALL(F) qk_dec_##F##_launch(L, tiled, x, nullptr, m, ldy, status, scratch, sm_count, s, peers)
  QK_BY_TYPE(L, qk_launch_gemv_mma(L, tiled, x, nullptr, m, ldy, status, scratch, sm_count, s, peers), CALL)
#undef CALL
  return cudaErrorNotSupported;
}
