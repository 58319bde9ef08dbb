// Q4_K decode matvec (1..4 activation rows): the Q4_K instantiation of the integer-MMA
// decode kernel (qk_gemv_skel.cuh with the policy of qk_dec_q4k.cuh), plus the route that
// always takes its split activations from a caller-provided image.
#include "qk_dec_q4k.cuh"

using namespace qkdec;

#ifdef QK_TRACE
__device__ unsigned long long *qk_trace_buf = nullptr;
extern "C" void qk_trace_set(unsigned long long *p) {
  cudaMemcpyToSymbol(qk_trace_buf, &p, sizeof(p));
}
#endif

bool qk_gemv_mma_supported(const QkLayout &L, uint32_t m) {
  return L.type == QK_T_Q4_K && supported<DecQ4K>(L, m);
}

size_t qk_gemv_mma_scratch_bytes(const QkLayout &L, uint32_t m) { return scratch_bytes<DecQ4K>(L, m); }

cudaError_t qk_launch_gemv_mma(const QkLayout &L, const uint8_t *tiled, const float *x, float *y,
                               uint32_t m, uint64_t ldy, unsigned *status, unsigned char *scratch,
                               int sm_count, cudaStream_t s, const QkPeers *peers) {
  return launch<DecQ4K>(L, tiled, x, y, m, ldy, status, scratch, sm_count, s, peers);
}

// Gate and up projection of a feed-forward block in one launch: h[i][j] = silu(gate_j . x_i) * (up_j . x_i).
bool qk_gemv_dual_supported(const QkLayout &L, uint32_t m) { return qk_gemv_mma_supported(L, m); }

cudaError_t qk_launch_gemv_dual(const QkLayout &L, const uint8_t *gate_tiled, const uint8_t *up_tiled, const float *x,
                                float *h, uint32_t m, uint64_t ldh, unsigned *status, unsigned char *scratch,
                                int sm_count, cudaStream_t s) {
  return launch<DecQ4K>(L, gate_tiled, x, h, m, ldh, status, scratch, sm_count, s, nullptr, up_tiled);
}

// Same matvec, always through qk_xsplit_kernel + the x image in `scratch` (never the
// in-CTA split), for callers that hand in their own scratch.
cudaError_t qk_launch_gemv_mma_split(const QkLayout &L, const uint8_t *tiled, const float *x,
                                     float *y, uint32_t m, uint64_t ldy, unsigned *status,
                                     unsigned char *scratch, int sm_count, cudaStream_t s) {
  PlanMma P;
  if (!make_plan_mma(L, m, &P, DecQ4K::XSB, true)) return cudaErrorInvalidConfiguration;
#define QK_SPLIT(MV)                                                                                       \
  switch (P.groups) {                                                                                      \
    case 4:                                                                                                \
      return launch_mma<DecQ4K, MV, false, 8, 4>(L, tiled, x, y, ldy, status, scratch, sm_count, P, s);   \
    case 2:                                                                                                \
      return launch_mma<DecQ4K, MV, false, 8, 2>(L, tiled, x, y, ldy, status, scratch, sm_count, P, s);   \
    default:                                                                                               \
      return launch_mma<DecQ4K, MV, false, 8, 1>(L, tiled, x, y, ldy, status, scratch, sm_count, P, s);   \
  }
  switch (m) {
    case 1:
      QK_SPLIT(1)
    case 2:
      QK_SPLIT(2)
    case 3:
      QK_SPLIT(3)
    default:
      QK_SPLIT(4)
  }
#undef QK_SPLIT
}
