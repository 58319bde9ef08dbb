// Device helpers of the tagged-slot gather (see QkPeers in qk_kernels.h): 64-bit
// (value, tag) slots written with one store and polled with one load.
#pragma once
#include <cstdint>

namespace qkpeer {

__device__ __forceinline__ void slot_store(unsigned long long *p, float v, unsigned tag) {
  const unsigned long long w = ((unsigned long long)tag << 32) | (unsigned long long)__float_as_uint(v);
#if defined(QK_SLOT_NONE)
  (void)p, (void)w;
#elif defined(QK_SLOT_WEAK)
  asm volatile("st.global.u64 [%0], %1;" ::"l"(p), "l"(w) : "memory");
#else
  asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(p), "l"(w) : "memory");
#endif
}
__device__ __forceinline__ unsigned long long slot_load(const unsigned long long *p) {
  unsigned long long w;
  asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(w) : "l"(p) : "memory");
  return w;
}
__device__ __forceinline__ void slot_load2(const unsigned long long *p, unsigned long long &a,
                                           unsigned long long &b) {  // p 16-byte aligned
  asm volatile("ld.relaxed.sys.global.v2.u64 {%0,%1}, [%2];" : "=l"(a), "=l"(b) : "l"(p) : "memory");
}
__device__ __forceinline__ unsigned long long now_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
constexpr unsigned long long WAIT_NS = 250000000ull;  // a quarter of a second

// Value of one slot once its tag is `want`; false (and v = 0) if it has not arrived in time.
__device__ __forceinline__ bool slot_wait(const unsigned long long *p, unsigned want, float &v) {
  unsigned long long w = slot_load(p);
  if ((unsigned)(w >> 32) != want) {
    const unsigned long long t0 = now_ns();
    do {
      w = slot_load(p);
      if ((unsigned)(w >> 32) == want) break;
      if (now_ns() - t0 > WAIT_NS) {
        v = 0.f;
        return false;
      }
    } while (true);
  }
  v = __uint_as_float((unsigned)w);
  return true;
}

// Four consecutive slots (p 16-byte aligned) -> four values, each once its tag is `want`.
__device__ __forceinline__ bool slot_wait4(const unsigned long long *p, unsigned want, float (&v)[4]) {
  unsigned long long w[4];
  slot_load2(p, w[0], w[1]);
  slot_load2(p + 2, w[2], w[3]);
  auto ready = [&]() {
    return (unsigned)(w[0] >> 32) == want && (unsigned)(w[1] >> 32) == want && (unsigned)(w[2] >> 32) == want &&
           (unsigned)(w[3] >> 32) == want;
  };
  if (!ready()) {
    const unsigned long long t0 = now_ns();
    do {
      slot_load2(p, w[0], w[1]);
      slot_load2(p + 2, w[2], w[3]);
      if (ready()) break;
      if (now_ns() - t0 > WAIT_NS) {
        v[0] = v[1] = v[2] = v[3] = 0.f;
        return false;
      }
    } while (true);
  }
#pragma unroll
  for (int i = 0; i < 4; i++) v[i] = __uint_as_float((unsigned)w[i]);
  return true;
}

}  // namespace qkpeer
