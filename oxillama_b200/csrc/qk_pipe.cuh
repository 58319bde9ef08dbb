// Shared device helpers of the bulk-copy pipelines: mbarrier + cp.async.bulk
// wrappers (every wait bounded), shared-memory vector loads, dp4a.
#pragma once
#include <cstdint>
#include <cuda_fp16.h>

#ifndef QK_PARK_NS
#define QK_PARK_NS 20000u  // how long a waiting thread may stay parked per poll
#endif

namespace qkpipe {

__device__ __forceinline__ uint32_t smem_u32(const void *p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void *src, uint32_t bytes,
                                         uint32_t bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
          dst),
      "l"(src), "r"(bytes), "r"(bar)
      : "memory");
}
// The same copy for data that is read once (weights streaming through a decode matvec):
// marked evict-first in L2, so that it does not push out the small buffers every launch
// re-reads (the activations, the outputs).
__device__ __forceinline__ uint64_t stream_policy() {
  uint64_t policy;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(policy));
  return policy;
}
// `policy` from stream_policy(), made once per thread: creating it costs the issuing thread a
// few hundred cycles (measured: a producer loop that made one per copy issued a copy every
// 250 ns).
__device__ __forceinline__ void bulk_g2s_stream(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar,
                                                uint64_t policy) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;" ::"r"(
          dst),
      "l"(src), "r"(bytes), "r"(bar), "l"(policy)
      : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// The same poll, letting the hardware park the thread for up to `hint_ns` while the
// phase is pending (it is woken when the phase completes), so that a waiting warp
// does not spend issue slots on its polling loop.
__device__ __forceinline__ bool mbar_try_wait_parked(uint32_t bar, uint32_t parity, uint32_t hint_ns) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity), "r"(hint_ns)
      : "memory");
  return ok != 0;
}
// Bounded wait: false if the barrier has not flipped after about a quarter of a
// second (checked against the global nanosecond timer every 256 polls).
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity) {
  if (mbar_try_wait(bar, parity)) return true;
  unsigned long long t0;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
  for (;;) {
    for (int i = 0; i < 256; i++)
      if (mbar_try_wait_parked(bar, parity, QK_PARK_NS)) return true;
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    if (t - t0 > 250000000ull) return false;
  }
}
__device__ __forceinline__ int dp4a_us(uint32_t a, uint32_t b, int c) {  // u8 x s8
  int d;
  asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  return d;
}
__device__ __forceinline__ int dp4a_ss(uint32_t a, uint32_t b, int c) {  // s8 x s8
  int d;
  asm("dp4a.s32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  return d;
}
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "r"(addr));
  return v;
}
__device__ __forceinline__ float4 lds128f(uint32_t addr) {
  float4 v;
  asm volatile("ld.shared.v4.f32 {%0,%1,%2,%3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "r"(addr));
  return v;
}
__device__ __forceinline__ uint32_t lds32(uint32_t addr) {
  uint32_t v;
  asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
  return v;
}
__device__ __forceinline__ float h2f_bits(uint32_t h) {
  return __half2float(__ushort_as_half((unsigned short)(h & 0xFFFFu)));
}


// Threads 0 .. n-1 of the caller each wait until flags[thread] has reached *epoch (written
// by another GPU with a system-scope release), for at most a quarter of a second.
// Returns false on the thread whose wait ran out.
__device__ __forceinline__ bool flags_wait_bounded(const unsigned *flags, const unsigned *epoch, uint32_t n,
                                                   uint32_t tid) {
  if (tid >= n) return true;
  const unsigned want = *reinterpret_cast<const volatile unsigned *>(epoch);
  unsigned long long t0;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
  for (;;) {
    unsigned v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(flags + tid) : "memory");
    if ((int)(v - want) >= 0) return true;
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    if (t - t0 > 250000000ull) return false;
  }
}

// Programmatic dependent launch: lets the next kernel in the stream start its
// prologue while this grid drains / waits until the previous grid's memory is
// visible.  Both are no-ops when the launch did not opt in.
__device__ __forceinline__ void pdl_launch_dependents() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

}  // namespace qkpipe
