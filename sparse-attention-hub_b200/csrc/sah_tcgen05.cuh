// tcgen05 / mbarrier / asynchronous-copy building blocks shared by the kernels that use the
// fifth-generation tensor cores: shared-memory matrix descriptors, the instruction descriptor
// of kind::f16 with bfloat16 operands and a float32 accumulator in tensor memory, commit and
// fences, tensor-memory loads and stores, mbarrier initialisation and bounded waits.
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cstdint>

#ifndef ATM_SPIN_LIMIT
#define ATM_SPIN_LIMIT (1 << 19)
#endif

// ---- mbarrier / tensor-map gather ------------------------------------------------
__device__ __forceinline__ void atm_mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void atm_mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(bar), "r"(bytes)
               : "memory");
}
// One try of the phase test; the hardware may suspend the thread for up to `hint_ns` while the
// phase is pending, so a waiting warp does not compete for issue slots.
__device__ __forceinline__ bool atm_mbar_try(uint32_t bar, uint32_t parity, uint32_t hint_ns) {
  uint32_t ok;
  asm volatile(
      "{\n.reg .pred p;\n"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n"
      "selp.u32 %0, 1, 0, p;\n}\n"
      : "=r"(ok)
      : "r"(bar), "r"(parity), "r"(hint_ns)
      : "memory");
  return ok != 0u;
}
// Bounded wait: false when the phase did not complete within the limit (about a second).
__device__ __forceinline__ bool atm_mbar_wait(uint32_t bar, uint32_t parity) {
  for (int i = 0; i < ATM_SPIN_LIMIT; ++i)
    if (atm_mbar_try(bar, parity, 2000u)) return true;
  return false;
}
__device__ __forceinline__ void atm_cp_async16(uint32_t dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(dst), "l"(src) : "memory");
}

// Shared-memory matrix descriptor of tcgen05.mma: start address, leading-dimension and stride
// byte offsets (all in units of 16 bytes), the descriptor version of this architecture, and
// the swizzle mode (0 none, 2 128-byte).
__device__ __forceinline__ uint64_t aum_desc(uint32_t saddr, uint32_t lbo, uint32_t sbo, uint32_t layout) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr & 0x3FFFFu) >> 4);
  d |= (uint64_t)((lbo >> 4) & 0x3FFFu) << 16;
  d |= (uint64_t)((sbo >> 4) & 0x3FFFu) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)(layout & 7u) << 61;
  return d;
}
// Instruction descriptor, kind::f16: fp32 accumulator, bf16 operands, M = 128, N = `n` (a
// multiple of 16, at most 256); bit 15 / 16: A / B are MN-major (0 = K-major).
__device__ __forceinline__ uint32_t aum_idesc(bool a_mn, bool b_mn, uint32_t n = 16u) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((a_mn ? 1u : 0u) << 15) | ((b_mn ? 1u : 0u) << 16) |
         ((n >> 3) << 17) | ((128u >> 4) << 24);
}
__device__ __forceinline__ void aum_mma(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                        uint32_t accumulate) {
  asm volatile(
      "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n" ::"r"(tmem_d),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// The mbarrier gets one arrival when all tcgen05.mma issued so far by this thread are complete.
__device__ __forceinline__ void aum_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(bar)
               : "memory");
}
__device__ __forceinline__ void aum_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void aum_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
}
__device__ __forceinline__ void aum_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
}
// 8 or 16 consecutive columns of this thread's lane of tensor memory
__device__ __forceinline__ void aum_tmem_ld8(uint32_t taddr, uint32_t* r) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
               : "r"(taddr));
  asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
}
__device__ __forceinline__ void aum_tmem_ld16(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];\n"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr));
  asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
}
__device__ __forceinline__ void aum_tmem_st16(uint32_t taddr, const uint32_t* r) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};\n" ::
          "r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
      "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
  asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory");
}

// Bounded wait that also gives up when another role of the CTA has given up.  The phase test
// carries no suspend-time hint: most waits of this kernel are entered before the phase
// completes and are satisfied a few hundred cycles later, and a hinted test was seen to keep
// the thread asleep for a good part of the hint.  The bound is wall time (about a second),
// looked at every 256 tests.
__device__ __forceinline__ bool aum_try(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n.reg .pred p;\n"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      "selp.u32 %0, 1, 0, p;\n}\n"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0u;
}
__device__ __forceinline__ uint64_t aum_now_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;\n" : "=l"(t));
  return t;
}
// `backoff_ns` > 0: sleep that long after a failed test (waits that are entered long before the
// phase completes -- a spinning warp takes issue slots and shared-memory bandwidth from the
// warps that compute); 0: test again at once (waits on the per-tile critical path).
__device__ __forceinline__ bool aum_wait(uint32_t bar, uint32_t parity, volatile int* abort_sm,
                                         int* __restrict__ errflag, unsigned backoff_ns = 0,
                                         unsigned long long limit_ns = 1000000000ull) {
  if (aum_try(bar, parity)) return true;
  const uint64_t t0 = aum_now_ns();
  for (int round = 0; round < (1 << 24); ++round) {
#pragma unroll 1
    for (int i = 0; i < 64; ++i) {
      if (backoff_ns) __nanosleep(backoff_ns);
      if (aum_try(bar, parity)) return true;
    }
    if (*abort_sm) return false;
    if (aum_now_ns() - t0 > limit_ns) break;
  }
  *abort_sm = 1;
  atomicExch(errflag, 1);
  return false;
}

// The same for a whole warp: every lane waits, and the warp continues only if all lanes saw the
// phase complete, so that no lane leaves a loop that the others stay in.  (One polling lane with
// the outcome handed round by a shuffle, and sleeping between polls, both measured slower in
// the attention kernel: the waits sit on the per-tile critical path.)
__device__ __forceinline__ bool aum_wait_warp(uint32_t bar, uint32_t parity, volatile int* abort_sm,
                                              int* __restrict__ errflag, unsigned backoff_ns = 0,
                                              unsigned long long limit_ns = 1000000000ull) {
  const bool ok = aum_wait(bar, parity, abort_sm, errflag, backoff_ns, limit_ns);
  return __all_sync(0xffffffffu, ok);
}
