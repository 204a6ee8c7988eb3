// Shared device helpers for the sm_100a W4A16 kernels: mbarrier / PDL wrappers with
// bounded waits, the INT4 nibble extraction, and the legacy warp MMA used by the skinny kernel.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace lbl {

// ---------------------------------------------------------------------------------------------
// Device status word (one int per device, owned by the host side of the library and passed to
// every kernel that waits).  A kernel whose bounded wait expires stores a code there and carries
// on to a normal exit (results are then undefined); the host reads it with lbl_device_status().
// ---------------------------------------------------------------------------------------------
constexpr int kStatusSkinnyFullWait = 101;   // skinny kernel: a stage never filled
constexpr int kStatusSkinnyEmptyWait = 102;  // skinny kernel: a stage was never released
constexpr int kStatusGemmWait = 200;         // tcgen05 GEMM: 200 + barrier role

// Upper bound of any spin on an mbarrier, in SM clock cycles (about 2 s at 2 GHz).
constexpr long long kWaitLimitCycles = 1LL << 32;

__device__ __forceinline__ uint32_t smem_addr(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(bar)), "r"(count) : "memory");
}

// Makes freshly initialised barriers visible to the async proxy (bulk copies, tcgen05.commit).
__device__ __forceinline__ void mbar_init_fence() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_addr(bar)) : "memory");
}

__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_addr(bar)),
               "r"(bytes)
               : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t done;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(done)
      : "r"(smem_addr(bar)), "r"(parity)
      : "memory");
  return done != 0;
}

// Waits for the phase with the given parity.  `abort_flag` lives in shared memory: once any
// thread of the CTA has given up, every later wait returns at once so that the CTA drains and
// exits instead of hanging.  Returns false if the wait was abandoned.
// Up to `kSpins` polls of the phase in one tight loop (three instructions per poll).  Each poll may
// park the warp for up to `kSuspendNs` before it reports "not yet", so a waiting warp leaves the
// issue slots to the warps that have work.
template <int kSpins, int kSuspendNs>
__device__ __forceinline__ bool mbar_poll(uint64_t* bar, uint32_t parity) {
  uint32_t done;
  asm volatile(
      "{\n\t.reg .pred p;\n\t.reg .pred q;\n\t.reg .u32 n;\n\t"
      "mov.u32 n, 0;\n"
      "LBL_POLL:\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
      "@p bra LBL_DONE;\n\t"
      "add.u32 n, n, 1;\n\t"
      "setp.lt.u32 q, n, %4;\n\t"
      "@q bra LBL_POLL;\n"
      "LBL_DONE:\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(done)
      : "r"(smem_addr(bar)), "r"(parity), "r"(static_cast<uint32_t>(kSuspendNs)), "n"(kSpins)
      : "memory");
  return done != 0;
}

__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, uint32_t parity,
                                                  volatile int* abort_flag, int* status_word,
                                                  int status_code) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long start = clock64();
  while (true) {
    if (mbar_poll<64, 2000>(bar, parity)) return true;
    // The abort flag and the clock are looked at once per batch of polls.
    if (*abort_flag) return false;
    if (clock64() - start > kWaitLimitCycles) {
      *abort_flag = 1;
      atomicCAS(status_word, 0, status_code);
      return false;
    }
  }
}

// Programmatic dependent launch.  Both are no-ops when the launch did not ask for it.
__device__ __forceinline__ void pdl_wait_for_previous_kernel() {
  asm volatile("griddepcontrol.wait;" ::: "memory");
}
__device__ __forceinline__ void pdl_allow_next_kernel() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

// Consumer-only barrier (id 1..15) over `threads` threads.
__device__ __forceinline__ void named_barrier(int id, int threads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

// D(16x8,f32) = A(16x16,f16,row) * B(16x8,f16,col) + C
__device__ __forceinline__ void mma_m16n8k16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0,
                                             uint32_t b1, const float (&c)[4]) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 "
      "{%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%11,%12,%13};"
      : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "f"(c[0]), "f"(c[1]),
        "f"(c[2]), "f"(c[3]));
}

// ---------------------------------------------------------------------------------------------
// Nibble extraction.  A packed word holds columns 8j..8j+7, column i at bits 4i..4i+3.
//
// An FP16 bit pattern with a zero exponent field is the subnormal  mantissa * 2^-24, so a nibble
// left at bits 0..3 of a 16-bit lane *is* the number q * 2^-24 and a nibble at bits 4..7 is
// 16 q * 2^-24 -- both exact, with no bias to subtract.  One AND per pair of columns therefore
// yields an MMA-ready half2; the constant 2^-24 is folded into the FP32 group scale and the
// factor 16 into the activation operand.
//   out[0] = (q0, q4)       out[1] = 16 * (q1, q5)
//   out[2] = (q2, q6)       out[3] = 16 * (q3, q7)          (all times 2^-24)
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void nibbles_as_subnormal_half2(uint32_t word, uint32_t (&out)[4]) {
  const uint32_t hi = word >> 8;
  out[0] = word & 0x000F000Fu;
  out[1] = word & 0x00F000F0u;
  out[2] = hi & 0x000F000Fu;
  out[3] = hi & 0x00F000F0u;
}
constexpr float kNibbleUnit = 16777216.0f;  // 2^24: the MMA sees q * 2^-24

// Nanoseconds of the GPU's global timer (measurement builds only).
__device__ __forceinline__ unsigned long long global_timer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

}  // namespace lbl
