// mbarrier helpers with bounded waits, and the error words that a wait which ran out reports through.
#pragma once
#include "common.cuh"

constexpr long long TLC_WAIT_LIMIT_CYCLES = 2000000000LL;   // the default limit of a wait: about a second

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try(uint32_t bar, uint32_t parity) {
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
// Bounded wait: false (and the error code recorded) if the phase does not complete in time.
// `err` points at two words: [0] in device memory (what kernels read), [1] the address of a
// host-mapped word that is written on failure only, so that the host can look without a copy.
// [2] how many cycles a wait may spin (tlc_wait_limit_cycles sets it).  A kernel reads the limit once, when it
// starts (mbar_wait_limit), and hands it to every wait: a load from global memory inside the wait would cost
// more than most waits last.
struct ErrWords { int flag; int* host; long long limit; };
__device__ __forceinline__ long long mbar_wait_limit(const ErrWords* err) { return *(const volatile long long*)&err->limit; }
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, ErrWords* err, int code, long long limit) {
  if (mbar_try(bar, parity)) return true;
  const long long t0 = clock64();
  while (!mbar_try(bar, parity)) {
    if (clock64() - t0 > limit) {
      atomicExch(&err->flag, code);
      *(volatile int*)err->host = code;
      return false;
    }
  }
  return true;
}

__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

// The error words of the library (set up by tlc_linear_init); nullptr before that.
ErrWords* tlc_error_words();
