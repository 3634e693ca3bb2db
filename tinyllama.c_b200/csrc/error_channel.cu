// The error channel of kernels whose waits are bounded, and its self-test.
//
// CodeClaper/tinyllama.c prints and exits on any CUDA error (gpu.h:41-50) and has no kernel that waits on
// another agent.  Here the tensor-core product waits on mbarriers (TMA loader, MMA issuer, epilogue); every
// such wait gives up after a limit, records which one it was in a device word with a host-visible copy, and
// the kernel frees what it holds and returns, so that the context stays usable and the host can raise.  The
// self-test below makes that path observable without a fault: one block waits on a barrier that nobody
// arrives at.
#include "common.cuh"
#include "mbarrier.cuh"

extern "C" int tlc_wait_limit_cycles(long long cycles) {
  ErrWords* err = tlc_error_words();
  TLC_REQUIRE(err != nullptr, "wait limit: the library is not set up (tlc_linear_init)");
  const long long v = cycles > 0 ? cycles : TLC_WAIT_LIMIT_CYCLES;
  if (cudaMemcpy(&err->limit, &v, sizeof(v), cudaMemcpyHostToDevice) != cudaSuccess)
    return tlc_fail(-2, "wait limit: cannot write the limit");
  return 0;
}

__global__ void selftest_bounded_wait_kernel(ErrWords* err) {
  tlc_pdl(err);
  __shared__ uint64_t bar;
  if (threadIdx.x == 0) {
    mbar_init(smem_u32(&bar), 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    mbar_wait(smem_u32(&bar), 0, err, 9, mbar_wait_limit(err));        // phase 0 never completes: the wait runs out and records 9
  }
}

extern "C" int tlc_selftest_bounded_wait(cudaStream_t stream) {
  ErrWords* err = tlc_error_words();
  TLC_REQUIRE(err != nullptr, "self-test: the library is not set up (tlc_linear_init)");
  tlc_launch(selftest_bounded_wait_kernel, dim3(1), dim3(32), 0, stream, err);
  TLC_CHECK_LAUNCH("selftest_bounded_wait");
  return 0;
}
