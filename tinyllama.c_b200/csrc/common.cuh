// Shared device helpers and the host-side error channel of the kernel library.
//
// Every exported function returns 0 on success or a negative code after storing a
// message that tlc_last_error() returns; nothing here exits or traps (the reference
// prints and exits on any CUDA error, gpu.h:41-50 -- a library must not).
#pragma once

#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>
#include <stdio.h>

#include "tinyllama_c_b200.h"   // every exported function: a definition that strays from its declaration does not compile

int tlc_fail(int code, const char* fmt, ...);

#define TLC_CHECK_LAUNCH(name)                                                  \
  do {                                                                          \
    cudaError_t e__ = cudaGetLastError();                                       \
    if (e__ != cudaSuccess) return tlc_fail(-2, "%s: %s", name, cudaGetErrorString(e__)); \
  } while (0)

#define TLC_REQUIRE(cond, ...)                       \
  do {                                               \
    if (!(cond)) return tlc_fail(-1, __VA_ARGS__);   \
  } while (0)

// ---- launches -----------------------------------------------------------------------------
// Every kernel begins with tlc_pdl(): it lets the next kernel of the stream be scheduled early
// and then waits until the previous kernel has finished and its writes are visible.  Both
// instructions do nothing unless the launch carries the programmatic-serialization attribute,
// which tlc_launch() adds while tlc_set_pdl(1) is in effect (the library turns it on when it is
// loaded): a step is hundreds of short kernels, and this hides the gap between one kernel's last
// block and the next kernel's first.
extern int g_tlc_pdl;

//
// The wait takes the pointers through which the kernel reads what earlier kernels of the stream
// wrote (or writes what they read): a load through a const __restrict__ pointer may otherwise be
// moved above the wait by the compiler, which knows that nothing in the kernel writes there; after
// tlc_wait the pointer's value comes out of an asm statement that follows the wait, so no access
// through it can start earlier.  Weights and tables that the host uploaded need not be listed.
template <typename P> __device__ __forceinline__ void tlc_launder(P& p) { asm volatile("" : "+l"(p) : : "memory"); }

template <typename... P> __device__ __forceinline__ void tlc_wait(P&... ptrs) {
  asm volatile("griddepcontrol.wait;" ::: "memory");
  (tlc_launder(ptrs), ...);
}

template <typename... P> __device__ __forceinline__ void tlc_pdl(P&... ptrs) {
  asm volatile("griddepcontrol.launch_dependents;");
  tlc_wait(ptrs...);
}

template <typename... KArgs, typename... Args>
inline cudaError_t tlc_launch_as(bool programmatic, void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                 cudaStream_t stream, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = (programmatic && g_tlc_pdl) ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

template <typename... KArgs, typename... Args>
inline cudaError_t tlc_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                              Args&&... args) {
  return tlc_launch_as(true, kernel, grid, block, smem, stream, static_cast<Args&&>(args)...);
}

// The step boundary.  Some kernels fetch, BEFORE their wait, cache contents that an earlier step wrote (a
// sequence's state, its convolution window, its old keys and values).  With programmatic launches alone that
// is a matter of timing: the kernel that wrote them may be many launches upstream and still running, since
// every kernel releases its successor at once.  So the first kernel of every step (the embedding) is launched
// WITHOUT the programmatic attribute: it starts only when all earlier work of the stream has completed and is
// visible, and no kernel of the step can be scheduled before it has started.  What a kernel may fetch ahead of
// its wait is therefore: weights and tables, and cache contents written by an earlier step -- never anything
// written by a kernel of the same step.
template <typename... KArgs, typename... Args>
inline cudaError_t tlc_launch_step_boundary(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                            cudaStream_t stream, Args&&... args) {
  return tlc_launch_as(false, kernel, grid, block, smem, stream, static_cast<Args&&>(args)...);
}

template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Sum over a block of up to 1024 threads; every thread gets the result.  `red` is a
// shared array of 33 floats.  The tree is fixed by the block size alone, so a row's
// result does not depend on what else is in the batch.
__device__ __forceinline__ float block_sum(float v, float* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float t = lane < nw ? red[lane] : 0.f;
    t = warp_sum(t);
    if (lane == 0) red[32] = t;
  }
  __syncthreads();
  return red[32];
}

__device__ __forceinline__ float silu_f(float x) { return x / (1.0f + expf(-x)); }
// SiLU for bfloat16 runs: exp and reciprocal by the special-function unit, a few units in the last place
// of 32 bits (far below the rounding of a bfloat16 or TF32 operand); the 32-bit path keeps silu_f, whose
// full-precision division costs several times as much.
__device__ __forceinline__ float silu_quick(float x) { return __fdividef(x, 1.0f + __expf(-x)); }
template <bool QUICK> __device__ __forceinline__ float silu_of(float x) { return QUICK ? silu_quick(x) : silu_f(x); }
// softplus with the reference's cut-over (cpu_op.c:354-356)
__device__ __forceinline__ float softplus_f(float x) { return x > 20.0f ? x : log1pf(expf(x)); }

// Dispatch a lambda-like macro over the two element types.
#define TLC_DISPATCH_DTYPE(code, T, ...)                                  \
  if ((code) == TLC_F32) { using T = float; __VA_ARGS__; }                \
  else if ((code) == TLC_BF16) { using T = __nv_bfloat16; __VA_ARGS__; }  \
  else return tlc_fail(-1, "unknown dtype code %d", (int)(code));
