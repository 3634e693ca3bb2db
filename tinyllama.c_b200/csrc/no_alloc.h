// An entry point for callers that must not allocate.  It has no counterpart in
// CodeClaper/tinyllama.c (whose GPU path allocates scratch buffers on demand, gpu.cu:2036-2049).
//
// Who needs it: code that drives the kernels without an allocator of its own and may not call
// cudaMalloc where it runs -- a real-time or embedded host loop with a no-allocation rule, a
// plugin inside another process that owns all device memory, code between two points where the
// driver must not be asked for memory.  The single-token attention kernel splits a sequence's keys
// across blocks and needs room for the blocks' partial results; the regular entry point
// (tlc_attention_decode) takes that room from the caller, this one carries it inside the library.
//
//   int tlc_attention_decode_no_alloc(q, dtype, k_pages, v_pages, block_table, max_pages, positions,
//                                     row_seq, slots, out, T, H, KV, hd, scale, window, max_keys, stream)
//
// Same arguments and result as tlc_attention_decode without its two scratch pointers; inputs
// and outputs are still the caller's.  Returns 0, or a negative code with a message in
// tlc_last_error().
//
// Limits and rules
//  * The scratch is one fixed array of TLC_NO_ALLOC_SCRATCH_FLOATS floats (8 MiB) in device
//    memory.  Every GPU whose context loads this library holds it until the process exits.
//  * A call needs T * H * ceil(max_keys / 128) * (hd + 2) floats; a larger call is refused with
//    an error and nothing is launched.
//  * The first call on a device looks up the device address of the array (one
//    cudaGetSymbolAddress, with that device current) and remembers it; make that first call
//    before any stream capture begins on the device.  No call allocates or frees: no
//    cudaMalloc, cudaFree or allocating library routine.
//  * All calls share the array.  It keeps what the last call left; the kernels write every
//    value before they read it (each block records its maximum and sum, empty splits record a
//    zero sum and are skipped), so nothing needs clearing.  Two calls that overlap on the GPU
//    (different streams, or different host threads without ordering) race on it: order them.
#pragma once
#include <cuda_runtime.h>

#define TLC_NO_ALLOC_SCRATCH_FLOATS (2 * 1024 * 1024)
#define TLC_NO_ALLOC_MAX_DEVICES 64

extern "C" int tlc_attention_decode_no_alloc(const void* q, int dtype, const void* k_pages, const void* v_pages,
                                             const int* block_table, int max_pages, const int* positions,
                                             const int* row_seq, const int* slots, void* out, int T, int H, int KV,
                                             int hd, float scale, int window, int max_keys, cudaStream_t stream);
