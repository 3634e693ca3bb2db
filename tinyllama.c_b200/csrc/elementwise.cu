// Embedding gather, RMSNorm, gated grouped RMSNorm and the SwiGLU product.
//
// Math follows CodeClaper/tinyllama.c's CPU ops: embedding row gather (cpu_op.c:508-524),
// RMSNorm ss=sum x^2, s=1/sqrt(ss/n+eps), o=x*s*w (cpu_op.c:44-64), SiLU x/(1+exp(-x))
// (cpu_op.c:332-335), the Mamba2 gate and grouped norm (cpu_op.c:950-958).  All
// statistics are 32-bit; only the stored result takes the activation type.
#include "common.cuh"
#include <stdarg.h>

int g_tlc_pdl = 0;
extern "C" void tlc_set_pdl(int on) { g_tlc_pdl = on; }

static thread_local char g_err[512];
extern "C" const char* tlc_last_error() { return g_err; }
int tlc_fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}

// ---- embedding ---------------------------------------------------------------------
template <typename TW>
__global__ void embed_kernel(const int* __restrict__ tokens, const TW* __restrict__ table, int D, int V,
                             float scale, float* __restrict__ out) {
  tlc_pdl(tokens, out);
  const int t = blockIdx.x;
  int tok = tokens[t];
  tok = tok < 0 ? 0 : (tok >= V ? V - 1 : tok);   // ids are validated on the host; never read out of bounds
  const TW* row = table + (size_t)tok * D;
  for (int d = threadIdx.x; d < D; d += blockDim.x) out[(size_t)t * D + d] = to_f32(row[d]) * scale;
}

extern "C" int tlc_embed(const int* tokens, const void* table, int table_dtype, int T, int D, int V, float scale,
                         float* out, cudaStream_t stream) {
  if (T == 0) return 0;
  // the first kernel of a step: a full dependency on everything before it (see tlc_launch_step_boundary)
  TLC_DISPATCH_DTYPE(table_dtype, TW, tlc_launch_step_boundary(embed_kernel<TW>, dim3(T), dim3(256), 0, stream, tokens,
                                                               (const TW*)table, D, V, scale, out));
  TLC_CHECK_LAUNCH("embed");
  return 0;
}

// ---- RMSNorm of 32-bit rows ----------------------------------------------------------
// One block per row.  The row stays in registers between the sum of squares and the scaling
// when it fits (up to RMS_MAX_PER_THREAD values per thread), otherwise it is read twice.
#define RMS_MAX_PER_THREAD 16
template <typename TO>
__global__ void __launch_bounds__(256)
rmsnorm_kernel(const float* __restrict__ x, const int* __restrict__ rows, const float* __restrict__ w,
               float eps, int D, TO* __restrict__ out) {
  tlc_pdl(x, rows, out);
  __shared__ float red[33];
  const int r = blockIdx.x;
  const float* xr = x + (size_t)(rows ? rows[r] : r) * D;
  float ss = 0.f;
  if (D <= 256 * RMS_MAX_PER_THREAD) {
    float v[RMS_MAX_PER_THREAD];
#pragma unroll
    for (int i = 0; i < RMS_MAX_PER_THREAD; i++) {
      const int d = threadIdx.x + i * 256;
      v[i] = d < D ? xr[d] : 0.f;
      ss += v[i] * v[i];
    }
    ss = block_sum(ss, red);
    const float s = 1.0f / sqrtf(ss / (float)D + eps);
#pragma unroll
    for (int i = 0; i < RMS_MAX_PER_THREAD; i++) {
      const int d = threadIdx.x + i * 256;
      if (d < D) out[(size_t)r * D + d] = from_f32<TO>(v[i] * s * w[d]);
    }
    return;
  }
  for (int d = threadIdx.x; d < D; d += blockDim.x) { float v = xr[d]; ss += v * v; }
  ss = block_sum(ss, red);
  const float s = 1.0f / sqrtf(ss / (float)D + eps);
  for (int d = threadIdx.x; d < D; d += blockDim.x) out[(size_t)r * D + d] = from_f32<TO>(xr[d] * s * w[d]);
}

// Rows whose width is a multiple of 4 (up to 16384): NT threads take PT float4 each.  The weight
// does not depend on the kernel before this one and is fetched before the wait on it.  NT and PT
// follow from the width alone, so a row's sum has the same tree whatever else is in the batch.
template <typename TO> struct Out4;
template <> struct Out4<float> {
  static __device__ __forceinline__ void put(float* p, float a, float b, float c, float d) {
    *reinterpret_cast<float4*>(p) = make_float4(a, b, c, d);
  }
};
template <> struct Out4<__nv_bfloat16> {
  static __device__ __forceinline__ void put(__nv_bfloat16* p, float a, float b, float c, float d) {
    __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
    uint2 u;
    u.x = *reinterpret_cast<unsigned*>(&lo);
    u.y = *reinterpret_cast<unsigned*>(&hi);
    *reinterpret_cast<uint2*>(p) = u;
  }
};

template <typename TO, int NT, int PT>
__global__ void __launch_bounds__(NT)
rmsnorm_vec_kernel(const float* __restrict__ x, const int* __restrict__ rows, const float* __restrict__ w,
                   float eps, int D, TO* __restrict__ out) {
  asm volatile("griddepcontrol.launch_dependents;");
  __shared__ float red[33];
  const int n4 = D >> 2;
  float4 wv[PT], v[PT];
#pragma unroll
  for (int i = 0; i < PT; i++) {
    const int c = threadIdx.x + i * NT;
    wv[i] = c < n4 ? __ldg(reinterpret_cast<const float4*>(w) + c) : make_float4(0.f, 0.f, 0.f, 0.f);
  }
  tlc_wait(x, rows, out);
  const int r = blockIdx.x;
  const float4* xr = reinterpret_cast<const float4*>(x + (size_t)(rows ? rows[r] : r) * D);
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < PT; i++) {
    const int c = threadIdx.x + i * NT;
    v[i] = c < n4 ? xr[c] : make_float4(0.f, 0.f, 0.f, 0.f);
  }
#pragma unroll
  for (int i = 0; i < PT; i++) ss += v[i].x * v[i].x + v[i].y * v[i].y + v[i].z * v[i].z + v[i].w * v[i].w;
  ss = block_sum(ss, red);
  const float s = 1.0f / sqrtf(ss / (float)D + eps);
#pragma unroll
  for (int i = 0; i < PT; i++) {
    const int c = threadIdx.x + i * NT;
    if (c < n4)
      Out4<TO>::put(out + (size_t)r * D + 4 * c, v[i].x * s * wv[i].x, v[i].y * s * wv[i].y, v[i].z * s * wv[i].z,
                    v[i].w * s * wv[i].w);
  }
}

// picks NT, PT from the number of float4 in a row (at most 4096 of them)
#define TLC_VEC_SHAPES(n4, LAUNCH)            \
  if ((n4) <= 128) { LAUNCH(128, 1); }        \
  else if ((n4) <= 256) { LAUNCH(256, 1); }   \
  else if ((n4) <= 512) { LAUNCH(512, 1); }   \
  else if ((n4) <= 1024) { LAUNCH(1024, 1); } \
  else if ((n4) <= 2048) { LAUNCH(1024, 2); } \
  else { LAUNCH(1024, 4); }

// The same for many rows (prompts): fewer threads a row with up to four float4 each, so that a thread has more
// loads in flight, more rows share an SM, and the block's sum has fewer warps to join.
#define TLC_VEC_SHAPES_MANY(n4, LAUNCH)       \
  if ((n4) <= 128) { LAUNCH(64, 2); }         \
  else if ((n4) <= 256) { LAUNCH(64, 4); }    \
  else if ((n4) <= 512) { LAUNCH(128, 4); }   \
  else if ((n4) <= 768) { LAUNCH(256, 3); }   \
  else if ((n4) <= 1024) { LAUNCH(256, 4); }  \
  else if ((n4) <= 2048) { LAUNCH(512, 4); }  \
  else { LAUNCH(1024, 4); }
constexpr int VEC_MANY_ROWS = 512;            // from this many rows on

extern "C" int tlc_rmsnorm(const float* x, const int* rows, const float* w, float eps, int R, int D, void* out,
                           int out_dtype, cudaStream_t stream) {
  if (R == 0) return 0;
  if (D % 4 == 0 && D <= 16384 && ((uintptr_t)x % 16) == 0 && ((uintptr_t)w % 16) == 0 && ((uintptr_t)out % 16) == 0) {
    const int n4 = D / 4;
#define TLC_RMS_LAUNCH(NT, PT)                                                                                        \
  TLC_DISPATCH_DTYPE(out_dtype, TO, tlc_launch(rmsnorm_vec_kernel<TO, NT, PT>, dim3(R), dim3(NT), 0, stream, x, rows, w, \
                                               eps, D, (TO*)out))
    if (R >= VEC_MANY_ROWS) { TLC_VEC_SHAPES_MANY(n4, TLC_RMS_LAUNCH) } else { TLC_VEC_SHAPES(n4, TLC_RMS_LAUNCH) }
#undef TLC_RMS_LAUNCH
    TLC_CHECK_LAUNCH("rmsnorm");
    return 0;
  }
  TLC_DISPATCH_DTYPE(out_dtype, TO, tlc_launch(rmsnorm_kernel<TO>, dim3(R), dim3(256), 0, stream, x, rows, w, eps, D, (TO*)out));
  TLC_CHECK_LAUNCH("rmsnorm");
  return 0;
}

// ---- gate and grouped RMSNorm of the scan output ---------------------------------------
// y [T, Di] 32-bit; z a strided slice of the input projection; out rows of out_ld elements, the whole
// result times out_scale; one block per (row, group).
template <typename TZ, typename TO>
__global__ void __launch_bounds__(256)
gated_rmsnorm_kernel(const float* __restrict__ y, const float* __restrict__ y2, const TZ* __restrict__ z, int ldz,
                                     const float* __restrict__ w, float eps, int Di, int gs, int norm_before_gate,
                                     TO* __restrict__ out, int out_ld, float out_scale) {
  tlc_pdl(y, y2, z, out);
  __shared__ float red[33];
  const int t = blockIdx.x, g = blockIdx.y;
  const float* yr = y + (size_t)t * Di + (size_t)g * gs;
  const float* y2r = y2 ? y2 + (size_t)t * Di + (size_t)g * gs : nullptr;    // a second summand of the input
  const TZ* zr = z + (size_t)t * ldz + (size_t)g * gs;
  TO* o = out + (size_t)t * out_ld + (size_t)g * gs;
  if (w == nullptr) {                                   // no norm: y * silu(z)
    for (int d = threadIdx.x; d < gs; d += blockDim.x) o[d] = from_f32<TO>((yr[d] + (y2r ? y2r[d] : 0.f)) * silu_f(to_f32(zr[d])) * out_scale);
    return;
  }
  const float* wg = w + (size_t)g * gs;
  float ss = 0.f;
  if (gs <= 256 * RMS_MAX_PER_THREAD) {
    // one pass: y and the gate are read once; what is normalised stays in registers
    float v[RMS_MAX_PER_THREAD], gate[RMS_MAX_PER_THREAD];
#pragma unroll
    for (int i = 0; i < RMS_MAX_PER_THREAD; i++) {          // every load is issued before the first exp
      const int d = threadIdx.x + i * 256;
      gate[i] = d < gs ? to_f32(zr[d]) : 0.f;
      v[i] = d < gs ? yr[d] + (y2r ? y2r[d] : 0.f) : 0.f;
    }
#pragma unroll
    for (int i = 0; i < RMS_MAX_PER_THREAD; i++) {
      gate[i] = silu_f(gate[i]);
      if (!norm_before_gate) v[i] *= gate[i];
      ss += v[i] * v[i];
    }
    ss = block_sum(ss, red);
    const float s = out_scale / sqrtf(ss / (float)gs + eps);
#pragma unroll
    for (int i = 0; i < RMS_MAX_PER_THREAD; i++) {
      const int d = threadIdx.x + i * 256;
      if (d < gs) o[d] = from_f32<TO>(norm_before_gate ? (v[i] * s * wg[d]) * gate[i] : v[i] * s * wg[d]);
    }
    return;
  }
  for (int d = threadIdx.x; d < gs; d += blockDim.x) {
    float v = yr[d] + (y2r ? y2r[d] : 0.f);
    if (!norm_before_gate) v *= silu_f(to_f32(zr[d]));
    ss += v * v;
  }
  ss = block_sum(ss, red);
  const float s = out_scale / sqrtf(ss / (float)gs + eps);
  for (int d = threadIdx.x; d < gs; d += blockDim.x) {
    const float gate = silu_f(to_f32(zr[d]));
    float v = yr[d] + (y2r ? y2r[d] : 0.f);
    v = norm_before_gate ? (v * s * wg[d]) * gate : (v * gate) * s * wg[d];
    o[d] = from_f32<TO>(v);
  }
}

// Groups whose width is a multiple of 4 (up to 16384), 32-bit gate: NT threads take PT float4 each;
// the weight is fetched before the wait on the previous kernel.
template <typename TO, int NT, int PT>
__global__ void __launch_bounds__(NT)
gated_rmsnorm_vec_kernel(const float* __restrict__ y, const float* __restrict__ y2, const float* __restrict__ z, int ldz, const float* __restrict__ w,
                         float eps, int Di, int gs, int norm_before_gate, TO* __restrict__ out, int out_ld,
                         float out_scale) {
  asm volatile("griddepcontrol.launch_dependents;");
  __shared__ float red[33];
  const int t = blockIdx.x, g = blockIdx.y;
  const int n4 = gs >> 2;
  float4 wv[PT], v[PT], gate[PT];
#pragma unroll
  for (int i = 0; i < PT; i++) {
    const int c = threadIdx.x + i * NT;
    wv[i] = c < n4 ? __ldg(reinterpret_cast<const float4*>(w + (size_t)g * gs) + c) : make_float4(0.f, 0.f, 0.f, 0.f);
  }
  tlc_wait(y, y2, z, out);
  const float4* yr = reinterpret_cast<const float4*>(y + (size_t)t * Di + (size_t)g * gs);
  const float4* y2r = y2 ? reinterpret_cast<const float4*>(y2 + (size_t)t * Di + (size_t)g * gs) : nullptr;
  const float4* zr = reinterpret_cast<const float4*>(z + (size_t)t * ldz + (size_t)g * gs);
#pragma unroll
  for (int i = 0; i < PT; i++) {
    const int c = threadIdx.x + i * NT;
    v[i] = c < n4 ? yr[c] : make_float4(0.f, 0.f, 0.f, 0.f);
    gate[i] = c < n4 ? zr[c] : make_float4(0.f, 0.f, 0.f, 0.f);
    if (y2r != nullptr && c < n4) {                     // the input comes as two summands
      const float4 u = y2r[c];
      v[i] = make_float4(v[i].x + u.x, v[i].y + u.y, v[i].z + u.z, v[i].w + u.w);
    }
  }
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < PT; i++) {
    constexpr bool QUICK = sizeof(TO) == 2;              // a bfloat16 output means a bfloat16 run
    gate[i] = make_float4(silu_of<QUICK>(gate[i].x), silu_of<QUICK>(gate[i].y), silu_of<QUICK>(gate[i].z), silu_of<QUICK>(gate[i].w));
    if (!norm_before_gate) { v[i].x *= gate[i].x; v[i].y *= gate[i].y; v[i].z *= gate[i].z; v[i].w *= gate[i].w; }
    ss += v[i].x * v[i].x + v[i].y * v[i].y + v[i].z * v[i].z + v[i].w * v[i].w;
  }
  ss = block_sum(ss, red);
  const float s = out_scale / sqrtf(ss / (float)gs + eps);
  TO* o = out + (size_t)t * out_ld + (size_t)g * gs;
#pragma unroll
  for (int i = 0; i < PT; i++) {
    const int c = threadIdx.x + i * NT;
    if (c < n4) {
      if (norm_before_gate)
        Out4<TO>::put(o + 4 * c, (v[i].x * s * wv[i].x) * gate[i].x, (v[i].y * s * wv[i].y) * gate[i].y,
                      (v[i].z * s * wv[i].z) * gate[i].z, (v[i].w * s * wv[i].w) * gate[i].w);
      else
        Out4<TO>::put(o + 4 * c, v[i].x * s * wv[i].x, v[i].y * s * wv[i].y, v[i].z * s * wv[i].z, v[i].w * s * wv[i].w);
    }
  }
}

extern "C" int tlc_gated_rmsnorm(const float* y, const float* y2, const void* z, int z_dtype, int ldz, const float* w, float eps, int T,
                                 int Di, int n_groups, int norm_before_gate, void* out, int out_dtype, int out_ld,
                                 float out_scale, cudaStream_t stream) {
  if (T == 0) return 0;
  if (out_ld <= 0) out_ld = Di;                          // elements between rows of out (0: dense)
  TLC_REQUIRE(n_groups > 0 && Di % n_groups == 0, "gated_rmsnorm: width %d is not a multiple of %d groups", Di, n_groups);
  const int gs = Di / n_groups;
  dim3 grid(T, n_groups);
  if (w != nullptr && z_dtype == TLC_F32 && gs % 4 == 0 && gs <= 16384 && ldz % 4 == 0 && ((uintptr_t)y % 16) == 0 &&
      ((uintptr_t)z % 16) == 0 && ((uintptr_t)w % 16) == 0 && ((uintptr_t)out % 16) == 0 && out_ld % 4 == 0 &&
      ((uintptr_t)y2 % 16) == 0) {
    const int n4 = gs / 4;
#define TLC_GRMS_LAUNCH(NT, PT)                                                                                         \
  TLC_DISPATCH_DTYPE(out_dtype, TO, tlc_launch(gated_rmsnorm_vec_kernel<TO, NT, PT>, grid, dim3(NT), 0, stream, y, y2,    \
                                               (const float*)z, ldz, w, eps, Di, gs, norm_before_gate, (TO*)out, out_ld, out_scale))
    if (T >= VEC_MANY_ROWS) { TLC_VEC_SHAPES_MANY(n4, TLC_GRMS_LAUNCH) } else { TLC_VEC_SHAPES(n4, TLC_GRMS_LAUNCH) }
#undef TLC_GRMS_LAUNCH
    TLC_CHECK_LAUNCH("gated_rmsnorm");
    return 0;
  }
  TLC_DISPATCH_DTYPE(z_dtype, TZ, TLC_DISPATCH_DTYPE(out_dtype, TO, tlc_launch(gated_rmsnorm_kernel<TZ, TO>, dim3(grid), dim3(256), 0, stream, 
      y, y2, (const TZ*)z, ldz, w, eps, Di, gs, norm_before_gate, (TO*)out, out_ld, out_scale)));
  TLC_CHECK_LAUNCH("gated_rmsnorm");
  return 0;
}

// ---- SwiGLU product: out = silu(gate) * up, gate|up side by side in one row ---------------
// interleave: gate and up come in groups of 16 columns (8 gates, then their 8 ups) instead of as two halves
template <typename TI, typename T>
__global__ void swiglu_kernel(const TI* __restrict__ gu, int ld, int F, T* __restrict__ out, size_t total, int interleave) {
  tlc_pdl(gu, out);
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const size_t t = i / F;
  const int f = (int)(i % F);
  const int gc = interleave ? (f >> 3) * 16 + (f & 7) : f, uc = interleave ? gc + 8 : F + f;
  const float g = to_f32(gu[t * ld + gc]), u = to_f32(gu[t * ld + uc]);
  out[i] = from_f32<T>(silu_f(g) * u);
}

extern "C" int tlc_swiglu(const void* gu, int in_dtype, int ld, int F, int T, void* out, int dtype, int interleave,
                          cudaStream_t stream) {
  const size_t total = (size_t)T * F;
  if (total == 0) return 0;
  const unsigned blocks = (unsigned)((total + 255) / 256);
  TLC_DISPATCH_DTYPE(in_dtype, TI, TLC_DISPATCH_DTYPE(dtype, TT, tlc_launch(swiglu_kernel<TI, TT>, dim3(blocks), dim3(256), 0, stream, 
      (const TI*)gu, ld, F, (TT*)out, total, interleave)));
  TLC_CHECK_LAUNCH("swiglu");
  return 0;
}

// ---- gather rows of a 32-bit matrix ------------------------------------------------------
__global__ void gather_rows_kernel(const float* __restrict__ x, const int* __restrict__ rows, int D,
                                   float* __restrict__ out) {
  tlc_pdl(x, rows, out);
  const float* xr = x + (size_t)rows[blockIdx.x] * D;
  for (int d = threadIdx.x; d < D; d += blockDim.x) out[(size_t)blockIdx.x * D + d] = xr[d];
}
extern "C" int tlc_gather_rows(const float* x, const int* rows, int R, int D, float* out, cudaStream_t stream) {
  if (R == 0) return 0;
  tlc_launch(gather_rows_kernel, dim3(R), dim3(256), 0, stream, x, rows, D, out);
  TLC_CHECK_LAUNCH("gather_rows");
  return 0;
}
