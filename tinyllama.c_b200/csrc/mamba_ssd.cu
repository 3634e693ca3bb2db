// Selective scan of long prompts in chunked matrix form, on the tensor cores.
//
// The recurrence is the reference's (cpu_op.c:932-951):
//     S_t = S_{t-1} * exp(dt_t A) + (dt_t x_t) (x) B_t ,   y_t = S_t . C_t + D x_t
// Over a chunk of rows i, j (L <= 128) with cum_i = sum_{k<=i} dt_k A this is three products:
//     y_i  = sum_{j<=i} (C_i . B_j) exp(cum_i - cum_j) dt_j x_j        "inside the chunk"
//          + exp(cum_i) * (S_in C_i)                                  "what came before"
//          + D x_i
//     S_c  = sum_j exp(cum_last - cum_j) dt_j x_j (x) B_j               the chunk's own contribution
//     S_in(c+1) = exp(cum_last) S_in(c) + S_c                           carried in chunk order
// Kernels: cumulative decay per (chunk, head); C B^T per (chunk, group) (shared by the group's
// heads); the chunk states; the carry (ssm_state_pass in mamba.cu); the outputs.  The products
// run on mma.sync.m16n8k8 with TF32 operands (10-bit mantissa; the 32-bit path of the library
// never comes here) and 32-bit accumulation; decays are exponentials of non-positive numbers.
// State, cumulative sums and all scalings are 32-bit.
#include "common.cuh"

int tlc_ssm_state_pass_launch(const float* chunk_decay, float* state, float* chunk_state, const int* seq_seg_start,
                              const int* slots, const int* start_pos, int B, int Hs, int PN, int write_final,
                              cudaStream_t stream);

namespace {

constexpr int Q = 128;       // rows per chunk (SCAN_CHUNK of the engine)

__device__ __forceinline__ uint32_t tf32(float v) {
  uint32_t r;
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(v));
  return r;
}
__device__ __forceinline__ void mma_tf32(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Four 8 x 8 matrices of 16-bit elements, i.e. four blocks of 8 rows x 4 32-bit words: thread T gets word T % 4 of
// row T / 4 of each, which is the layout of the TF32 fragments wherever K runs along the rows in memory.
__device__ __forceinline__ void ldsm_x4_b32(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ uint32_t tf32_bits(uint32_t v) { return tf32(__uint_as_float(v)); }
// 2^x by the special-function unit (two units in the last place; the result becomes a TF32 operand)
__device__ __forceinline__ float ex2_quick(float x) {
  float r;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
  return r;
}

// ---- cumulative log-decay per (chunk, head) --------------------------------------------------------
// cum[t, h] = sum of dt*A over the chunk's rows up to t; chunk_decay[seg, h] = exp(cum at the last row)
__global__ void __launch_bounds__(128)
ssd_cumsum_kernel(const float* __restrict__ dt, const float* __restrict__ A, const int* __restrict__ seg_start,
                  float* __restrict__ cum, float* __restrict__ chunk_decay, int Hs) {
  tlc_pdl(dt, cum, chunk_decay);
  // a warp per (chunk, head): lane l owns rows 4l .. 4l+3 of the chunk; prefix sums by shuffles
  const int seg = blockIdx.x;
  const int h = blockIdx.y * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (h >= Hs) return;
  const int t0 = seg_start[seg], L = seg_start[seg + 1] - t0;
  const float a = A[h];
  float d[Q / 32];
#pragma unroll
  for (int u = 0; u < Q / 32; u++) {
    const int r = lane * (Q / 32) + u;
    d[u] = r < L ? dt[(size_t)(t0 + r) * Hs + h] * a : 0.f;
  }
#pragma unroll
  for (int u = 1; u < Q / 32; u++) d[u] += d[u - 1];
  float run = d[Q / 32 - 1];                            // inclusive sum of the lanes up to this one
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const float v = __shfl_up_sync(0xffffffffu, run, o);
    if (lane >= o) run += v;
  }
  const float before = run - d[Q / 32 - 1];
#pragma unroll
  for (int u = 0; u < Q / 32; u++) {
    const int r = lane * (Q / 32) + u;
    if (r < L) cum[(size_t)(t0 + r) * Hs + h] = before + d[u];
  }
  if (lane == 31) chunk_decay[(size_t)seg * Hs + h] = expf(run);   // rows past L add nothing
}

// ---- C B^T per (chunk, group): cb[seg, g, i, j] for j <= i -----------------------------------------
// grid (seg, G, 8): a block of 4 warps computes a strip of 16 rows x 128 columns, warp w the columns
// [32 w, 32 w + 32); K = N in slabs of 64.
__global__ void __launch_bounds__(128)
ssd_cb_kernel(const float* __restrict__ xbc, const int* __restrict__ seg_start, float* __restrict__ cb, int Di, int N,
              int G, int Cd) {
  tlc_pdl(xbc, cb);
  constexpr int LD = 68;
  extern __shared__ uint32_t ssd_sm[];
  uint32_t* Cs = ssd_sm;                 // [16][LD]   rows i, columns n
  uint32_t* Bs = ssd_sm + 16 * LD;       // [Q][LD]    rows j, columns n
  const int seg = blockIdx.x, g = blockIdx.y;
  const int t0 = seg_start[seg], L = seg_start[seg + 1] - t0;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, gq = lane >> 2, tq = lane & 3;
  const int i_base = blockIdx.z * 16;                      // the block's 16 rows
  if (i_base >= L) return;
  const int n_tiles = min(16, (i_base + 16 + 7) / 8);      // columns j <= i only
  const int j_rows = min(Q, n_tiles * 8);                  // rows of B that matter
  float acc[4][4];
#pragma unroll
  for (int j = 0; j < 4; j++)
#pragma unroll
    for (int k = 0; k < 4; k++) acc[j][k] = 0.f;
  const float* Bg = xbc + Di + (size_t)g * N;
  const float* Cg = xbc + Di + (size_t)G * N + (size_t)g * N;
  for (int n0 = 0; n0 < N; n0 += 64) {
    __syncthreads();
    // 16 float4 per row; all loads of a batch are issued before the first conversion
#pragma unroll 1
    for (int it0 = 0; it0 < 16; it0 += 8) {
      float4 bv[8], cv[8];
#pragma unroll
      for (int u = 0; u < 8; u++) {
        const int idx = threadIdx.x + (it0 + u) * 128;
        const int r = idx >> 4, c4 = (idx & 15) * 4;
        bv[u] = cv[u] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (r < L && r < j_rows && n0 + c4 < N) bv[u] = *reinterpret_cast<const float4*>(Bg + (size_t)(t0 + r) * Cd + n0 + c4);
        const int ri = i_base + r;
        if (r < 16 && ri < L && n0 + c4 < N) cv[u] = *reinterpret_cast<const float4*>(Cg + (size_t)(t0 + ri) * Cd + n0 + c4);
      }
#pragma unroll
      for (int u = 0; u < 8; u++) {
        const int idx = threadIdx.x + (it0 + u) * 128;
        const int r = idx >> 4, c4 = (idx & 15) * 4;
        uint32_t* bd = Bs + r * LD + c4;
        bd[0] = tf32(bv[u].x); bd[1] = tf32(bv[u].y); bd[2] = tf32(bv[u].z); bd[3] = tf32(bv[u].w);
        if (r < 16) {
          uint32_t* cd = Cs + r * LD + c4;
          cd[0] = tf32(cv[u].x); cd[1] = tf32(cv[u].y); cd[2] = tf32(cv[u].z); cd[3] = tf32(cv[u].w);
        }
      }
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < 8; kk++) {
      const uint32_t* ar = Cs + gq * LD + kk * 8 + tq;
      const uint32_t a0 = ar[0], a1 = ar[8 * LD], a2 = ar[4], a3 = ar[8 * LD + 4];
#pragma unroll
      for (int j = 0; j < 4; j++) {
        if (warp * 4 + j < n_tiles) {
          const uint32_t* br = Bs + ((warp * 4 + j) * 8 + gq) * LD + kk * 8 + tq;
          mma_tf32(acc[j], a0, a1, a2, a3, br[0], br[4]);
        }
      }
    }
  }
  float* out = cb + (((size_t)seg * G + g) * Q) * Q;
#pragma unroll
  for (int j = 0; j < 4; j++) {
    if (warp * 4 + j < n_tiles) {
      const int col = (warp * 4 + j) * 8 + 2 * tq;
      *reinterpret_cast<float2*>(out + (size_t)(i_base + gq) * Q + col) = make_float2(acc[j][0], acc[j][1]);
      *reinterpret_cast<float2*>(out + (size_t)(i_base + gq + 8) * Q + col) = make_float2(acc[j][2], acc[j][3]);
    }
  }
}

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, bool pred) {
  const int bytes = pred ? 16 : 0;                 // 0: the 16 bytes are filled with zeros, nothing is read
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N_> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N_) : "memory"); }

// ---- chunk states: S_c[p, n] = sum_j w_j x[j, p] B[j, n],  w_j = exp(cum_last - cum_j) dt_j ----------
// grid (seg, Hs, N / 128); 8 warps; output P x 128 with K = 128 rows of the chunk.  x and B arrive as they
// are, by cp.async, all at once; the weights w_j are computed meanwhile.  x is then scaled by them and rounded
// to TF32 once, in place (the kernel is bound by instruction issue: every warp needs every x fragment);
// B is rounded in registers.  A warp owns half of the head's rows and 32 of the columns.
template <int P>
__global__ void __launch_bounds__(256)
ssd_chunk_state_kernel(const float* __restrict__ xbc, const float* __restrict__ dt, const float* __restrict__ cum,
                       const int* __restrict__ seg_start, float* __restrict__ chunk_state, int Hs, int N, int G, int Cd) {
  tlc_pdl(xbc, dt, cum, chunk_state);
  constexpr int LDX = P + 8, LDB = 128 + 8;
  extern __shared__ __align__(16) uint32_t ssd_sm[];
  float* Xs = reinterpret_cast<float*>(ssd_sm);     // [j][p]   raw x
  float* Bs = Xs + Q * LDX;                         // [j][n]   128 columns of B, raw
  float* ws = Bs + Q * LDB;                         // [j]      w_j
  const int seg = blockIdx.x, h = blockIdx.y, nb = blockIdx.z * 128;
  const int g = h / (Hs / G);
  const int Di = Hs * P;
  const int t0 = seg_start[seg], L = seg_start[seg + 1] - t0;
  const int tid = threadIdx.x;
  const uint32_t xs0 = (uint32_t)__cvta_generic_to_shared(Xs), bs0 = (uint32_t)__cvta_generic_to_shared(Bs);
  for (int idx = tid; idx < Q * (P / 4); idx += 256) {
    const int r = idx / (P / 4), c4 = (idx % (P / 4)) * 4;
    const bool in = r < L;
    cp_async16(xs0 + (uint32_t)(r * LDX + c4) * 4, xbc + (size_t)(t0 + (in ? r : 0)) * Cd + (size_t)h * P + c4, in);
  }
  for (int idx = tid; idx < Q * 32; idx += 256) {
    const int r = idx >> 5, c4 = (idx & 31) * 4;
    const bool in = r < L && nb + c4 < N;
    cp_async16(bs0 + (uint32_t)(r * LDB + c4) * 4,
               xbc + (size_t)(t0 + (r < L ? r : 0)) * Cd + Di + (size_t)g * N + (in ? nb + c4 : 0), in);
  }
  cp_async_commit();
  if (tid < Q) {
    float w = 0.f;
    if (tid < L) {
      const float cum_last = cum[(size_t)(t0 + L - 1) * Hs + h];
      w = expf(cum_last - cum[(size_t)(t0 + tid) * Hs + h]) * dt[(size_t)(t0 + tid) * Hs + h];
    }
    ws[tid] = w;
  }
  cp_async_wait<0>();
  __syncthreads();
  // x times its row's weight, rounded to TF32, once and in place: every warp reads it from there
  uint32_t* Xt = reinterpret_cast<uint32_t*>(Xs);
  for (int idx = tid; idx < Q * (P / 4); idx += 256) {
    const int r = idx / (P / 4), c4 = (idx % (P / 4)) * 4;
    const float4 v = *reinterpret_cast<const float4*>(Xs + r * LDX + c4);
    const float wr = ws[r];
    *reinterpret_cast<uint4*>(Xt + r * LDX + c4) = make_uint4(tf32(v.x * wr), tf32(v.y * wr), tf32(v.z * wr), tf32(v.w * wr));
  }
  __syncthreads();
  const int warp = tid >> 5, lane = tid & 31, gq = lane >> 2, tq = lane & 3;
  // warp w: rows p of half w & 1 of the head (P/32 tiles) x columns n in [32 (w >> 1), +32) (4 tiles)
  constexpr int MT = P / 32;
  const int p0 = (warp & 1) * (P / 2), n_w = (warp >> 1) * 32;
  float acc[MT][4][4];
#pragma unroll
  for (int m = 0; m < MT; m++)
#pragma unroll
    for (int jn = 0; jn < 4; jn++)
#pragma unroll
      for (int k = 0; k < 4; k++) acc[m][jn][k] = 0.f;
#pragma unroll 4
  for (int kk = 0; kk < Q / 8; kk++) {
    uint32_t b[4][2];
#pragma unroll
    for (int jn = 0; jn < 4; jn++) {
      const float* br = Bs + (kk * 8 + tq) * LDB + n_w + jn * 8 + gq;
      b[jn][0] = tf32(br[0]);
      b[jn][1] = tf32(br[4 * LDB]);
    }
#pragma unroll
    for (int m = 0; m < MT; m++) {
      const uint32_t* ar = Xt + (kk * 8 + tq) * LDX + p0 + m * 16 + gq;               // A(row p, col j) = x[j][p] w_j
      const uint32_t a0 = ar[0], a1 = ar[8], a2 = ar[4 * LDX], a3 = ar[4 * LDX + 8];
#pragma unroll
      for (int jn = 0; jn < 4; jn++) mma_tf32(acc[m][jn], a0, a1, a2, a3, b[jn][0], b[jn][1]);
    }
  }
  float* out = chunk_state + (((size_t)seg * Hs + h) * P) * N;
#pragma unroll
  for (int m = 0; m < MT; m++)
#pragma unroll
    for (int jn = 0; jn < 4; jn++) {
      const int n = nb + n_w + jn * 8 + 2 * tq;
      if (n < N) {
        *reinterpret_cast<float2*>(out + (size_t)(p0 + m * 16 + gq) * N + n) = make_float2(acc[m][jn][0], acc[m][jn][1]);
        *reinterpret_cast<float2*>(out + (size_t)(p0 + m * 16 + gq + 8) * N + n) = make_float2(acc[m][jn][2], acc[m][jn][3]);
      }
    }
}

// ---- chunk outputs ------------------------------------------------------------------------------------
// grid (seg, Hs, 2); a block of 8 warps owns 64 rows of the chunk: warp w has rows [16 (w & 3), +16) and
// the columns of half w >> 2 of the head.
//   acc  = M X,        M[i,j] = cb[i,j] exp(cum_i - cum_j) dt_j (j <= i),  X[j,p] = x[j,p]
//   acc2 = C S_in^T    (the state the chunk starts from), scaled by exp(cum_i) at the end
//   y = acc + exp(cum_i) acc2 + D x
// M is built in shared memory by the block (it needs the exponentials); X, C and S_in arrive as they
// are, by cp.async, and are rounded to TF32 in registers: X and the first slab of 32 state columns
// are on their way while M is built, and each further slab while the one before it is multiplied.
constexpr int OUT_R = 64;                  // rows of the chunk per block
constexpr int OUT_SL = 32;                 // state columns per slab
constexpr int OUT_LDM = Q + 4, OUT_LDS = OUT_SL + 4;

template <int P>
__global__ void __launch_bounds__(256)
ssd_chunk_out_kernel(const float* __restrict__ xbc, const float* __restrict__ dt, const float* __restrict__ cum,
                     const float* __restrict__ cb, const float* __restrict__ s_in, const float* __restrict__ Dskip,
                     const int* __restrict__ seg_start, float* __restrict__ y, int Hs, int N, int G, int Cd) {
  tlc_pdl(xbc, dt, cum, cb, s_in, y);
  constexpr int R = OUT_R, LDM = OUT_LDM, LDX = P + 8, LDS = OUT_LDS, SL = OUT_SL;
  constexpr int NT = P / 16;               // 8-column tiles of a warp's half of the head
  extern __shared__ __align__(16) uint32_t ssd_sm[];
  uint32_t* Ms = ssd_sm;                   // [R][j]            TF32
  float* Xs = reinterpret_cast<float*>(Ms + R * LDM);        // [j][p]            raw
  float* Cb = Xs + Q * LDX;                // [2][R][slab]      raw
  float* Sb = Cb + 2 * R * LDS;            // [2][p][slab]      raw
  float* cums = Sb + 2 * P * LDS;          // [Q]
  float* dts = cums + Q;                   // [Q]
  const int seg = blockIdx.x, h = blockIdx.y, r0 = blockIdx.z * R;
  const int g = h / (Hs / G);
  const int Di = Hs * P;
  const int t0 = seg_start[seg], L = seg_start[seg + 1] - t0;
  if (r0 >= L) return;
  const int jmax = min(L, r0 + R);         // columns j < jmax matter for these rows
  const int tid = threadIdx.x;
  const float* Cg = xbc + Di + (size_t)G * N + (size_t)g * N;
  const float* Sg = s_in + (((size_t)seg * Hs + h) * P) * N;
  const uint32_t xs0 = (uint32_t)__cvta_generic_to_shared(Xs), cb0 = (uint32_t)__cvta_generic_to_shared(Cb),
                 sb0 = (uint32_t)__cvta_generic_to_shared(Sb);
  // X: rows j < jmax, zeros below
  for (int idx = tid; idx < Q * (P / 4); idx += 256) {
    const int r = idx / (P / 4), c4 = (idx % (P / 4)) * 4;
    const bool in = r < jmax;
    cp_async16(xs0 + (uint32_t)(r * LDX + c4) * 4, xbc + (size_t)(t0 + (in ? r : 0)) * Cd + (size_t)h * P + c4, in);
  }
  cp_async_commit();
  auto fetch_slab = [&](int n0, int buf) {
    for (int idx = tid; idx < R * (SL / 4); idx += 256) {           // C rows of this block
      const int rl = idx / (SL / 4), c4 = (idx % (SL / 4)) * 4;
      const bool in = r0 + rl < L;
      cp_async16(cb0 + (uint32_t)((buf * R + rl) * LDS + c4) * 4, Cg + (size_t)(t0 + (in ? r0 + rl : 0)) * Cd + n0 + c4, in);
    }
    for (int idx = tid; idx < P * (SL / 4); idx += 256) {           // the incoming state
      const int p = idx / (SL / 4), c4 = (idx % (SL / 4)) * 4;
      cp_async16(sb0 + (uint32_t)((buf * P + p) * LDS + c4) * 4, Sg + (size_t)p * N + n0 + c4, true);
    }
    cp_async_commit();
  };
  fetch_slab(0, 0);
  if (tid < Q) {
    const int r = min(tid, L - 1);
    cums[tid] = cum[(size_t)(t0 + r) * Hs + h] * 1.4426950408889634f;      // in powers of two from here on
    dts[tid] = tid < L ? dt[(size_t)(t0 + tid) * Hs + h] : 0.f;
  }
  __syncthreads();
  // M: R rows x 32 float4, 8 loads in flight per thread
  const float* cbg = cb + (((size_t)seg * G + g) * Q) * Q;
  {
    float4 v[8];
#pragma unroll
    for (int u = 0; u < 8; u++) {
      const int idx = tid + u * 256;
      const int i = r0 + (idx >> 5), j4 = (idx & 31) * 4;
      v[u] = (j4 <= i && i < L) ? *reinterpret_cast<const float4*>(cbg + (size_t)i * Q + j4) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
#pragma unroll
    for (int u = 0; u < 8; u++) {
      const int idx = tid + u * 256;
      const int il = idx >> 5, i = r0 + il, j4 = (idx & 31) * 4;
      uint4 d = make_uint4(0u, 0u, 0u, 0u);
      if (j4 <= i && i < L) {
        const float ci = cums[i];
        const float4 cj = *reinterpret_cast<const float4*>(cums + j4), dj = *reinterpret_cast<const float4*>(dts + j4);
        d.x = tf32(v[u].x * ex2_quick(ci - cj.x) * dj.x);
        if (j4 + 1 <= i) d.y = tf32(v[u].y * ex2_quick(ci - cj.y) * dj.y);
        if (j4 + 2 <= i) d.z = tf32(v[u].z * ex2_quick(ci - cj.z) * dj.z);
        if (j4 + 3 <= i) d.w = tf32(v[u].w * ex2_quick(ci - cj.w) * dj.w);
      }
      *reinterpret_cast<uint4*>(Ms + il * LDM + j4) = d;
    }
  }
  cp_async_wait<1>();                      // X has arrived (the first slab may still be on its way)
  __syncthreads();
  const int warp = tid >> 5, lane = tid & 31, gq = lane >> 2, tq = lane & 3;
  const int il_base = (warp & 3) * 16, i_base = r0 + il_base, p_base = (warp >> 2) * (P / 2);
  float acc[NT][4], acc2[NT][4];
#pragma unroll
  for (int j = 0; j < NT; j++)
#pragma unroll
    for (int k = 0; k < 4; k++) acc[j][k] = acc2[j][k] = 0.f;
  // inside the chunk: columns j <= i only
  const int k_steps = (i_base + 16) / 8;
  for (int kk = 0; kk < k_steps; kk++) {
    const uint32_t* ar = Ms + (il_base + gq) * LDM + kk * 8 + tq;
    const uint32_t a0 = ar[0], a1 = ar[8 * LDM], a2 = ar[4], a3 = ar[8 * LDM + 4];
#pragma unroll
    for (int j = 0; j < NT; j++) {
      const float* br = Xs + (kk * 8 + tq) * LDX + p_base + j * 8 + gq;
      mma_tf32(acc[j], a0, a1, a2, a3, tf32(br[0]), tf32(br[4 * LDX]));
    }
  }
  // what came before the chunk: C times the incoming state, a slab of state columns at a time
  const int n_slabs = N / SL;
  for (int sl = 0; sl < n_slabs; sl++) {
    cp_async_wait<0>();
    __syncthreads();                       // slab sl is in shared memory; everybody is done with slab sl-1
    if (sl + 1 < n_slabs) fetch_slab((sl + 1) * SL, (sl + 1) & 1);
    // C and the state have K (the state column) along their rows: whole fragments come by ldmatrix
    const uint32_t cs_u = cb0 + (uint32_t)((sl & 1) * R * LDS) * 4, ss_u = sb0 + (uint32_t)((sl & 1) * P * LDS) * 4;
#pragma unroll
    for (int kk = 0; kk < SL / 8; kk++) {
      uint32_t a0, a1, a2, a3;     // rows 0-7 | 8-15 of the warp's strip, columns kk*8 + (0-3 | 4-7)
      ldsm_x4_b32(cs_u + (uint32_t)((il_base + (lane & 7) + ((lane >> 3) & 1) * 8) * LDS + kk * 8 + (lane >> 4) * 4) * 4, a0, a1, a2, a3);
      a0 = tf32_bits(a0); a1 = tf32_bits(a1); a2 = tf32_bits(a2); a3 = tf32_bits(a3);
#pragma unroll
      for (int jp = 0; jp < NT / 2; jp++) {
        uint32_t b00, b01, b10, b11;   // B(k = n, col = p) = S_in[p][n]: rows p of two tiles, columns kk*8 + (0-3 | 4-7)
        ldsm_x4_b32(ss_u + (uint32_t)((p_base + jp * 16 + (lane & 7) + (lane >> 4) * 8) * LDS + kk * 8 + ((lane >> 3) & 1) * 4) * 4,
                    b00, b01, b10, b11);
        mma_tf32(acc2[2 * jp], a0, a1, a2, a3, tf32_bits(b00), tf32_bits(b01));
        mma_tf32(acc2[2 * jp + 1], a0, a1, a2, a3, tf32_bits(b10), tf32_bits(b11));
      }
    }
  }
  const float Dh = Dskip[h];
#pragma unroll
  for (int r = 0; r < 2; r++) {
    const int i = i_base + gq + 8 * r;
    if (i < L) {
      const float e = exp2f(cums[i]);
#pragma unroll
      for (int j = 0; j < NT; j++) {
        const int p = p_base + j * 8 + 2 * tq;
        const float2 xv = *reinterpret_cast<const float2*>(Xs + i * LDX + p);
        *reinterpret_cast<float2*>(y + (size_t)(t0 + i) * Di + (size_t)h * P + p) =
            make_float2(acc[j][2 * r] + e * acc2[j][2 * r] + Dh * xv.x, acc[j][2 * r + 1] + e * acc2[j][2 * r + 1] + Dh * xv.y);
      }
    }
  }
}

// The state after a sequence's last chunk, decay * S_in + S_c, is what the carry would hand to a
// next chunk; the carry kernel (ssm_state_pass_kernel in mamba.cu) writes it to the slot.

inline size_t pad64(size_t n) { return (n + 63) / 64 * 64; }

template <int P> size_t state_smem() { return (size_t)(Q * (P + 8) + Q * 136 + Q) * 4; }
template <int P> size_t out_smem() {
  return (size_t)(OUT_R * OUT_LDM + Q * (P + 8) + 2 * OUT_R * OUT_LDS + 2 * P * OUT_LDS + 2 * Q) * 4;
}

template <int P> int configure() {
  if (cudaFuncSetAttribute(ssd_chunk_state_kernel<P>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)state_smem<P>()) != cudaSuccess ||
      cudaFuncSetAttribute(ssd_chunk_out_kernel<P>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)out_smem<P>()) != cudaSuccess)
    return tlc_fail(-2, "ssm_scan(chunked): cannot reserve shared memory");
  return 0;
}

template <int P>
int run(const float* xbc, const float* dt, const float* A, const float* Dskip, float* state, float* scratch,
        const int* seg_start, const int* seg_seq, const int* seq_seg_start, const int* slots, const int* start_pos, float* y,
        int B, int n_seg, int T, int Hs, int N, int G, int Cd, cudaStream_t stream) {
  const int Di = Hs * P;
  // every part starts on a 256-byte boundary of the scratch (float4 loads need 16)
  float* chunk_state = scratch;                                          // [n_seg, Hs, P, N]
  float* chunk_decay = chunk_state + pad64((size_t)n_seg * Hs * P * N);  // [n_seg, Hs]
  float* cum = chunk_decay + pad64((size_t)n_seg * Hs);                  // [T, Hs]
  float* cb = cum + pad64((size_t)T * Hs);                               // [n_seg, G, Q, Q]
  tlc_launch(ssd_cumsum_kernel, dim3(n_seg, (Hs + 3) / 4), dim3(128), 0, stream, dt, A, seg_start, cum, chunk_decay, Hs);
  tlc_launch(ssd_cb_kernel, dim3(n_seg, G, Q / 16), dim3(128), (16 + Q) * 68 * 4, stream, xbc, seg_start, cb, Di, N, G, Cd);
  tlc_launch(ssd_chunk_state_kernel<P>, dim3(n_seg, Hs, (N + 127) / 128), dim3(256), state_smem<P>(), stream, xbc, dt,
             (const float*)cum, seg_start, chunk_state, Hs, N, G, Cd);
  TLC_CHECK_LAUNCH("ssm_scan(chunk states)");
  if (int rc = tlc_ssm_state_pass_launch(chunk_decay, state, chunk_state, seq_seg_start, slots, start_pos, B, Hs, P * N, 1, stream))
    return rc;
  tlc_launch(ssd_chunk_out_kernel<P>, dim3(n_seg, Hs, 2), dim3(256), out_smem<P>(), stream, xbc, dt, (const float*)cum,
             (const float*)cb, (const float*)chunk_state, Dskip, seg_start, y, Hs, N, G, Cd);
  TLC_CHECK_LAUNCH("ssm_scan(chunk outputs)");
  return 0;
}

}  // namespace

extern "C" int tlc_ssd_init() {
  if (cudaFuncSetAttribute(ssd_cb_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (16 + Q) * 68 * 4) != cudaSuccess)
    return tlc_fail(-2, "ssm_scan(chunked): cannot reserve shared memory");
  if (int rc = configure<64>()) return rc;
  return configure<128>();
}

// Sizes this form is built for: head size 64 or 128, state size a multiple of 64, 16-byte aligned rows.
extern "C" int tlc_ssd_ok(int Hs, int P, int N, int G, int Cd) {
  return (P == 64 || P == 128) && N % 64 == 0 && N >= 64 && Cd % 4 == 0 && G > 0 && Hs % G == 0;
}

// floats of scratch for n_seg chunks of T rows in all
extern "C" long long tlc_ssd_scratch_floats(int n_seg, int T, int Hs, int P, int N, int G) {
  return (long long)(pad64((size_t)n_seg * Hs * P * N) + pad64((size_t)n_seg * Hs) + pad64((size_t)T * Hs) +
                     pad64((size_t)n_seg * G * Q * Q));
}

extern "C" int tlc_ssm_scan_ssd(const float* xbc, const float* dt, const float* A, const float* Dskip, float* state,
                                float* scratch, const int* seg_start, const int* seg_seq, const int* seq_seg_start,
                                const int* slots, const int* start_pos, float* y, int B, int n_seg, int T, int Hs, int P,
                                int N, int G, int Cd, cudaStream_t stream) {
  if (B == 0 || n_seg == 0) return 0;
  TLC_REQUIRE(tlc_ssd_ok(Hs, P, N, G, Cd), "ssm_scan(chunked, tensor cores): sizes Hs=%d P=%d N=%d G=%d are not built", Hs, P, N, G);
  TLC_REQUIRE(Hs <= 65535 && G <= 65535, "ssm_scan: too many heads or groups");
  if (P == 64)
    return run<64>(xbc, dt, A, Dskip, state, scratch, seg_start, seg_seq, seq_seg_start, slots, start_pos, y, B, n_seg, T, Hs, N, G, Cd, stream);
  return run<128>(xbc, dt, A, Dskip, state, scratch, seg_start, seg_seq, seq_seg_start, slots, start_pos, y, B, n_seg, T, Hs, N, G, Cd, stream);
}
