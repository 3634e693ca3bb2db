// Selective scan of prompts in chunked matrix form, on the tensor cores, with the state kept on chip.
//
// The recurrence is the reference's (cpu_op.c:932-951):
//     S_t = S_{t-1} * exp(dt_t A) + (dt_t x_t) (x) B_t ,   y_t = S_t . C_t + D x_t
// Over a chunk of rows i, j (L <= 128) with cum_i = sum_{k<=i} dt_k A this is three products:
//     y_i  = sum_{j<=i} (C_i . B_j) exp(cum_i - cum_j) dt_j x_j        "inside the chunk"
//          + exp(cum_i) * (S_in C_i)                                  "what came before"
//          + D x_i
//     S_out = exp(cum_last) S_in + sum_j exp(cum_last - cum_j) dt_j x_j (x) B_j
// The kernels:
//   ssd_cb_kernel    C B^T of every (chunk, group), shared by the group's heads (bfloat16 in and out); for the walk
//                    on tcgen05 also B transposed and, in blocks of their own, the rows' decays;
//   ssd_intra_kernel (with the walk on tcgen05) the first and third terms of y for every (chunk, head) at once:
//                    they need no state, so they stand beside the walk, on a second stream where there is one;
//   ssd_walk_kernel  one block per (sequence, head, 32 rows p of the head) walks the sequence's chunks in
//                    order.  The state S[32, N] lives in the accumulator registers of the last product from
//                    the slot's state before the first chunk to the slot's state after the last; it is never
//                    written to global memory in between.  Per chunk: the state goes to shared memory in
//                    bfloat16 for C S^T; the score matrix M[i, j] = cb exp(cum_i - cum_j) dt_j is built in
//                    registers, as the operand fragments of M X, by the warp that owns rows i; x scaled by
//                    its row's weight is the operand of the state update.  C, C B^T and B of the next chunk
//                    arrive by cp.async while the current chunk is multiplied (each buffer is refilled as soon
//                    as its product is done).
// Products are mma.sync.m16n8k16 with bfloat16 operands and 32-bit accumulation.  Cumulative sums, decay
// factors, the carried state, D x and every accumulator are 32-bit; decays are exponentials of non-positive
// numbers.  The 32-bit path of the library never comes here (mamba.cu has its three-pass scan).
#include "common.cuh"

// the same walk with tcgen05.mma and the state in tensor memory (mamba_ssd_tc.cu), for states of 128 or 256 columns
int tlc_ssd_tc_init();
int tlc_ssd_tc_run(const __nv_bfloat16* xbc, const float* row_w, const float* row_e, const float* seg_decay,
                   __nv_bfloat16* bt, float* state, const int* seg_start, const int* seq_seg_start, const int* slots,
                   const int* start_pos, float* y, int add_to_y, int B, int n_seg, int T, int Hs, int P, int N, int G, int Cd,
                   cudaStream_t stream);

namespace {

constexpr int Q = 128;       // rows per chunk
constexpr int PB = 32;       // rows p of a head per block of the walk
constexpr float LOG2E = 1.4426950408889634f;

__device__ __forceinline__ void mma_bf16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x2_t(uint32_t addr, uint32_t& r0, uint32_t& r1) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0,%1}, [%2];" : "=r"(r0), "=r"(r1) : "r"(addr));
}
__device__ __forceinline__ float ex2_quick(float x) {     // 2^x by the special-function unit
  float r;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
  return r;
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&v);
}
__device__ __forceinline__ float2 unpack_bf16(uint32_t v) {
  return make_float2(__uint_as_float(v << 16), __uint_as_float(v & 0xffff0000u));
}
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, bool pred) {
  const int bytes = pred ? 16 : 0;                 // 0: the 16 bytes are filled with zeros, nothing is read
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N_> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N_) : "memory"); }

// Rows in shared memory are padded by 16 bytes: the row strides used here are then 16 or 80 modulo 128, so that
// the eight rows an ldmatrix reads lie in eight different 16-byte columns of the banks.
__host__ __device__ constexpr int padded(int row_bytes) { return row_bytes + 16; }

// ---- C B^T per (chunk, group): cb[seg, g, i, j] for j <= i (bfloat16) -------------------------------------
// grid (seg, G, 2), 4 warps: a block owns 64 rows i, warp w the rows [16 w, 16 w + 16) of them and the columns
// j up to its diagonal; K = N.  With bt (the walk on tcgen05 wants B transposed) the grid has N / 64 more blocks
// along z, each of which writes bt[seg, g, n, j] = B[row j of the chunk, n] for 64 columns n (zero past the chunk),
// and from z_decay on blocks that scan the decays of the chunk's rows for four heads each.
__global__ void __launch_bounds__(128)
ssd_cb_kernel(const __nv_bfloat16* __restrict__ xbc, const int* __restrict__ seg_start, __nv_bfloat16* __restrict__ cb,
              __nv_bfloat16* __restrict__ bt, int Di, int N, int G, int Cd, const float* __restrict__ dt,
              const float* __restrict__ A, int Hs, float* __restrict__ row_w, float* __restrict__ row_e,
              float* __restrict__ seg_decay, int z_decay) {
  tlc_pdl(xbc, cb, bt, dt, row_w, row_e, seg_decay);
  extern __shared__ __align__(16) unsigned char ssd_sm[];
  if (z_decay > 0 && (int)blockIdx.z >= z_decay) {
    // The rows' decays for the walk, four heads of the group a block (a warp each): for row i of the chunk the
    // cumulative log2 decay cum_i, then its weight in the chunk's state update w = 2^(total - cum) dt, its factor
    // e = 2^cum on C S^T, and the chunk's decay 2^total.  A lane takes four consecutive rows.
    const int seg = blockIdx.x, g = blockIdx.y, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int hg = 4 * ((int)blockIdx.z - z_decay) + warp;
    if (hg >= Hs / G) return;
    const int h = g * (Hs / G) + hg;
    const int t0 = seg_start[seg], L = seg_start[seg + 1] - t0;
    const float a_log2 = A[h] * LOG2E;
    float d[4], c[4];
    float run = 0.f;
#pragma unroll
    for (int k = 0; k < 4; k++) {
      const int i = 4 * lane + k;
      d[k] = i < L ? dt[(size_t)(t0 + i) * Hs + h] : 0.f;
      run += d[k] * a_log2;
      c[k] = run;
    }
    float incl = run;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const float u = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += u;
    }
    const float before = incl - run, total = __shfl_sync(0xffffffffu, incl, 31);
#pragma unroll
    for (int k = 0; k < 4; k++) {
      const int i = 4 * lane + k;
      if (i < L) {
        const float cum = before + c[k];
        row_w[(size_t)(t0 + i) * Hs + h] = ex2_quick(total - cum) * d[k];
        row_e[(size_t)(t0 + i) * Hs + h] = ex2_quick(cum);
      }
    }
    if (lane == 0) seg_decay[(size_t)seg * Hs + h] = exp2f(total);
    return;
  }
  if (blockIdx.z >= 2) {
    unsigned short (*tile)[64 + 2] = reinterpret_cast<unsigned short (*)[64 + 2]>(ssd_sm);     // [Q][66]
    const int seg = blockIdx.x, g = blockIdx.y, n0 = (blockIdx.z - 2) * 64;
    const int t0 = seg_start[seg], L = seg_start[seg + 1] - t0;
    const unsigned short* Bg = reinterpret_cast<const unsigned short*>(xbc) + Di + (size_t)g * N + n0;
    for (int idx = threadIdx.x; idx < Q * 32; idx += 128) {
      const int j = idx >> 5, c = (idx & 31) * 2;
      uint32_t v = 0;
      if (j < L) v = *reinterpret_cast<const uint32_t*>(Bg + (size_t)(t0 + j) * Cd + c);
      tile[j][c] = (unsigned short)(v & 0xffffu);
      tile[j][c + 1] = (unsigned short)(v >> 16);
    }
    __syncthreads();
    unsigned short* out = reinterpret_cast<unsigned short*>(bt) + (((size_t)seg * G + g) * N + n0) * Q;
    for (int idx = threadIdx.x; idx < 64 * (Q / 2); idx += 128) {
      const int n = idx / (Q / 2), j = (idx % (Q / 2)) * 2;
      *reinterpret_cast<uint32_t*>(out + (size_t)n * Q + j) = (uint32_t)tile[j][n] | ((uint32_t)tile[j + 1][n] << 16);
    }
    return;
  }
  const int LDN = padded(N * 2);
  unsigned char* Cs = ssd_sm;                     // [64][LDN]   rows i
  unsigned char* Bs = ssd_sm + 64 * LDN;          // [Q][LDN]    rows j
  const int seg = blockIdx.x, g = blockIdx.y, i_blk = blockIdx.z * 64;
  const int t0 = seg_start[seg], L = seg_start[seg + 1] - t0;
  if (i_blk >= L) return;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, gq = lane >> 2, tq = lane & 3;
  const int j_rows = min(L, i_blk + 64);          // rows of B that matter
  const __nv_bfloat16* Bg = xbc + Di + (size_t)g * N;
  const __nv_bfloat16* Cg = xbc + Di + (size_t)G * N + (size_t)g * N;
  const uint32_t cs0 = (uint32_t)__cvta_generic_to_shared(Cs), bs0 = (uint32_t)__cvta_generic_to_shared(Bs);
  const int pieces = N / 8;                       // 16-byte pieces of a row
  for (int idx = tid; idx < 64 * pieces; idx += 128) {
    const int r = idx / pieces, c = idx % pieces;
    const bool in = i_blk + r < L;
    cp_async16(cs0 + r * LDN + c * 16, Cg + (size_t)(t0 + (in ? i_blk + r : 0)) * Cd + c * 8, in);
  }
  for (int idx = tid; idx < Q * pieces; idx += 128) {
    const int r = idx / pieces, c = idx % pieces;
    const bool in = r < j_rows;
    cp_async16(bs0 + r * LDN + c * 16, Bg + (size_t)(t0 + (in ? r : 0)) * Cd + c * 8, in);
  }
  cp_async_commit();
  cp_async_wait<0>();
  __syncthreads();
  const int i_base = i_blk + warp * 16;           // the warp's 16 rows
  if (i_base >= L) return;
  const int n_pairs = (i_base + 16) / 16;         // pairs of 8-column tiles up to and including the diagonal
  float acc[16][4];
#pragma unroll
  for (int j = 0; j < 16; j++)
#pragma unroll
    for (int k = 0; k < 4; k++) acc[j][k] = 0.f;
  const uint32_t a_addr = cs0 + (warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * LDN + (lane >> 4) * 16;
  const uint32_t b_addr = bs0 + ((lane & 7) + (lane >> 4) * 8) * LDN + ((lane >> 3) & 1) * 16;
  for (int ks = 0; ks < N / 16; ks++) {
    uint32_t a0, a1, a2, a3;
    ldsm_x4(a_addr + ks * 32, a0, a1, a2, a3);
#pragma unroll
    for (int jp = 0; jp < 8; jp++) {
      if (jp < n_pairs) {
        uint32_t b0, b1, b2, b3;
        ldsm_x4(b_addr + jp * 16 * LDN + ks * 32, b0, b1, b2, b3);
        mma_bf16(acc[2 * jp], a0, a1, a2, a3, b0, b1);
        mma_bf16(acc[2 * jp + 1], a0, a1, a2, a3, b2, b3);
      }
    }
  }
  __nv_bfloat16* out = cb + (((size_t)seg * G + g) * Q) * Q;
#pragma unroll
  for (int jp = 0; jp < 8; jp++) {
    if (jp < n_pairs) {
#pragma unroll
      for (int u = 0; u < 2; u++) {
        const int col = (2 * jp + u) * 8 + 2 * tq;
        *reinterpret_cast<uint32_t*>(out + (size_t)(i_base + gq) * Q + col) = pack_bf16(acc[2 * jp + u][0], acc[2 * jp + u][1]);
        *reinterpret_cast<uint32_t*>(out + (size_t)(i_base + gq + 8) * Q + col) = pack_bf16(acc[2 * jp + u][2], acc[2 * jp + u][3]);
      }
    }
  }
}

// ---- the part of a chunk's outputs that needs no state: y = M x + D x ------------------------------------
// M[i, j] = cb[i, j] 2^(cum_i - cum_j) dt_j for j <= i.  grid (seg, Hs, P / PBI), 4 warps: every chunk of every
// sequence at once, so that the walk that follows has only the state's share on its path.  Warp w owns the 16-row
// tiles w and 7 - w of the chunk (nine tiles of 16 columns j up to their diagonals between them).  M is never
// stored: a thread computes the elements of its mma.sync A fragment from C B^T, read in the fragment's own
// pattern (the matrix of a chunk is 32 KB and shared by all heads of its group), and the cumulative sums; x [j, p]
// lies in shared memory as it lies in x|B|C, and ldmatrix.trans turns it into B fragments.
template <int PBI>
__global__ void __launch_bounds__(128, 6)
ssd_intra_kernel(const __nv_bfloat16* __restrict__ xbc, const float* __restrict__ dt, const float* __restrict__ A,
                 const float* __restrict__ Dskip, const __nv_bfloat16* __restrict__ cb, const int* __restrict__ seg_start,
                 float* __restrict__ y, int Hs, int P, int G, int Cd) {
  tlc_pdl(xbc, dt, cb, y);
  constexpr int LDX = padded(PBI * 2);                    // bytes per row of the x tile
  constexpr int NT = PBI / 8;
  __shared__ __align__(16) unsigned char xs[Q * LDX];
  __shared__ __align__(16) float cums[Q], ljs[Q];         // lj = cum_j - log2(dt_j): M = cb 2^(cum_i - lj)
  __shared__ float wsum[4];
  const int seg = blockIdx.x, h = blockIdx.y, p0 = blockIdx.z * PBI;
  const int g = h / (Hs / G), Di = Hs * P;
  const int t0 = seg_start[seg], L = seg_start[seg + 1] - t0;
  if (L <= 0) return;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, gq = lane >> 2, tq = lane & 3;
  const __nv_bfloat16* Xg = xbc + (size_t)h * P + p0;
  const uint32_t xs0 = (uint32_t)__cvta_generic_to_shared(xs);
  constexpr int pieces = PBI / 8;
  for (int idx = tid; idx < Q * pieces; idx += 128) {
    const int r = idx / pieces, c = idx % pieces;
    const bool in = r < L;
    cp_async16(xs0 + r * LDX + c * 16, Xg + (size_t)(t0 + (in ? r : 0)) * Cd + c * 8, in);
  }
  cp_async_commit();
  // cumulative log2 decay of the chunk's rows (row = thread)
  const float dt_reg = tid < L ? dt[(size_t)(t0 + tid) * Hs + h] : 0.f;
  float v = dt_reg * (A[h] * LOG2E);
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const float u = __shfl_up_sync(0xffffffffu, v, o);
    if (lane >= o) v += u;
  }
  if (lane == 31) wsum[warp] = v;
  __syncthreads();
  {
    float off = 0.f;
#pragma unroll
    for (int q = 0; q < 3; q++) if (q < warp) off += wsum[q];
    cums[tid] = v + off;
    ljs[tid] = v + off - log2f(dt_reg);                  // +inf past the chunk's end (dt = 0): those columns of M are 0
  }
  cp_async_wait<0>();
  __syncthreads();
  const __nv_bfloat16* cbg = cb + (((size_t)seg * G + g) * Q) * Q;
  const float Dh = Dskip[h];
#pragma unroll 1
  for (int half = 0; half < 2; half++) {
    const int rt = half == 0 ? warp : 7 - warp;
    const int r0 = 16 * rt;
    if (r0 >= L) continue;
    const int ra = r0 + gq, rb = ra + 8;
    const float ca = cums[ra], cq = cums[rb];
    float acc[NT][4];
#pragma unroll
    for (int nt = 0; nt < NT; nt++)
#pragma unroll
      for (int k = 0; k < 4; k++) acc[nt][k] = 0.f;
#pragma unroll 1
    for (int kt = 0; kt <= rt; kt++) {
      const int j0 = 16 * kt, ja = j0 + 2 * tq, jb = ja + 8;
      const uint32_t v0 = __ldg(reinterpret_cast<const uint32_t*>(cbg + (size_t)ra * Q + ja));
      const uint32_t v1 = __ldg(reinterpret_cast<const uint32_t*>(cbg + (size_t)rb * Q + ja));
      const uint32_t v2 = __ldg(reinterpret_cast<const uint32_t*>(cbg + (size_t)ra * Q + jb));
      const uint32_t v3 = __ldg(reinterpret_cast<const uint32_t*>(cbg + (size_t)rb * Q + jb));
      const float2 la = *reinterpret_cast<const float2*>(ljs + ja), lb = *reinterpret_cast<const float2*>(ljs + jb);
      const bool diag = kt == rt;
      auto elems = [&](uint32_t vv, float ci, float2 lj, int row, int col) -> uint32_t {
        const float2 m = unpack_bf16(vv);
        float e0 = m.x * ex2_quick(ci - lj.x), e1 = m.y * ex2_quick(ci - lj.y);
        if (diag) {
          if (col > row) e0 = 0.f;
          if (col + 1 > row) e1 = 0.f;
        }
        return pack_bf16(e0, e1);
      };
      const uint32_t a0 = elems(v0, ca, la, ra, ja), a1 = elems(v1, cq, la, rb, ja);
      const uint32_t a2 = elems(v2, ca, lb, ra, jb), a3 = elems(v3, cq, lb, rb, jb);
      const uint32_t b_addr = xs0 + (j0 + (lane & 15)) * LDX + (lane >> 4) * 16;
#pragma unroll
      for (int np = 0; np < NT / 2; np++) {
        uint32_t b0, b1, b2, b3;
        ldsm_x4_t(b_addr + np * 32, b0, b1, b2, b3);
        mma_bf16(acc[2 * np], a0, a1, a2, a3, b0, b1);
        mma_bf16(acc[2 * np + 1], a0, a1, a2, a3, b2, b3);
      }
    }
#pragma unroll
    for (int nt = 0; nt < NT; nt++) {
      const int col = 8 * nt + 2 * tq;
      if (ra < L) {
        const float2 x2 = unpack_bf16(*reinterpret_cast<const uint32_t*>(xs + ra * LDX + col * 2));
        *reinterpret_cast<float2*>(y + (size_t)(t0 + ra) * Di + (size_t)h * P + p0 + col) =
            make_float2(fmaf(Dh, x2.x, acc[nt][0]), fmaf(Dh, x2.y, acc[nt][1]));
      }
      if (rb < L) {
        const float2 x2 = unpack_bf16(*reinterpret_cast<const uint32_t*>(xs + rb * LDX + col * 2));
        *reinterpret_cast<float2*>(y + (size_t)(t0 + rb) * Di + (size_t)h * P + p0 + col) =
            make_float2(fmaf(Dh, x2.x, acc[nt][2]), fmaf(Dh, x2.y, acc[nt][3]));
      }
    }
  }
}

// ---- the walk over a sequence's chunks ------------------------------------------------------------------
// NT: state columns / 64 (1..4).  8 warps.  Warp w owns
//   * rows i in [16 w, 16 w + 16) of the chunk in the products that give y (all 32 columns p of the block),
//   * the state columns n in [8 NT w, 8 NT (w + 1)) in the state update (all 32 rows p).
struct WalkSmem {
  int ldn, c, b, cb, x, xw, s, f, total;          // byte offsets
  __host__ __device__ WalkSmem(int N) {
    ldn = padded(N * 2);
    c = 0;
    b = c + Q * ldn;
    cb = b + Q * ldn;
    x = cb + Q * padded(Q * 2);
    xw = x + 2 * Q * padded(PB * 2);
    s = xw + Q * padded(PB * 2);
    f = s + PB * ldn;
    total = f + (4 * Q + 8) * 4;
  }
};

template <int NT>
__global__ void __launch_bounds__(256, 1)
ssd_walk_kernel(const __nv_bfloat16* __restrict__ xbc, const float* __restrict__ dt, const float* __restrict__ A,
                const float* __restrict__ Dskip, const __nv_bfloat16* __restrict__ cb, float* __restrict__ state,
                const int* __restrict__ seg_start, const int* __restrict__ seq_seg_start, const int* __restrict__ slots,
                const int* __restrict__ start_pos, float* __restrict__ y, int Hs, int P, int G, int Cd) {
  tlc_pdl(xbc, dt, cb, state, y);
  constexpr int N = 64 * NT;
  constexpr int LDX = padded(PB * 2), LDCB = padded(Q * 2);
  const WalkSmem lay(N);
  const int LDN = lay.ldn;
  extern __shared__ __align__(16) unsigned char ssd_sm[];
  float* cums = reinterpret_cast<float*>(ssd_sm + lay.f);     // [Q] cumulative log2 decay
  float* dts = cums + Q;                                      // [Q]
  float* ws = dts + Q;                                        // [Q] weight of row j in the state update
  float* es = ws + Q;                                         // [Q] 2^cum
  float* wsum = es + Q;                                       // [4] warp totals of the prefix sum
  const uint32_t sm0 = (uint32_t)__cvta_generic_to_shared(ssd_sm);
  const uint32_t cs0 = sm0 + lay.c, bs0 = sm0 + lay.b, cb0 = sm0 + lay.cb, xs0 = sm0 + lay.x, xw0 = sm0 + lay.xw,
                 ss0 = sm0 + lay.s;
  const int b = blockIdx.x, h = blockIdx.y, p0 = blockIdx.z * PB;
  const int g = h / (Hs / G);
  const int Di = Hs * P;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, gq = lane >> 2, tq = lane & 3;
  const int c0 = seq_seg_start[b], c1 = seq_seg_start[b + 1];
  if (c1 <= c0) return;
  const float a_log2 = A[h] * LOG2E, Dh = Dskip[h];
  const __nv_bfloat16* Xg = xbc + (size_t)h * P + p0;
  const __nv_bfloat16* Bg = xbc + Di + (size_t)g * N;
  const __nv_bfloat16* Cg = xbc + Di + (size_t)G * N + (size_t)g * N;

  // ---- what moves the inputs of a chunk: three groups of copies, each into the buffer of one product ----
  auto fetch_xc = [&](int c, int buf) {            // x (this block's 32 columns) and C
    if (c < c1) {
      const int t0 = seg_start[c], L = seg_start[c + 1] - t0;
      for (int idx = tid; idx < Q * (PB / 8); idx += 256) {
        const int r = idx / (PB / 8), k = idx % (PB / 8);
        const bool in = r < L;
        cp_async16(xs0 + (buf * Q + r) * LDX + k * 16, Xg + (size_t)(t0 + (in ? r : 0)) * Cd + k * 8, in);
      }
      for (int idx = tid; idx < Q * (N / 8); idx += 256) {
        const int r = idx / (N / 8), k = idx % (N / 8);
        const bool in = r < L;
        cp_async16(cs0 + r * LDN + k * 16, Cg + (size_t)(t0 + (in ? r : 0)) * Cd + k * 8, in);
      }
    }
    cp_async_commit();
  };
  auto fetch_cb = [&](int c) {
    if (c < c1) {
      const int L = seg_start[c + 1] - seg_start[c];
      const __nv_bfloat16* src = cb + (((size_t)c * G + g) * Q) * Q;
      for (int idx = tid; idx < Q * (Q / 8); idx += 256) {
        const int r = idx / (Q / 8), k = idx % (Q / 8);
        const bool in = r < L && k * 8 <= r;        // columns beyond the diagonal's piece are never read
        cp_async16(cb0 + r * LDCB + k * 16, src + (size_t)(in ? r : 0) * Q + (in ? k * 8 : 0), in);
      }
    }
    cp_async_commit();
  };
  auto fetch_b = [&](int c) {
    if (c < c1) {
      const int t0 = seg_start[c], L = seg_start[c + 1] - t0;
      for (int idx = tid; idx < Q * (N / 8); idx += 256) {
        const int r = idx / (N / 8), k = idx % (N / 8);
        const bool in = r < L;
        cp_async16(bs0 + r * LDN + k * 16, Bg + (size_t)(t0 + (in ? r : 0)) * Cd + k * 8, in);
      }
    }
    cp_async_commit();
  };
  auto load_dt = [&](int c) -> float {             // dt of row tid of chunk c (threads 0..127)
    if (c < c1 && tid < Q) {
      const int t0 = seg_start[c], L = seg_start[c + 1] - t0;
      if (tid < L) return dt[(size_t)(t0 + tid) * Hs + h];
    }
    return 0.f;
  };

  fetch_xc(c0, 0);
  fetch_cb(c0);
  fetch_b(c0);
  float dt_reg = load_dt(c0);

  // ---- the state: rows p0 + 16 mt + gq (+ 8), columns 8 NT warp + 8 nt + 2 tq (+ 1) --------------------
  float S[2][NT][4];
  float* slot = state + (((size_t)slots[b] * Hs + h) * P + p0) * N;
  bool have_state = start_pos[b] > 0;
#pragma unroll
  for (int mt = 0; mt < 2; mt++)
#pragma unroll
    for (int nt = 0; nt < NT; nt++) {
      const int n = 8 * NT * warp + 8 * nt + 2 * tq;
      float2 lo = make_float2(0.f, 0.f), hi = lo;
      if (have_state) {
        lo = *reinterpret_cast<const float2*>(slot + (size_t)(16 * mt + gq) * N + n);
        hi = *reinterpret_cast<const float2*>(slot + (size_t)(16 * mt + gq + 8) * N + n);
      }
      S[mt][nt][0] = lo.x; S[mt][nt][1] = lo.y; S[mt][nt][2] = hi.x; S[mt][nt][3] = hi.y;
    }

  const int i_base = warp * 16;
#pragma unroll 1
  for (int c = c0; c < c1; c++) {
    const int buf = (c - c0) & 1;
    const int t0 = seg_start[c], L = seg_start[c + 1] - t0;
    // ---- cumulative log2 decay of the chunk's rows, and what follows from it ----
    float v = dt_reg * a_log2;                     // 0 for rows past L
    if (tid < Q) {
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const float u = __shfl_up_sync(0xffffffffu, v, o);
        if (lane >= o) v += u;
      }
      if (lane == 31) wsum[warp] = v;
    }
    __syncthreads();
    const float total = wsum[0] + wsum[1] + wsum[2] + wsum[3];
    if (tid < Q) {
      float off = 0.f;
#pragma unroll
      for (int k = 0; k < 3; k++) if (k < warp) off += wsum[k];
      const float cum = v + off;
      cums[tid] = cum;
      dts[tid] = dt_reg;
      ws[tid] = ex2_quick(total - cum) * dt_reg;
      es[tid] = ex2_quick(cum);
    }
    const float decay = exp2f(total);
    // ---- the state as the chunk finds it, in bfloat16, for C S^T ----
    if (have_state) {
#pragma unroll
      for (int mt = 0; mt < 2; mt++)
#pragma unroll
        for (int nt = 0; nt < NT; nt++) {
          const int n = 8 * NT * warp + 8 * nt + 2 * tq;
          *reinterpret_cast<uint32_t*>(ssd_sm + lay.s + (16 * mt + gq) * LDN + n * 2) = pack_bf16(S[mt][nt][0], S[mt][nt][1]);
          *reinterpret_cast<uint32_t*>(ssd_sm + lay.s + (16 * mt + gq + 8) * LDN + n * 2) = pack_bf16(S[mt][nt][2], S[mt][nt][3]);
        }
    }
    cp_async_wait<2>();                            // x and C of this chunk (C B^T and B may still be on their way)
    __syncthreads();
    float acc[4][4];                               // y of rows i_base + gq (+ 8), columns 8 nt + 2 tq (+ 1)
#pragma unroll
    for (int nt = 0; nt < 4; nt++) acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0.f;
    const bool rows_live = i_base < L;
    if (have_state && rows_live) {
      // what came before: C S^T, K = the state columns
      const uint32_t a_addr = cs0 + (i_base + (lane & 7) + ((lane >> 3) & 1) * 8) * LDN + (lane >> 4) * 16;
      const uint32_t b_addr = ss0 + ((lane & 7) + (lane >> 4) * 8) * LDN + ((lane >> 3) & 1) * 16;
#pragma unroll 4
      for (int ks = 0; ks < N / 16; ks++) {
        uint32_t a0, a1, a2, a3, b0, b1, b2, b3;
        ldsm_x4(a_addr + ks * 32, a0, a1, a2, a3);
        ldsm_x4(b_addr + ks * 32, b0, b1, b2, b3);
        mma_bf16(acc[0], a0, a1, a2, a3, b0, b1);
        mma_bf16(acc[1], a0, a1, a2, a3, b2, b3);
        ldsm_x4(b_addr + 16 * LDN + ks * 32, b0, b1, b2, b3);
        mma_bf16(acc[2], a0, a1, a2, a3, b0, b1);
        mma_bf16(acc[3], a0, a1, a2, a3, b2, b3);
      }
      const float e_lo = es[i_base + gq], e_hi = es[i_base + gq + 8];
#pragma unroll
      for (int nt = 0; nt < 4; nt++) { acc[nt][0] *= e_lo; acc[nt][1] *= e_lo; acc[nt][2] *= e_hi; acc[nt][3] *= e_hi; }
    }
    __syncthreads();                               // everybody is done with C and with the state's copy
    fetch_xc(c + 1, buf ^ 1);
    dt_reg = load_dt(c + 1);
    cp_async_wait<2>();                            // C B^T of this chunk
    __syncthreads();
    const uint32_t xb = xs0 + buf * Q * LDX;
    if (rows_live) {
      // inside the chunk: M X with M built in registers from C B^T; K = rows j up to the diagonal block
      const float ci_lo = cums[i_base + gq], ci_hi = cums[i_base + gq + 8];
      const uint32_t a_addr = cb0 + (i_base + (lane & 7) + ((lane >> 3) & 1) * 8) * LDCB + (lane >> 4) * 16;
      const uint32_t b_addr = xb + ((lane & 7) + ((lane >> 3) & 1) * 8) * LDX + (lane >> 4) * 16;
#pragma unroll 1
      for (int ks = 0; ks <= warp; ks++) {
        uint32_t r[4];
        ldsm_x4(a_addr + ks * 32, r[0], r[1], r[2], r[3]);
        const int j0 = 16 * ks + 2 * tq;
        const float2 cj0 = *reinterpret_cast<const float2*>(cums + j0), cj1 = *reinterpret_cast<const float2*>(cums + j0 + 8);
        const float2 dj0 = *reinterpret_cast<const float2*>(dts + j0), dj1 = *reinterpret_cast<const float2*>(dts + j0 + 8);
        const bool diag = ks == warp;
#pragma unroll
        for (int q = 0; q < 4; q++) {
          // register q: row i_base + gq + 8 (q & 1), columns j0 + 8 (q >> 1) + {0, 1}
          const float ci = (q & 1) ? ci_hi : ci_lo;
          const float2 cj = (q >> 1) ? cj1 : cj0, dj = (q >> 1) ? dj1 : dj0;
          const float2 m = unpack_bf16(r[q]);
          float m0 = m.x * ex2_quick(ci - cj.x) * dj.x, m1 = m.y * ex2_quick(ci - cj.y) * dj.y;
          if (diag) {
            const int il = gq + 8 * (q & 1), jl = 2 * tq + 8 * (q >> 1);
            if (jl > il) m0 = 0.f;
            if (jl + 1 > il) m1 = 0.f;
          }
          r[q] = pack_bf16(m0, m1);
        }
        uint32_t b0, b1, b2, b3;
        ldsm_x4_t(b_addr + ks * 16 * LDX, b0, b1, b2, b3);
        mma_bf16(acc[0], r[0], r[1], r[2], r[3], b0, b1);
        mma_bf16(acc[1], r[0], r[1], r[2], r[3], b2, b3);
        ldsm_x4_t(b_addr + ks * 16 * LDX + 32, b0, b1, b2, b3);
        mma_bf16(acc[2], r[0], r[1], r[2], r[3], b0, b1);
        mma_bf16(acc[3], r[0], r[1], r[2], r[3], b2, b3);
      }
      // y = acc + D x
#pragma unroll
      for (int half = 0; half < 2; half++) {
        const int i = i_base + gq + 8 * half;
        if (i < L) {
          float* yr = y + (size_t)(t0 + i) * Di + (size_t)h * P + p0;
#pragma unroll
          for (int nt = 0; nt < 4; nt++) {
            const int p = 8 * nt + 2 * tq;
            const float2 xv = unpack_bf16(*reinterpret_cast<const uint32_t*>(ssd_sm + lay.x + (buf * Q + i) * LDX + p * 2));
            *reinterpret_cast<float2*>(yr + p) = make_float2(acc[nt][2 * half] + Dh * xv.x, acc[nt][2 * half + 1] + Dh * xv.y);
          }
        }
      }
    }
    // x times its row's weight, the operand of the state update
    for (int idx = tid; idx < Q * (PB / 2); idx += 256) {
      const int r = idx / (PB / 2), k = idx % (PB / 2);
      const float2 xv = unpack_bf16(*reinterpret_cast<const uint32_t*>(ssd_sm + lay.x + (buf * Q + r) * LDX + k * 4));
      const float w = ws[r];
      *reinterpret_cast<uint32_t*>(ssd_sm + lay.xw + r * LDX + k * 4) = pack_bf16(xv.x * w, xv.y * w);
    }
    __syncthreads();                               // everybody is done with C B^T; the scaled x is in place
    fetch_cb(c + 1);
    cp_async_wait<2>();                            // B of this chunk
    __syncthreads();
    // ---- S = decay S + (w x)^T B,  K = the chunk's rows ----
#pragma unroll
    for (int mt = 0; mt < 2; mt++)
#pragma unroll
      for (int nt = 0; nt < NT; nt++) { S[mt][nt][0] *= decay; S[mt][nt][1] *= decay; S[mt][nt][2] *= decay; S[mt][nt][3] *= decay; }
    {
      const int k_steps = (L + 15) / 16;
      const uint32_t a_addr = xw0 + ((lane & 7) + (lane >> 4) * 8) * LDX + ((lane >> 3) & 1) * 16;
      const uint32_t b_addr = bs0 + ((lane & 7) + ((lane >> 3) & 1) * 8) * LDN + (8 * NT * warp) * 2 + (lane >> 4) * 16;
#pragma unroll 2
      for (int ks = 0; ks < k_steps; ks++) {
        uint32_t a[2][4];
        ldsm_x4_t(a_addr + ks * 16 * LDX, a[0][0], a[0][1], a[0][2], a[0][3]);
        ldsm_x4_t(a_addr + ks * 16 * LDX + 32, a[1][0], a[1][1], a[1][2], a[1][3]);
#pragma unroll
        for (int np = 0; np < NT / 2; np++) {
          uint32_t b0, b1, b2, b3;
          ldsm_x4_t(b_addr + ks * 16 * LDN + np * 32, b0, b1, b2, b3);
#pragma unroll
          for (int mt = 0; mt < 2; mt++) {
            mma_bf16(S[mt][2 * np], a[mt][0], a[mt][1], a[mt][2], a[mt][3], b0, b1);
            mma_bf16(S[mt][2 * np + 1], a[mt][0], a[mt][1], a[mt][2], a[mt][3], b2, b3);
          }
        }
        if (NT & 1) {
          uint32_t b0, b1;
          ldsm_x2_t(b_addr + ks * 16 * LDN + (NT / 2) * 32, b0, b1);
#pragma unroll
          for (int mt = 0; mt < 2; mt++) mma_bf16(S[mt][NT - 1], a[mt][0], a[mt][1], a[mt][2], a[mt][3], b0, b1);
        }
      }
    }
    have_state = true;
    __syncthreads();                               // everybody is done with B and with the scaled x
    fetch_b(c + 1);
  }
  cp_async_wait<0>();
  // ---- the state after the sequence's last chunk goes to its slot ----
#pragma unroll
  for (int mt = 0; mt < 2; mt++)
#pragma unroll
    for (int nt = 0; nt < NT; nt++) {
      const int n = 8 * NT * warp + 8 * nt + 2 * tq;
      *reinterpret_cast<float2*>(slot + (size_t)(16 * mt + gq) * N + n) = make_float2(S[mt][nt][0], S[mt][nt][1]);
      *reinterpret_cast<float2*>(slot + (size_t)(16 * mt + gq + 8) * N + n) = make_float2(S[mt][nt][2], S[mt][nt][3]);
    }
}

size_t cb_smem(int N) { return (size_t)(64 + Q) * padded(N * 2); }

template <int NT>
int launch_walk(const __nv_bfloat16* xbc, const float* dt, const float* A, const float* Dskip, const __nv_bfloat16* cb,
                float* state, const int* seg_start, const int* seq_seg_start, const int* slots, const int* start_pos,
                float* y, int B, int Hs, int P, int G, int Cd, cudaStream_t stream) {
  const WalkSmem lay(64 * NT);
  tlc_launch(ssd_walk_kernel<NT>, dim3(B, Hs, P / PB), dim3(256), (size_t)lay.total, stream, xbc, dt, A, Dskip, cb, state,
             seg_start, seq_seg_start, slots, start_pos, y, Hs, P, G, Cd);
  TLC_CHECK_LAUNCH("ssm_scan(chunk walk)");
  return 0;
}

}  // namespace

extern "C" int tlc_ssd_init() {
  if (cudaFuncSetAttribute(ssd_cb_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)cb_smem(256)) != cudaSuccess ||
      cudaFuncSetAttribute(ssd_walk_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, WalkSmem(64).total) != cudaSuccess ||
      cudaFuncSetAttribute(ssd_walk_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, WalkSmem(128).total) != cudaSuccess ||
      cudaFuncSetAttribute(ssd_walk_kernel<3>, cudaFuncAttributeMaxDynamicSharedMemorySize, WalkSmem(192).total) != cudaSuccess ||
      cudaFuncSetAttribute(ssd_walk_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, WalkSmem(256).total) != cudaSuccess)
    return tlc_fail(-2, "ssm_scan(chunked): cannot reserve shared memory");
  return tlc_ssd_tc_init();
}

// Test hook: which walk runs where both are built (0: tcgen05 for states of 128 or 256 columns, else mma.sync;
// 1: always mma.sync).
static int g_ssd_walk = 0;
extern "C" void tlc_ssd_walk_override(int mode) { g_ssd_walk = mode; }

// Sizes this form is built for: heads whose size is a multiple of 32, a state of 64, 128, 192 or 256 columns,
// rows of x|B|C that start on 16-byte boundaries in bfloat16.
extern "C" int tlc_ssd_ok(int Hs, int P, int N, int G, int Cd) {
  return P % PB == 0 && P >= PB && N % 64 == 0 && N >= 64 && N <= 256 && Cd % 8 == 0 && G > 0 && Hs % G == 0 &&
         Hs <= 65535 && G <= 65535 && P / PB <= 65535;
}

// floats of scratch for n_seg chunks of T rows in all: per row and head the weight of the row in its chunk's state
// update and its factor on C S^T, per chunk and head the chunk's decay; then C B^T [128, 128] and B^T [N, 128] of
// every (chunk, group) in bfloat16
static long long ssd_row_floats(int n_seg, int T, int Hs) { return (2LL * T * Hs + (long long)n_seg * Hs + 3) / 4 * 4; }
extern "C" long long tlc_ssd_scratch_floats(int n_seg, int T, int Hs, int P, int N, int G) {
  return ssd_row_floats(n_seg, T, Hs) + ((long long)n_seg * G * Q * (Q + N) + 1) / 2;
}

// y_part, aux: with the walk on tcgen05 the part of the outputs that needs no state (M x + D x) goes to y_part
// [T, Hs*P] and only the state's share to y; *used_part = 1 then tells the caller to add the two.  That part
// does not stand on the walk's path: with a second stream `aux` (not while capturing) it runs there, beside the
// walk, and `stream` waits for it before this function returns.  Without y_part everything is added up in y.
extern "C" int tlc_ssm_scan_ssd(const void* xbc, const float* dt, const float* A, const float* Dskip, float* state,
                                float* scratch, const int* seg_start, const int* seg_seq, const int* seq_seg_start,
                                const int* slots, const int* start_pos, float* y, float* y_part, int* used_part, int B,
                                int n_seg, int T, int Hs, int P, int N, int G, int Cd, cudaStream_t stream,
                                cudaStream_t aux) {
  if (used_part) *used_part = 0;
  if (B == 0 || n_seg == 0) return 0;
  TLC_REQUIRE(tlc_ssd_ok(Hs, P, N, G, Cd), "ssm_scan(chunked, tensor cores): sizes Hs=%d P=%d N=%d G=%d Cd=%d are not built",
              Hs, P, N, G, Cd);
  TLC_REQUIRE(((uintptr_t)xbc % 16) == 0 && ((uintptr_t)scratch % 16) == 0 && ((uintptr_t)state % 8) == 0 &&
              ((uintptr_t)y % 8) == 0 && ((uintptr_t)y_part % 8) == 0, "ssm_scan(chunked, tensor cores): misaligned buffers");
  const __nv_bfloat16* x = (const __nv_bfloat16*)xbc;
  float* row_w = scratch;                         // [T, Hs], [T, Hs], [n_seg, Hs]: the rows' decays, for the walk
  float* row_e = row_w + (size_t)T * Hs;
  float* seg_decay = row_e + (size_t)T * Hs;
  __nv_bfloat16* cb = (__nv_bfloat16*)(scratch + ssd_row_floats(n_seg, T, Hs));
  const bool tc = (N == 128 || N == 256) && g_ssd_walk == 0;
  __nv_bfloat16* bt = tc ? cb + (size_t)n_seg * G * Q * Q : nullptr;
  const int z_cb = 2 + (tc ? N / 64 : 0), z_decay = tc ? (Hs / G + 3) / 4 : 0;
  tlc_launch(ssd_cb_kernel, dim3(n_seg, G, z_cb + z_decay), dim3(128), cb_smem(N), stream, x, seg_start, cb, bt, Hs * P, N, G, Cd,
             dt, A, Hs, row_w, row_e, seg_decay, tc ? z_cb : 0);
  TLC_CHECK_LAUNCH("ssm_scan(C B^T)");
  if (tc) {
    const bool apart = y_part != nullptr && used_part != nullptr;
    cudaStreamCaptureStatus capturing = cudaStreamCaptureStatusNone;
    cudaStreamIsCapturing(stream, &capturing);
    const bool beside = apart && aux != nullptr && aux != stream && capturing == cudaStreamCaptureStatusNone;
    cudaStream_t s_part = beside ? aux : stream;
    // the two events of a calling thread are made once: a record overwrites an event's last state, and each wait
    // below follows its record in this thread's program order
    static thread_local cudaEvent_t e_cb = nullptr, e_part = nullptr;
    if (beside) {
      if (e_cb == nullptr && (cudaEventCreateWithFlags(&e_cb, cudaEventDisableTiming) != cudaSuccess ||
                              cudaEventCreateWithFlags(&e_part, cudaEventDisableTiming) != cudaSuccess)) {
        e_cb = e_part = nullptr;
        return tlc_fail(-3, "ssm_scan: cannot create events");
      }
      cudaEventRecord(e_cb, stream);
      cudaStreamWaitEvent(aux, e_cb, 0);
    }
    float* y_free = apart ? y_part : y;            // where M x + D x goes
    // every chunk's outputs as far as they need no state
    if (P % 64 == 0)
      tlc_launch_as(!beside, ssd_intra_kernel<64>, dim3(n_seg, Hs, P / 64), dim3(128), 0, s_part, x, dt, A, Dskip, cb, seg_start, y_free,
                    Hs, P, G, Cd);
    else
      tlc_launch_as(!beside, ssd_intra_kernel<32>, dim3(n_seg, Hs, P / 32), dim3(128), 0, s_part, x, dt, A, Dskip, cb, seg_start, y_free,
                    Hs, P, G, Cd);
    TLC_CHECK_LAUNCH("ssm_scan(chunk outputs without the state)");
    if (beside) cudaEventRecord(e_part, aux);
    // the walk: the state's share, written to y (added to what is there when the other part went there too)
    int rc = tlc_ssd_tc_run(x, row_w, row_e, seg_decay, bt, state, seg_start, seq_seg_start, slots, start_pos, y, apart ? 0 : 1, B,
                            n_seg, T, Hs, P, N, G, Cd, stream);
    if (beside) cudaStreamWaitEvent(stream, e_part, 0);
    if (rc == 0 && apart) *used_part = 1;
    return rc;
  }
  switch (N / 64) {
    case 1: return launch_walk<1>(x, dt, A, Dskip, cb, state, seg_start, seq_seg_start, slots, start_pos, y, B, Hs, P, G, Cd, stream);
    case 2: return launch_walk<2>(x, dt, A, Dskip, cb, state, seg_start, seq_seg_start, slots, start_pos, y, B, Hs, P, G, Cd, stream);
    case 3: return launch_walk<3>(x, dt, A, Dskip, cb, state, seg_start, seq_seg_start, slots, start_pos, y, B, Hs, P, G, Cd, stream);
    default: return launch_walk<4>(x, dt, A, Dskip, cb, state, seg_start, seq_seg_start, slots, start_pos, y, B, Hs, P, G, Cd, stream);
  }
}
