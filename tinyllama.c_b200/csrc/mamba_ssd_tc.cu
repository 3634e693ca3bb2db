// The walk over a sequence's chunks (see mamba_ssd.cu for the math) with the products on the 5th-generation
// tensor cores: tcgen05.mma from shared-memory operands into tensor memory, for states of 128 or 256 columns.
//
// One block per (sequence, head, 32 rows p of the head): 8 warps of workers and one warp whose first lane issues
// the copies and the products.  Tensor memory holds the state transposed,
// S^T[n, p] (lanes = state columns, two tiles of 128 for N = 256), from the slot's state before the first
// chunk to the slot's state after the last, and the two accumulators of a chunk's outputs.  Per chunk:
//   * C [128 rows, N] and B^T [N, 128 rows] arrive by TMA (128-byte swizzle, K along the rows of shared memory:
//     the state columns for C, the chunk's rows for B^T, which ssd_cb_kernel wrote transposed beside C B^T);
//   * the threads read the state back (tcgen05.ld), leave a bfloat16 copy [p, n] in shared memory for C S^T,
//     scale it by the chunk's decay and store it again (tcgen05.st); they build the score matrix
//     M[i, j] = cb exp(cum_i - cum_j) dt_j, x^T and (w x)^T in shared memory in the layout tcgen05.mma reads;
//   * the issuing thread starts D1 = C S^T, D2 = M x and S^T += B^T (w x), commits them to mbarriers, and
//     refills C's and B^T's buffers for the next chunk as soon as the products that read them are done;
//   * the threads read D1 and D2 back and write y = exp(cum_i) D1 + D2 + D x.
// Every operand is K-major with the 128-byte swizzle, the layout of the linear layers' tiles.  Every wait on an
// mbarrier is bounded; a wait that runs out is recorded in the library's error word, the walk goes on without
// further waits (its output is then wrong, and reported), frees its tensor memory and returns.
#include "common.cuh"
#include "mbarrier.cuh"
#include "tcgen05.cuh"

int tlc_ssd_tc_run(const __nv_bfloat16* xbc, const float* dt, const float* A, const float* Dskip, const __nv_bfloat16* cb,
                   __nv_bfloat16* bt, float* state, const int* seg_start, const int* seq_seg_start, const int* slots,
                   const int* start_pos, float* y, int B, int n_seg, int T, int Hs, int P, int N, int G, int Cd,
                   cudaStream_t stream);

namespace {

constexpr int Q = 128;       // rows per chunk
constexpr int PB = 32;       // rows p of a head per block
constexpr float LOG2E = 1.4426950408889634f;

__device__ __forceinline__ float ex2_quick(float x) {
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
__device__ __forceinline__ unsigned short bf16_bits(float v) {
  const __nv_bfloat16 b = __float2bfloat16_rn(v);
  return *reinterpret_cast<const unsigned short*>(&b);
}

// Byte offset of element (row, k) of a K-major operand whose rows are 64 elements (128 bytes) per slab, with the
// 128-byte swizzle: slab k / 64 (of `slab_bytes`), row * 128, and the 16-byte piece index xor-ed with row % 8.
__device__ __forceinline__ uint32_t sw128(int row, int k, int slab_bytes) {
  return (uint32_t)((k >> 6) * slab_bytes + row * 128 + ((((k & 63) >> 3) ^ (row & 7)) << 4) + (k & 7) * 2);
}

// Shared memory of the walk (byte offsets from a 1024-byte boundary).  NTILES = N / 128.
template <int NTILES>
struct TcSmem {
  static constexpr int N = 128 * NTILES;
  static constexpr int C_SLAB = Q * 128, C = 0, C_BYTES = (N / 64) * C_SLAB;            // [128 rows i][N], slabs of 64 n
  static constexpr int BT_SLAB = N * 128, BT = C + C_BYTES, BT_BYTES = 2 * BT_SLAB;      // [N rows n][128 j], slabs of 64 j
  static constexpr int M_SLAB = Q * 128, M = BT + BT_BYTES, M_BYTES = 2 * M_SLAB;        // [128 rows i][128 j]
  static constexpr int X_SLAB = PB * 128, XT = M + M_BYTES, XWT = XT + 2 * X_SLAB;       // [32 rows p][128 j]; (w x)^T twice
  static constexpr int S_SLAB = PB * 128, S = XWT + 4 * X_SLAB, S_BYTES = (N / 64) * S_SLAB;   // [32 rows p][N]
  static constexpr int F = S + S_BYTES;                                                  // floats: cums, dts, ws, es, wsum
  static constexpr int BARS = F + (4 * Q + 8) * 4;                                       // 4 mbarriers, tmem slot, dead flag
  static constexpr int TOTAL = BARS + 64 + 1024;                                         // + alignment slack
};

constexpr int WORKERS = 256, THREADS = WORKERS + 32;
__device__ __forceinline__ void workers_sync() { asm volatile("bar.sync 1, 256;" ::: "memory"); }

template <int NTILES>
__global__ void __launch_bounds__(THREADS, 1)
ssd_walk_tc_kernel(const __grid_constant__ CUtensorMap map_c, const __grid_constant__ CUtensorMap map_bt,
                   const __nv_bfloat16* __restrict__ xbc, const float* __restrict__ dt, const float* __restrict__ A,
                   const float* __restrict__ Dskip, const __nv_bfloat16* __restrict__ cb, float* __restrict__ state,
                   const int* __restrict__ seg_start, const int* __restrict__ seq_seg_start, const int* __restrict__ slots,
                   const int* __restrict__ start_pos, float* __restrict__ y, int Hs, int P, int G, int Cd, ErrWords* err) {
  tlc_pdl(xbc, dt, cb, state, y);
  using L_ = TcSmem<NTILES>;
  constexpr int N = L_::N;
  constexpr int TCOLS = NTILES == 1 ? 128 : 128;     // tensor-memory columns: state 32 per tile, D1 at 64, D2 at 96
  extern __shared__ uint8_t smem_raw[];
  uint8_t* sm = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  float* cums = reinterpret_cast<float*>(sm + L_::F);
  float* dts = cums + Q;
  float* ws = dts + Q;
  float* es = ws + Q;
  float* wsum = es + Q;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sm + L_::BARS);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 4);
  volatile int* dead = reinterpret_cast<volatile int*>(tmem_slot + 1);
  const uint32_t sm0 = smem_u32(sm);
  const uint32_t bar_c = smem_u32(bars), bar_bt = smem_u32(bars + 1), bar_y = smem_u32(bars + 2), bar_s = smem_u32(bars + 3);

  const int b = blockIdx.x, h = blockIdx.y, p0 = blockIdx.z * PB;
  const int g = h / (Hs / G);
  const int Di = Hs * P;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int c0 = seq_seg_start[b], c1 = seq_seg_start[b + 1];
  if (c1 <= c0) return;
  const float a_log2 = A[h] * LOG2E, Dh = Dskip[h];
  const long long wait_limit = mbar_wait_limit(err);
  const unsigned short* Xg = reinterpret_cast<const unsigned short*>(xbc) + (size_t)h * P + p0;
  const int c_col0 = Di + G * N + g * N;               // first column of this group's C in a row of x|B|C

  if (tid == 0) {
    for (int i = 0; i < 4; i++) mbar_init(bar_c + 8 * i, 1);
    *dead = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(TCOLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  // the score matrix's pieces above the diagonal are never written again: zero once
  for (int i = tid; i < L_::M_BYTES / 16; i += THREADS) reinterpret_cast<uint4*>(sm + L_::M)[i] = make_uint4(0u, 0u, 0u, 0u);
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem = *tmem_slot;

  // a bounded wait; once one has run out, no further wait is attempted
  auto wait = [&](uint32_t bar, uint32_t parity, int code) {
    if (*dead) return;
    if (!mbar_wait(bar, parity, err, code, wait_limit)) *dead = 1;
  };
  auto fetch_c = [&](int c) {                          // thread 0: C of chunk c
    mbar_expect_tx(bar_c, L_::C_BYTES);
    const int t0 = seg_start[c];
    for (int s = 0; s < N / 64; s++) tma_load_2d(sm0 + L_::C + s * L_::C_SLAB, &map_c, bar_c, c_col0 + 64 * s, t0);
  };
  auto fetch_bt = [&](int c) {                         // thread 0: B^T of chunk c
    mbar_expect_tx(bar_bt, L_::BT_BYTES);
    for (int s = 0; s < 2; s++) tma_load_2d(sm0 + L_::BT + s * L_::BT_SLAB, &map_bt, bar_bt, 64 * s, (c * G + g) * N);
  };
  auto load_dt = [&](int c) -> float {
    if (c < c1 && tid < Q) {
      const int t0 = seg_start[c], L = seg_start[c + 1] - t0;
      if (tid < L) return dt[(size_t)(t0 + tid) * Hs + h];
    }
    return 0.f;
  };
  if (warp == WORKERS / 32) {
    // ---- the issuing warp: its first lane starts copies and products; nothing else runs here ----
    constexpr uint32_t idesc = instr_desc(128, PB);
    if (lane == 0) {
      fetch_c(c0);
      fetch_bt(c0);
    }
    __syncwarp();
#pragma unroll 1
    for (int c = c0; c < c1; c++) {
      const uint32_t ph = (uint32_t)((c - c0) & 1);
      const int xw_off = L_::XWT + (int)ph * 2 * L_::X_SLAB;
      asm volatile("bar.sync 2, %0;" ::"n"(THREADS) : "memory");      // the workers' operands of this chunk are in place
      if (lane == 0) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        wait(bar_c, ph, 11);                           // C of this chunk has landed
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        // D1 = C S^T (K = the state columns)
#pragma unroll
        for (int s = 0; s < N / 64; s++)
#pragma unroll
          for (int kk = 0; kk < 4; kk++)
            umma(tmem + 64u, smem_desc(sm0 + L_::C + s * L_::C_SLAB + kk * 32), smem_desc(sm0 + L_::S + s * L_::S_SLAB + kk * 32),
                 idesc, (s > 0 || kk > 0) ? 1u : 0u);
        // D2 = M x (K = the chunk's rows)
#pragma unroll
        for (int s = 0; s < 2; s++)
#pragma unroll
          for (int kk = 0; kk < 4; kk++)
            umma(tmem + 96u, smem_desc(sm0 + L_::M + s * L_::M_SLAB + kk * 32), smem_desc(sm0 + L_::XT + s * L_::X_SLAB + kk * 32),
                 idesc, (s > 0 || kk > 0) ? 1u : 0u);
        umma_commit(bar_y);
        wait(bar_bt, ph, 12);                          // B^T of this chunk has landed
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        // S^T += B^T (w x) (K = the chunk's rows), a tile of 128 state columns at a time
#pragma unroll
        for (int t = 0; t < NTILES; t++)
#pragma unroll
          for (int s = 0; s < 2; s++)
#pragma unroll
            for (int kk = 0; kk < 4; kk++)
              umma(tmem + (uint32_t)(32 * t), smem_desc(sm0 + L_::BT + s * L_::BT_SLAB + t * (128 * 128) + kk * 32),
                   smem_desc(sm0 + xw_off + s * L_::X_SLAB + kk * 32), idesc, 1u);
        umma_commit(bar_s);
        if (c + 1 < c1) {
          wait(bar_y, ph, 14);                         // C's buffer is free again
          fetch_c(c + 1);
          wait(bar_s, ph, 13);                         // and B^T's
          fetch_bt(c + 1);
        }
      }
      __syncwarp();
    }
  } else {
  // ---- the workers ----
  float dt_reg = load_dt(c0);

  // the state: this thread holds column n = 128 tile + 32 quarter + lane of S^T, all 32 rows p
  const int tile = NTILES == 1 ? 0 : (warp >> 2), quarter = warp & 3;
  const bool owns_state = NTILES == 2 || warp < 4;     // with one tile, warps 4..7 hold no state
  const int n_mine = 128 * tile + 32 * quarter + lane;
  const uint32_t t_state = tmem + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(tile * 32);
  const uint32_t t_d1 = tmem + ((uint32_t)(quarter * 32) << 16) + 64u + (uint32_t)((warp >> 2) * 16);
  const uint32_t t_d2 = t_d1 + 32u;
  float* slot = state + (((size_t)slots[b] * Hs + h) * P + p0) * N;
  uint32_t sreg[32];
  if (owns_state) {
    const bool have = start_pos[b] > 0;
#pragma unroll
    for (int p = 0; p < 32; p++) sreg[p] = have ? __float_as_uint(slot[(size_t)p * N + n_mine]) : 0u;
  }

  // What a thread reads from global memory for a chunk, fetched one chunk ahead.
  // Of C B^T: rows r = tid / 4 and 127 - r have 17 pieces of 8 columns up to their diagonals between them; the four
  // threads of the pair take every fourth piece (the first a fifth one), so that every thread has four or five.
  // Of x: row mi = tid % 128, columns [16 mhalf, 16 mhalf + 16) of the block's 32; the same values serve x^T, (w x)^T
  // and the D x of the output row mi.
  const int mi = tid & 127, mhalf = tid >> 7;
  const int pr = tid >> 2, pu = tid & 3, n_first = (pr >> 3) + 1;      // pieces of row pr; row 127 - pr has 17 - n_first
  uint4 cbv[5], xv[2], xv_next[2];
  auto piece = [&](int e, int& row, int& q) {            // piece e of the pair's 17: its row and its index in the row
    const bool first = e < n_first;
    row = first ? pr : 127 - pr;
    q = first ? e : e - n_first;
  };
  auto load_cb = [&](int c) {
    if (c < c1) {
      const int L = seg_start[c + 1] - seg_start[c];
      const __nv_bfloat16* base = cb + (((size_t)c * G + g) * Q) * Q;
#pragma unroll
      for (int u = 0; u < 5; u++) {
        const int e = pu + 4 * u;
        int row, q;
        piece(e, row, q);
        if (e < 17 && row < L) cbv[u] = __ldg(reinterpret_cast<const uint4*>(base + (size_t)row * Q + 8 * q));
      }
    }
  };
  auto load_x = [&](int c, uint4 (&dst)[2]) {
    dst[0] = dst[1] = make_uint4(0u, 0u, 0u, 0u);
    if (c < c1) {
      const int t0 = seg_start[c], L = seg_start[c + 1] - t0;
      if (mi < L) {
        const uint4* src = reinterpret_cast<const uint4*>(Xg + (size_t)(t0 + mi) * Cd + 16 * mhalf);
        dst[0] = __ldg(src);
        dst[1] = __ldg(src + 1);
      }
    }
  };
  load_cb(c0);
  load_x(c0, xv);

#pragma unroll 1
  for (int c = c0; c < c1; c++) {
    const int k = c - c0;
    const uint32_t ph = (uint32_t)(k & 1);
    const int t0 = seg_start[c], L = seg_start[c + 1] - t0;
    // ---- cumulative log2 decay of the chunk's rows ----
    float v = dt_reg * a_log2;
    if (tid < Q) {
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const float u = __shfl_up_sync(0xffffffffu, v, o);
        if (lane >= o) v += u;
      }
      if (lane == 31) wsum[warp] = v;
    }
    workers_sync();
    const float total = wsum[0] + wsum[1] + wsum[2] + wsum[3];
    if (tid < Q) {
      float off = 0.f;
#pragma unroll
      for (int q = 0; q < 3; q++) if (q < warp) off += wsum[q];
      const float cum = v + off;
      cums[tid] = cum;
      dts[tid] = dt_reg;
      ws[tid] = ex2_quick(total - cum) * dt_reg;
      es[tid] = ex2_quick(cum);
    }
    const float decay = exp2f(total);
    dt_reg = load_dt(c + 1);
    if (c > c0) {
      wait(bar_y, ph ^ 1, 14);                         // the products that read M, x^T and the state's copy are done
    }
    workers_sync();                                    // cums, dts, ws, es are in place
    // ---- the score matrix M, K-major: row i, the pieces of 8 columns up to the diagonal ----
#pragma unroll
    for (int u = 0; u < 5; u++) {
      const int e = pu + 4 * u;
      int row, q;
      piece(e, row, q);
      if (e < 17 && row < L) {
        const int j0 = 8 * q;
        const float ci = cums[row];
        const float4 cj0 = *reinterpret_cast<const float4*>(cums + j0), cj1 = *reinterpret_cast<const float4*>(cums + j0 + 4);
        const float4 dj0 = *reinterpret_cast<const float4*>(dts + j0), dj1 = *reinterpret_cast<const float4*>(dts + j0 + 4);
        const float cj[8] = {cj0.x, cj0.y, cj0.z, cj0.w, cj1.x, cj1.y, cj1.z, cj1.w};
        const float dj[8] = {dj0.x, dj0.y, dj0.z, dj0.w, dj1.x, dj1.y, dj1.z, dj1.w};
        const uint32_t w4[4] = {cbv[u].x, cbv[u].y, cbv[u].z, cbv[u].w};
        uint32_t r4[4];
#pragma unroll
        for (int x = 0; x < 4; x++) {
          const float2 m = unpack_bf16(w4[x]);
          const int j = j0 + 2 * x;
          const float m0 = j <= row ? m.x * ex2_quick(ci - cj[2 * x]) * dj[2 * x] : 0.f;
          const float m1 = j + 1 <= row ? m.y * ex2_quick(ci - cj[2 * x + 1]) * dj[2 * x + 1] : 0.f;
          r4[x] = pack_bf16(m0, m1);
        }
        *reinterpret_cast<uint4*>(sm + L_::M + (q >> 3) * L_::M_SLAB + row * 128 + (((q & 7) ^ (row & 7)) << 4)) =
            make_uint4(r4[0], r4[1], r4[2], r4[3]);
      }
    }
    load_cb(c + 1);                                    // its registers are free: the next chunk's share is on its way
    // ---- x^T and (w x)^T, K-major: row p, column j.  (w x)^T alternates between two buffers: the state update of
    // the chunk before may still be reading the other ----
    const int xw_off = L_::XWT + (k & 1) * 2 * L_::X_SLAB;
    {
      const float w = ws[mi];
      const uint32_t w8[8] = {xv[0].x, xv[0].y, xv[0].z, xv[0].w, xv[1].x, xv[1].y, xv[1].z, xv[1].w};
#pragma unroll
      for (int e = 0; e < 8; e++) {
        const int p = 16 * mhalf + 2 * e;
        const float2 x2 = unpack_bf16(w8[e]);
        *reinterpret_cast<unsigned short*>(sm + L_::XT + sw128(p, mi, L_::X_SLAB)) = (unsigned short)(w8[e] & 0xffffu);
        *reinterpret_cast<unsigned short*>(sm + L_::XT + sw128(p + 1, mi, L_::X_SLAB)) = (unsigned short)(w8[e] >> 16);
        *reinterpret_cast<unsigned short*>(sm + xw_off + sw128(p, mi, L_::X_SLAB)) = bf16_bits(x2.x * w);
        *reinterpret_cast<unsigned short*>(sm + xw_off + sw128(p + 1, mi, L_::X_SLAB)) = bf16_bits(x2.y * w);
      }
    }
    load_x(c + 1, xv_next);
    // ---- the state: wait for the last update, copy it in bfloat16 for C S^T, decay it, hand it back ----
    if (c > c0) {
      wait(bar_s, ph ^ 1, 13);                         // the state update of the chunk before
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      __syncwarp();
      if (owns_state) tmem_ld32(t_state, sreg);
    }
    if (owns_state) {
#pragma unroll
      for (int p = 0; p < 32; p++) {
        const float s = __uint_as_float(sreg[p]);
        *reinterpret_cast<unsigned short*>(sm + L_::S + sw128(p, n_mine, L_::S_SLAB)) = bf16_bits(s);
        sreg[p] = __float_as_uint(s * decay);
      }
      __syncwarp();
      tmem_st32(t_state, sreg);
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");     // what the threads wrote, before the tensor cores read it
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    asm volatile("bar.sync 2, %0;" ::"n"(THREADS) : "memory");       // hands the chunk to the issuing thread
    // ---- y = exp(cum_i) D1 + D2 + D x for row i = 32 quarter + lane (= mi), columns [16 mhalf, 16 mhalf + 16) ----
    wait(bar_y, ph, 14);
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    {
      uint32_t d1[16], d2[16];
      __syncwarp();
      tmem_ld16(t_d1, d1);
      tmem_ld16(t_d2, d2);
      if (mi < L) {
        const float e = es[mi];
        const uint32_t x8[8] = {xv[0].x, xv[0].y, xv[0].z, xv[0].w, xv[1].x, xv[1].y, xv[1].z, xv[1].w};
        float out[16];
#pragma unroll
        for (int q = 0; q < 8; q++) {
          const float2 x2 = unpack_bf16(x8[q]);
          out[2 * q] = fmaf(e, __uint_as_float(d1[2 * q]), __uint_as_float(d2[2 * q])) + Dh * x2.x;
          out[2 * q + 1] = fmaf(e, __uint_as_float(d1[2 * q + 1]), __uint_as_float(d2[2 * q + 1])) + Dh * x2.y;
        }
        float4* yr = reinterpret_cast<float4*>(y + (size_t)(t0 + mi) * Di + (size_t)h * P + p0 + 16 * mhalf);
#pragma unroll
        for (int q = 0; q < 4; q++) yr[q] = make_float4(out[4 * q], out[4 * q + 1], out[4 * q + 2], out[4 * q + 3]);
      }
    }
    xv[0] = xv_next[0];
    xv[1] = xv_next[1];
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  }
  // ---- the state after the sequence's last chunk goes to its slot ----
  wait(bar_s, (uint32_t)((c1 - 1 - c0) & 1), 13);
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  __syncwarp();
  if (owns_state) {
    tmem_ld32(t_state, sreg);
#pragma unroll
    for (int p = 0; p < 32; p++) slot[(size_t)p * N + n_mine] = __uint_as_float(sreg[p]);
  }
  }   // workers
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 0)
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TCOLS) : "memory");
}

template <int NTILES>
int launch(const CUtensorMap& mc, const CUtensorMap& mbt, const __nv_bfloat16* xbc, const float* dt, const float* A,
           const float* Dskip, const __nv_bfloat16* cb, float* state, const int* seg_start, const int* seq_seg_start,
           const int* slots, const int* start_pos, float* y, int B, int Hs, int P, int G, int Cd, cudaStream_t stream) {
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(ssd_walk_tc_kernel<NTILES>, cudaFuncAttributeMaxDynamicSharedMemorySize, TcSmem<NTILES>::TOTAL) !=
        cudaSuccess)
      return tlc_fail(-2, "ssm_scan(chunk walk, tcgen05): cannot reserve %d bytes of shared memory", TcSmem<NTILES>::TOTAL);
    configured = true;
  }
  tlc_launch(ssd_walk_tc_kernel<NTILES>, dim3(B, Hs, P / PB), dim3(THREADS), (size_t)TcSmem<NTILES>::TOTAL, stream, mc, mbt, xbc, dt,
             A, Dskip, cb, state, seg_start, seq_seg_start, slots, start_pos, y, Hs, P, G, Cd, tlc_error_words());
  TLC_CHECK_LAUNCH("ssm_scan(chunk walk, tcgen05)");
  return 0;
}

}  // namespace

// Prepares the kernels' attributes outside any stream capture (called from tlc_ssd_init).
int tlc_ssd_tc_init() {
  if (cudaFuncSetAttribute(ssd_walk_tc_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, TcSmem<1>::TOTAL) != cudaSuccess ||
      cudaFuncSetAttribute(ssd_walk_tc_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, TcSmem<2>::TOTAL) != cudaSuccess)
    return tlc_fail(-2, "ssm_scan(chunk walk, tcgen05): cannot reserve shared memory");
  return 0;
}

// The walk.  N is 128 or 256; bt [n_seg, G, N, 128]: B of every chunk transposed (ssd_cb_kernel writes it beside C B^T).
int tlc_ssd_tc_run(const __nv_bfloat16* xbc, const float* dt, const float* A, const float* Dskip, const __nv_bfloat16* cb,
                   __nv_bfloat16* bt, float* state, const int* seg_start, const int* seq_seg_start, const int* slots,
                   const int* start_pos, float* y, int B, int n_seg, int T, int Hs, int P, int N, int G, int Cd,
                   cudaStream_t stream) {
  TLC_REQUIRE(N == 128 || N == 256, "ssm_scan(chunk walk, tcgen05): a state of %d columns", N);
  TLC_REQUIRE(tlc_error_words() != nullptr, "ssm_scan(chunk walk, tcgen05): the library is not set up (tlc_linear_init)");
  CUtensorMap mc, mbt;
  if (int rc = tlc_tensor_map_bf16(xbc, T, Cd, Cd, 64, Q, &mc)) return rc;
  if (int rc = tlc_tensor_map_bf16(bt, (long long)n_seg * G * N, Q, Q, 64, N, &mbt)) return rc;
  if (N == 128)
    return launch<1>(mc, mbt, xbc, dt, A, Dskip, cb, state, seg_start, seq_seg_start, slots, start_pos, y, B, Hs, P, G, Cd, stream);
  return launch<2>(mc, mbt, xbc, dt, A, Dskip, cb, state, seg_start, seq_seg_start, slots, start_pos, y, B, Hs, P, G, Cd, stream);
}
