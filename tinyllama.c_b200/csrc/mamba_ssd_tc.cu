// The walk over a sequence's chunks (see mamba_ssd.cu for the math) with the products on the 5th-generation
// tensor cores: tcgen05.mma from shared-memory operands into tensor memory, for states of 128 or 256 columns.
// It computes the STATE'S share of the outputs, y_i = 2^cum_i C_i S^T, and carries the state; what needs no state
// (M x + D x) is computed for all chunks at once by ssd_intra_kernel (mamba_ssd.cu), on a second stream where the
// caller gives one, and the rows' decays (cum, the weight w = 2^(total - cum) dt of a row in its chunk's state
// update, the chunk's decay) come from blocks of ssd_cb_kernel.  Nothing on this kernel's path scans, shuffles or
// synchronises the workers among themselves while the tensor cores stream operands.
//
// One block per (sequence, head, 32 rows p of the head): 8 warps of workers and one warp whose first lane issues
// the copies and the products.  Tensor memory holds the state transposed, S^T[n, p] (lanes = state columns, two
// tiles of 128 for N = 256), from the slot's state before the first chunk to the slot's state after the last,
// and the accumulator D1 of a chunk's outputs.  Per chunk:
//   * C [128 rows, N] and B^T [N, 128 rows] arrive by TMA (128-byte swizzle, K along the rows of shared memory:
//     the state columns for C, the chunk's rows for B^T, which ssd_cb_kernel wrote transposed beside C B^T);
//   * the workers read the state back (tcgen05.ld), leave a bfloat16 copy in shared memory for C S^T (row n, the 32
//     values p along the row: an MN-major B operand, four 16-byte stores a thread), scale the state by the
//     chunk's decay and store it again (tcgen05.st); that is all that stands between two chunks' products;
//   * the issuing thread starts D1 = C S^T and S^T += B^T (w x), commits them to mbarriers, and refills C's and
//     B^T's buffers for the next chunk as soon as the products that read them are done;
//   * while they run the workers write (w x)^T of the NEXT chunk (K-major, two buffers) and ask for what they
//     need from global memory two chunks ahead (behind the 128 KB refill a load waits thousands of cycles; the
//     chunks' boundaries are kept in registers so that no address depends on a load); then they read D1 back and
//     write y = 2^cum_i D1 (added to what is there if the other part was written to the same matrix).
// Every wait on an mbarrier is bounded; a wait that runs out is recorded in the library's error word, the walk goes
// on without further waits (its output is then wrong, and reported), frees its tensor memory and returns.
#include "common.cuh"
#include "mbarrier.cuh"
#include "tcgen05.cuh"

int tlc_ssd_tc_run(const __nv_bfloat16* xbc, const float* row_w, const float* row_e, const float* seg_decay,
                   __nv_bfloat16* bt, float* state,
                   const int* seg_start, const int* seq_seg_start, const int* slots,
                   const int* start_pos, float* y, int add_to_y, int B, int n_seg, int T, int Hs, int P, int N, int G, int Cd,
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
  static constexpr int X_SLAB = PB * 128, XW_BYTES = 2 * X_SLAB, XW = BT + BT_BYTES;     // (w x)^T [32 rows p][128 j], twice
  static constexpr int S = XW + 2 * XW_BYTES, S_BYTES = N * 128;                         // the state's copy [N rows n][32 p of 64]
  static constexpr int BARS = S + S_BYTES;                                               // 4 mbarriers, tmem slot, dead flag
  static constexpr int TOTAL = BARS + 64 + 1024;                                         // + alignment slack
};

constexpr int WORKERS = 256, THREADS = WORKERS + 32;
__device__ __forceinline__ void workers_sync() { asm volatile("bar.sync 1, 256;" ::: "memory"); }

template <int NTILES>
__global__ void __launch_bounds__(THREADS, 1)
ssd_walk_tc_kernel(const __grid_constant__ CUtensorMap map_c, const __grid_constant__ CUtensorMap map_bt,
                   const __nv_bfloat16* __restrict__ xbc, const float* __restrict__ row_w, const float* __restrict__ row_e,
                   const float* __restrict__ seg_decay, float* __restrict__ state,
                   const int* __restrict__ seg_start, const int* __restrict__ seq_seg_start, const int* __restrict__ slots,
                   const int* __restrict__ start_pos, float* __restrict__ y, int add_to_y, int n_seqs, int Hs, int P, int G, int Cd,
                   ErrWords* err) {
  tlc_pdl(xbc, row_w, row_e, seg_decay, state, y);
  using L_ = TcSmem<NTILES>;
  constexpr int N = L_::N;
  constexpr int TCOLS = 128;                         // tensor-memory columns: state 32 per tile, D1 at 64
  extern __shared__ uint8_t smem_raw[];
  uint8_t* sm = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint64_t* bars = reinterpret_cast<uint64_t*>(sm + L_::BARS);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 4);
  volatile int* dead = reinterpret_cast<volatile int*>(tmem_slot + 1);
  const uint32_t sm0 = smem_u32(sm);
  const uint32_t bar_c = smem_u32(bars), bar_bt = smem_u32(bars + 1), bar_y = smem_u32(bars + 2), bar_s = smem_u32(bars + 3);

  const int Di = Hs * P;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const long long wait_limit = mbar_wait_limit(err);
  if (tid == 0) *dead = 0;
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(TCOLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem = *tmem_slot;

  // An item is (sequence, head, 32 rows of the head).  A block takes items blockIdx.x, + gridDim.x, ...: with many
  // short sequences (32 prompts of 64 tokens are 3,072 items of one chunk each) a block an item spent more time on
  // its start-up (tensor-memory allocation, barriers, the first copies) than on its chunk.  Consecutive items are
  // the heads of one sequence, so a block's items are of many sequences, long and short.  Tensor memory is
  // allocated once; the four barriers are made anew per item, after a block-wide barrier behind which nothing is
  // pending on them (every copy and every commit of an item is waited for by somebody before the item ends).
  const int per_seq = Hs * (P / PB);
  bool first = true;
#pragma unroll 1
  for (int item = blockIdx.x; item < n_seqs * per_seq; item += gridDim.x) {
  const int b = item / per_seq, h = (item % per_seq) / (P / PB), p0 = (item % (P / PB)) * PB;
  const int g = h / (Hs / G);
  const int c0 = seq_seg_start[b], c1 = seq_seg_start[b + 1];
  if (c1 <= c0) continue;
  const unsigned short* Xg = reinterpret_cast<const unsigned short*>(xbc) + (size_t)h * P + p0;
  const int c_col0 = Di + G * N + g * N;               // first column of this group's C in a row of x|B|C
  if (tid == 0) {
    for (int i = 0; i < 4; i++) {
      if (!first) asm volatile("mbarrier.inval.shared::cta.b64 [%0];" ::"r"(bar_c + 8 * i) : "memory");
      mbar_init(bar_c + 8 * i, 1);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  first = false;
  __syncthreads();

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
  if (warp == WORKERS / 32) {
    // ---- the issuing warp: its first lane starts copies and products; nothing else runs here ----
    constexpr uint32_t idesc = instr_desc(128, PB);
    constexpr uint32_t idesc_mn = idesc | (1u << 16);                // the state's copy has p along its rows (MN-major B operand)
    if (lane == 0) {
      fetch_c(c0);
      fetch_bt(c0);
    }
    __syncwarp();
#pragma unroll 1
    for (int c = c0; c < c1; c++) {
      const uint32_t ph = (uint32_t)((c - c0) & 1);
      const int xw_off = L_::XW + (int)ph * L_::XW_BYTES;
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
            umma(tmem + 64u, smem_desc(sm0 + L_::C + s * L_::C_SLAB + kk * 32), smem_desc(sm0 + L_::S + (64 * s + 16 * kk) * 128),
                 idesc_mn, (s > 0 || kk > 0) ? 1u : 0u);
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
  // the state: this thread holds column n = 128 tile + 32 quarter + lane of S^T, all 32 rows p
  const int tile = NTILES == 1 ? 0 : (warp >> 2), quarter = warp & 3;
  const bool owns_state = NTILES == 2 || warp < 4;     // with one tile, warps 4..7 hold no state
  const int n_mine = 128 * tile + 32 * quarter + lane;
  const uint32_t t_state = tmem + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(tile * 32);
  const uint32_t t_d1 = tmem + ((uint32_t)(quarter * 32) << 16) + 64u + (uint32_t)((warp >> 2) * 16);
  float* slot = state + (((size_t)slots[b] * Hs + h) * P + p0) * N;
  uint32_t sreg[32];
  if (owns_state) {
    const bool have = start_pos[b] > 0;
#pragma unroll
    for (int p = 0; p < 32; p++) sreg[p] = have ? __float_as_uint(slot[(size_t)p * N + n_mine]) : 0u;
  }

  // Row mi = tid % 128 of a chunk and columns [16 mhalf, 16 mhalf + 16) of the block's 32 are this thread's: its
  // share of w x and of the outputs.  The row's weight w = 2^(total - cum) dt in the chunk's state update, its
  // factor e = 2^cum on C S^T and the chunk's decay come from ssd_intra_kernel, which has scanned the chunk's
  // decays anyway: no shuffle, barrier or shared memory is needed here while the tensor cores stream operands.
  const int mi = tid & 127, mhalf = tid >> 7;
  // What a thread reads from global memory is asked for at the top of an iteration, two chunks ahead of its use
  // and before the refills of C and B^T for the next chunk start: behind those 128 KB a load waits thousands of
  // cycles.  The chunks' boundaries are kept in registers for the same reason (an address then depends on no load).
  auto load_x = [&](int t0, int L, uint4 (&dst)[2]) {
    dst[0] = dst[1] = make_uint4(0u, 0u, 0u, 0u);
    if (mi < L) {
      const uint4* src = reinterpret_cast<const uint4*>(Xg + (size_t)(t0 + mi) * Cd + 16 * mhalf);
      dst[0] = __ldg(src);
      dst[1] = __ldg(src + 1);
    }
  };
  struct RowFactors { float w, e, decay; };
  auto load_factors = [&](int c, int t0, int L) -> RowFactors {
    RowFactors f{0.f, 0.f, 1.f};
    if (mi < L) {
      f.w = row_w[(size_t)(t0 + mi) * Hs + h];
      f.e = row_e[(size_t)(t0 + mi) * Hs + h];
    }
    if (c < c1) f.decay = seg_decay[(size_t)c * Hs + h];
    return f;
  };
  auto boundary = [&](int c) { return seg_start[min(c, c1)]; };
  // (w x)^T of chunk c into shared memory, K-major: row p, column j = mi (the transposing two-byte stores run while
  // the tensor cores work on the chunk before; with p along the rows instead, an MN-major operand and two 16-byte
  // stores a thread, the 32 products of the state update took three times as long)
  auto store_wx = [&](int c, float w, const uint4 (&x)[2]) {
    uint8_t* base = sm + L_::XW + ((c - c0) & 1) * L_::XW_BYTES;
    const uint32_t w8[8] = {x[0].x, x[0].y, x[0].z, x[0].w, x[1].x, x[1].y, x[1].z, x[1].w};
#pragma unroll
    for (int e = 0; e < 8; e++) {
      const int p = 16 * mhalf + 2 * e;
      const float2 x2 = unpack_bf16(w8[e]);
      *reinterpret_cast<unsigned short*>(base + sw128(p, mi, L_::X_SLAB)) = bf16_bits(x2.x * w);
      *reinterpret_cast<unsigned short*>(base + sw128(p + 1, mi, L_::X_SLAB)) = bf16_bits(x2.y * w);
    }
  };
  uint4 xv[2], xv_next[2];
  int sb0 = boundary(c0), sb1 = boundary(c0 + 1), sb2 = boundary(c0 + 2), sb3 = boundary(c0 + 3);
  RowFactors f_cur = load_factors(c0, sb0, sb1 - sb0), f_next, f_after;
  load_x(sb0, sb1 - sb0, xv);
  store_wx(c0, f_cur.w, xv);
  f_next = load_factors(c0 + 1, sb1, sb2 - sb1);
  load_x(sb1, sb2 - sb1, xv);

#pragma unroll 1
  for (int c = c0; c < c1; c++) {
    const int k = c - c0;
    const uint32_t ph = (uint32_t)(k & 1);
    const int t0 = sb0, L = sb1 - sb0;
    const int sb4 = boundary(c + 4);
    float4* yr = reinterpret_cast<float4*>(y + (size_t)(t0 + mi) * Di + (size_t)h * P + p0 + 16 * mhalf);
    float4 old[4];                                     // this chunk's outputs so far (M x + D x), if they are here
#pragma unroll
    for (int q = 0; q < 4; q++) old[q] = make_float4(0.f, 0.f, 0.f, 0.f);
    if (add_to_y && mi < L) {
#pragma unroll
      for (int q = 0; q < 4; q++) old[q] = yr[q];
    }
    f_after = load_factors(c + 2, sb2, sb3 - sb2);
    load_x(sb2, sb3 - sb2, xv_next);
    // ---- the state: wait for the last update, leave a bfloat16 copy for C S^T (row n, p along the row: the MN-major
    // B operand), decay it, hand it back ----
    if (c > c0) {
      wait(bar_s, ph ^ 1, 13);                         // the state update of the chunk before
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      __syncwarp();
      if (owns_state) tmem_ld32(t_state, sreg);
    }
    if (owns_state) {
      uint8_t* row = sm + L_::S + n_mine * 128;
#pragma unroll
      for (int u = 0; u < 4; u++) {
        uint32_t r4[4];
#pragma unroll
        for (int e = 0; e < 4; e++) r4[e] = pack_bf16(__uint_as_float(sreg[8 * u + 2 * e]), __uint_as_float(sreg[8 * u + 2 * e + 1]));
        *reinterpret_cast<uint4*>(row + ((u ^ (n_mine & 7)) << 4)) = make_uint4(r4[0], r4[1], r4[2], r4[3]);
      }
#pragma unroll
      for (int p = 0; p < 32; p++) sreg[p] = __float_as_uint(__uint_as_float(sreg[p]) * f_cur.decay);
      __syncwarp();
      tmem_st32(t_state, sreg);
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");     // what the threads wrote, before the tensor cores read it
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    asm volatile("bar.sync 2, %0;" ::"n"(THREADS) : "memory");       // hands the chunk to the issuing thread
    // ---- while its products run: w x of the next chunk (the other buffer was last read by the state update of
    // chunk c - 1: done, see the wait above) ----
    if (c + 1 < c1) store_wx(c + 1, f_next.w, xv);
    // ---- y += exp(cum_i) D1 for row i = 32 quarter + lane (= mi), columns [16 mhalf, 16 mhalf + 16); the part that
    // needs no state (M x + D x) is there already ----
    wait(bar_y, ph, 14);
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    {
      uint32_t d1[16];
      __syncwarp();
      tmem_ld16(t_d1, d1);
      if (mi < L) {
#pragma unroll
        for (int q = 0; q < 4; q++)
          yr[q] = make_float4(fmaf(f_cur.e, __uint_as_float(d1[4 * q]), old[q].x), fmaf(f_cur.e, __uint_as_float(d1[4 * q + 1]), old[q].y),
                              fmaf(f_cur.e, __uint_as_float(d1[4 * q + 2]), old[q].z), fmaf(f_cur.e, __uint_as_float(d1[4 * q + 3]), old[q].w));
      }
    }
    xv[0] = xv_next[0];
    xv[1] = xv_next[1];
    f_cur = f_next;
    f_next = f_after;
    sb0 = sb1; sb1 = sb2; sb2 = sb3; sb3 = sb4;
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
  // every agent is done with the item: tensor memory, shared memory and the barriers may be used again
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  }   // items
  if (warp == 0)
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TCOLS) : "memory");
}

int g_walk_blocks = 0;       // test hook: the grid of the walk (0: one block an SM, at most one an item)

template <int NTILES>
int launch(const CUtensorMap& mc, const CUtensorMap& mbt, const __nv_bfloat16* xbc, const float* row_w, const float* row_e,
           const float* seg_decay, float* state, const int* seg_start, const int* seq_seg_start,
           const int* slots, const int* start_pos, float* y, int add_to_y, int B, int Hs, int P, int G, int Cd, cudaStream_t stream) {
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(ssd_walk_tc_kernel<NTILES>, cudaFuncAttributeMaxDynamicSharedMemorySize, TcSmem<NTILES>::TOTAL) !=
        cudaSuccess)
      return tlc_fail(-2, "ssm_scan(chunk walk, tcgen05): cannot reserve %d bytes of shared memory", TcSmem<NTILES>::TOTAL);
    configured = true;
  }
  static int sms = 0;
  if (sms == 0) { int dev = 0; cudaGetDevice(&dev); cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev); }
  const long long items = (long long)B * Hs * (P / PB);
  const int blocks = (int)std::min<long long>(items, g_walk_blocks > 0 ? g_walk_blocks : sms);      // one block an SM (shared memory)
  tlc_launch(ssd_walk_tc_kernel<NTILES>, dim3(blocks), dim3(THREADS), (size_t)TcSmem<NTILES>::TOTAL, stream, mc, mbt, xbc, row_w,
             row_e, seg_decay, state, seg_start, seq_seg_start, slots, start_pos, y, add_to_y, B, Hs, P, G, Cd, tlc_error_words());
  TLC_CHECK_LAUNCH("ssm_scan(chunk walk, tcgen05)");
  return 0;
}

}  // namespace

// Test hook: how many blocks walk the items (0: chosen); with 1 one block walks every sequence and head in turn.
extern "C" void tlc_ssd_walk_blocks(int blocks) { g_walk_blocks = blocks; }

// Prepares the kernels' attributes outside any stream capture (called from tlc_ssd_init).
int tlc_ssd_tc_init() {
  if (cudaFuncSetAttribute(ssd_walk_tc_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, TcSmem<1>::TOTAL) != cudaSuccess ||
      cudaFuncSetAttribute(ssd_walk_tc_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, TcSmem<2>::TOTAL) != cudaSuccess)
    return tlc_fail(-2, "ssm_scan(chunk walk, tcgen05): cannot reserve shared memory");
  return 0;
}

// The walk.  N is 128 or 256; bt [n_seg, G, N, 128]: B of every chunk transposed (ssd_cb_kernel writes it beside C B^T).
int tlc_ssd_tc_run(const __nv_bfloat16* xbc, const float* row_w, const float* row_e, const float* seg_decay,
                   __nv_bfloat16* bt, float* state,
                   const int* seg_start, const int* seq_seg_start, const int* slots,
                   const int* start_pos, float* y, int add_to_y, int B, int n_seg, int T, int Hs, int P, int N, int G, int Cd,
                   cudaStream_t stream) {
  TLC_REQUIRE(N == 128 || N == 256, "ssm_scan(chunk walk, tcgen05): a state of %d columns", N);
  TLC_REQUIRE(tlc_error_words() != nullptr, "ssm_scan(chunk walk, tcgen05): the library is not set up (tlc_linear_init)");
  CUtensorMap mc, mbt;
  if (int rc = tlc_tensor_map_bf16(xbc, T, Cd, Cd, 64, Q, &mc)) return rc;
  if (int rc = tlc_tensor_map_bf16(bt, (long long)n_seg * G * N, Q, Q, 64, N, &mbt)) return rc;
  if (N == 128) return launch<1>(mc, mbt, xbc, row_w, row_e, seg_decay, state, seg_start, seq_seg_start, slots, start_pos, y, add_to_y, B, Hs, P, G, Cd, stream);
  return launch<2>(mc, mbt, xbc, row_w, row_e, seg_decay, state, seg_start, seq_seg_start, slots, start_pos, y, add_to_y, B, Hs, P, G, Cd, stream);
}
