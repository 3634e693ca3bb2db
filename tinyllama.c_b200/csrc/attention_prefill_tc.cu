// Attention for the prompts of a step on the 5th-generation tensor cores (sm_100a).
//
// Same math as the reference's op_attn (cpu_op.c:1010-1062): causal grouped-query attention, scale
// 1/sqrt(head_dim), max-subtracted softmax, optional window.  A block takes 128 consecutive new rows of one
// sequence and one query head and walks the sequence's key tiles (a page of 64 keys each) up to the diagonal:
//   * Q [128, hd] is loaded once by TMA; K and V tiles [64 keys, hd] come by TMA straight from the cache pages.
//     For S = Q K^T the keys are the rows of the B operand (K-major, as the pages have them); for O += P V the keys
//     are the reduction and hd runs along the rows of shared memory: V is an MN-major operand (its descriptor has
//     the 8-key groups 1,024 bytes apart and the 64-column halves of hd a slab apart), so no copy is transposed.
//     Keys past a sequence's end have P = 0; the values there must be finite (a cache starts as zeros and only
//     kernels write it), since 0 x NaN would spoil the row;
//   * three warps of one agent each, on three schedulers: one starts the copies, one issues S = Q K^T (M 128,
//     N 64, K hd) into one of two score buffers in tensor memory, two tiles ahead of the workers, and one issues
//     O += P V (M 128, N hd, K 64) into the output accumulator, also in tensor memory;
//   * eight worker warps in two groups: group w takes key tiles w, w + 2, ... with a score buffer, a P buffer
//     and an output accumulator of its own.  A thread owns a row of its group's tile: it reads the row's 64 scores
//     (tcgen05.ld), masks, takes the maximum, writes P = 2^(s - m) in bfloat16 into shared memory in the layout
//     tcgen05.mma reads, and keeps the row's sum.  Threads share nothing until the end, so the groups drift half
//     a tile apart: one's exponentials run under the other's loads and products;
//   * the maximum a row's numerators refer to moves only when the true maximum has grown by more than 2^8: the
//     row of the group's output accumulator is then read back, scaled and stored again (tcgen05.ld / st); P stays
//     below 2^8, far inside bfloat16's range, and the sum is 32-bit;
//   * at the end the groups' maxima and sums meet in shared memory and each group writes half of the columns of
//     O = (O_0 2^(m_0 - m) + O_1 2^(m_1 - m)) / (l_0 2^(m_0 - m) + l_1 2^(m_1 - m)).
// A tcgen05.mma of M 128, N 64, K 16 takes about 64 cycles here and one of N 128 about 96 (measured with clock
// stamps around the issue): 32 + N / 2, so the products take about 900 of the 1,300 cycles a tile costs.
// Sequences of unequal length are packed back to back; a block finds its sequence from cu_seqlens.  Every wait
// on an mbarrier is bounded (codes 21-27 of the error word); after one that ran out the block goes on without
// waiting, frees its tensor memory and returns, and the host raises.
#include "common.cuh"
#include "mbarrier.cuh"
#include "tcgen05.cuh"
#include <mutex>
#include <unordered_map>

namespace {

constexpr int BM = 128;                  // query rows per block
constexpr int BN = 64;                   // keys per tile = one page
static_assert(BN == TLC_PAGE, "a key tile is one page");
constexpr int KS = 4, VS = 3;            // stages of the K and V rings
constexpr int WORKERS = 256, THREADS = WORKERS + 96;
constexpr int NG = WORKERS / 128;        // worker groups: each takes every NG-th key tile, with an output accumulator of its own
static_assert(NG == 2, "two groups of workers");
constexpr float TAU = 8.0f;              // how far (in powers of two) a row's maximum may run ahead of its reference

__device__ __forceinline__ void workers_sync() { asm volatile("bar.sync 1, %0;" ::"n"(WORKERS) : "memory"); }
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&v);
}
__device__ __forceinline__ float ex2_quick(float x) {
  float r;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
  return r;
}

template <int HD>
struct FaSmem {
  static constexpr int Q_SLAB = BM * 128, Q = 0, Q_BYTES = (HD / 64) * Q_SLAB;
  static constexpr int K_SLAB = BN * 128, K_STAGE = (HD / 64) * K_SLAB, K = Q + Q_BYTES;
  static constexpr int V_STAGE = HD * 128, V = K + KS * K_STAGE;
  static constexpr int P_BUF = BM * 128, P = V + VS * V_STAGE;
  static constexpr int X = P + 2 * P_BUF;                 // [2][NG][128] floats: the groups' reference maxima and sums, at the end
  static constexpr int BARS = X + 2 * NG * BM * 4;        // mbarriers, tmem slot, dead flag
  static constexpr int N_BARS = 1 + 2 * KS + 2 * VS + 8;
  static constexpr int TABLE = BARS + N_BARS * 8 + 16;    // the block's page indices
  static int total(int max_tiles) { return TABLE + max_tiles * 4 + 1024; }
};

template <int HD>
__global__ void __launch_bounds__(THREADS, 1)
attention_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                            const __grid_constant__ CUtensorMap map_v, const int* __restrict__ block_table, int max_pages,
                            const int* __restrict__ cu_seqlens, const int* __restrict__ slots,
                            const int* __restrict__ start_pos, __nv_bfloat16* __restrict__ out, int n_seqs, int n_tiles, int H,
                            int KV, float scale_log2, int window, int out_ld, int n_split, float* __restrict__ part_o,
                            float* __restrict__ part_ml, ErrWords* err) {
  tlc_pdl(out);
  using L_ = FaSmem<HD>;
  constexpr int TCOLS = HD == 128 ? 512 : 256;            // the groups' scores at 0 and 64, their outputs at 128 and 128 + hd
  extern __shared__ uint8_t fa_raw[];
  uint8_t* sm = (uint8_t*)(((uintptr_t)fa_raw + 1023) & ~(uintptr_t)1023);
  float* xch = reinterpret_cast<float*>(sm + L_::X);
  uint64_t* bars = reinterpret_cast<uint64_t*>(sm + L_::BARS);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + L_::N_BARS);
  volatile int* dead = reinterpret_cast<volatile int*>(tmem_slot + 1);
  int* pages = reinterpret_cast<int*>(sm + L_::TABLE);
  __shared__ int s_seq, s_row0;
  const uint32_t sm0 = smem_u32(sm);
  const uint32_t bar_q = smem_u32(bars);
  auto k_full = [&](int s) { return smem_u32(bars + 1 + s); };
  auto k_empty = [&](int s) { return smem_u32(bars + 1 + KS + s); };
  auto v_full = [&](int s) { return smem_u32(bars + 1 + 2 * KS + s); };
  auto v_empty = [&](int s) { return smem_u32(bars + 1 + 2 * KS + VS + s); };
  auto s_full = [&](int i) { return smem_u32(bars + 1 + 2 * KS + 2 * VS + i); };
  auto s_free = [&](int i) { return smem_u32(bars + 1 + 2 * KS + 2 * VS + 2 + i); };
  auto p_ready = [&](int i) { return smem_u32(bars + 1 + 2 * KS + 2 * VS + 4 + i); };
  auto pv_done = [&](int i) { return smem_u32(bars + 1 + 2 * KS + 2 * VS + 6 + i); };

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
  auto wait = [&](uint32_t bar, uint32_t parity, int code) {
    if (*dead) return;
    if (!mbar_wait(bar, parity, err, code, wait_limit)) *dead = 1;
  };
  // An item is a 128-row tile of a sequence and a head; items are numbered with the tiles of most keys first and
  // a tile's heads side by side.  With one block an item (the launcher's choice when the GPU is the kernel's
  // alone) the loop below runs once.  With fewer blocks, block x takes items x, 2 nb - 1 - x, 2 nb + x, ...
  // (back and forth, so that every block gets long and short ones): the kernel then holds nb SMs, each for
  // about the same time, and leaves the others to kernels of other streams.  Between items the barriers are
  // made anew; tensor memory and the tiles of shared memory are simply used again.
  // With n_split > 1 (few row tiles and many keys: a piece of a long prompt) an item is also one of n_split
  // ranges of the tile's key tiles: it leaves its rows' maxima, sums and unnormalised outputs in part_ml
  // [T, H, n_split, 2] and part_o [T, H, n_split, hd], and attention_tc_merge_kernel adds the ranges up.
  const int n_items = n_tiles * H * n_split, nb = (int)gridDim.x;
#pragma unroll 1
  for (int round = 0;; round++) {
  const int item = round * nb + ((round & 1) ? nb - 1 - (int)blockIdx.x : (int)blockIdx.x);
  if (item >= n_items) break;
  const int key_range = item % n_split, h = (item / n_split) % H;
  // which sequence, and which of its 128-row tiles, is this item's
  if (tid == 0) {
    int tile = n_tiles - 1 - item / (H * n_split), found = -1, row0 = 0;
    for (int b = 0; b < n_seqs; b++) {
      const int nt = (cu_seqlens[b + 1] - cu_seqlens[b] + BM - 1) / BM;
      if (tile < nt) { found = b; row0 = tile * BM; break; }
      tile -= nt;
    }
    s_seq = found;
    s_row0 = row0;
    for (int i = 0; i < L_::N_BARS; i++) {
      const uint32_t bar = bar_q + 8 * i;               // every worker warp arrives once on s_free and p_ready, one agent on the rest
      if (round > 0) asm volatile("mbarrier.inval.shared::cta.b64 [%0];" ::"r"(bar) : "memory");   // nothing is pending on it (see the loader's last waits)
      mbar_init(bar, (bar == s_free(0) || bar == s_free(1) || bar == p_ready(0) || bar == p_ready(1)) ? 4 : 1);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  __syncthreads();
  const int b = s_seq;
  if (b >= 0) {
  const int i0 = s_row0;
  const int g = h / (H / KV);
  const int t0 = cu_seqlens[b], n_new = cu_seqlens[b + 1] - t0;
  const int rows = min(BM, n_new - i0);
  const int p0 = start_pos[b] + i0;                       // position of the block's first row
  const int tile_hi_all = (p0 + rows - 1) / BN;
  const int tile_lo_all = window > 0 ? max(0, p0 + 1 - window) / BN : 0;
  const int per_range = (tile_hi_all - tile_lo_all + n_split) / n_split;             // key tiles of a range, rounded up
  const int tile_lo = tile_lo_all + key_range * per_range;
  const int tile_hi = min(tile_hi_all, tile_lo + per_range - 1);
  const int n = max(0, tile_hi - tile_lo + 1);            // key tiles of this item (none: a range past the tile's keys)
  for (int i = tid; i < n; i += THREADS) pages[i] = block_table[(size_t)slots[b] * max_pages + tile_lo + i];
  __syncthreads();

  if (warp >= WORKERS / 32) {
    // ---- three warps of one agent each (their first lanes), on three schedulers: the copies, the products
    // S = Q K^T, the products O += P V.  One thread for all three was the kernel's bound: its instructions
    // share a scheduler's issue slots with four worker warps. ----
    const int role = warp - WORKERS / 32;
    constexpr uint32_t DESC_HI = (uint32_t)(1024 >> 4) | (1u << 14) | (2u << 29);      // see smem_desc
    auto desc_lo = [](uint32_t addr) { return ((addr & 0x3FFFFu) >> 4) | (1u << 16); };
    if (lane == 0 && role == 0) {
      mbar_expect_tx(bar_q, L_::Q_BYTES);
      for (int c = 0; c < HD / 64; c++) tma_load_2d(sm0 + L_::Q + c * L_::Q_SLAB, &map_q, bar_q, h * HD + 64 * c, t0 + i0);
      for (int t = 0; t < n; t++) {
        {
          const int st = t % KS;
          if (t >= KS) wait(k_empty(st), (uint32_t)(((t - KS) / KS) & 1), 26);       // S of tile t - KS is done
          mbar_expect_tx(k_full(st), L_::K_STAGE);
          for (int c = 0; c < HD / 64; c++)
            tma_load_2d(sm0 + L_::K + st * L_::K_STAGE + c * L_::K_SLAB, &map_k, k_full(st), 64 * c, (pages[t] * KV + g) * BN);
        }
        {
          const int st = t % VS;
          if (t >= VS) wait(v_empty(st), (uint32_t)(((t - VS) / VS) & 1), 27);       // P V of tile t - VS is done
          mbar_expect_tx(v_full(st), L_::V_STAGE);
          for (int c = 0; c < HD / 64; c++)
            tma_load_2d(sm0 + L_::V + st * L_::V_STAGE + c * L_::K_SLAB, &map_v, v_full(st), 64 * c, (pages[t] * KV + g) * BN);
        }
      }
      // the last arrivals on the stages' barriers (the products' commits), which nothing else waits for: after
      // them no barrier of this item has anything pending, and the next item may make them anew
      for (int t = max(0, n - KS); t < n; t++) wait(k_empty(t % KS), (uint32_t)((t / KS) & 1), 26);
      for (int t = max(0, n - VS); t < n; t++) wait(v_empty(t % VS), (uint32_t)((t / VS) & 1), 27);
    } else if (lane == 0 && role == 1) {
      // the scores run two tiles ahead of the workers: both score buffers are in use from the start
      constexpr uint32_t idesc_s = instr_desc(BM, BN);
      const uint32_t q_lo = desc_lo(sm0 + L_::Q);
      wait(bar_q, 0, 21);
      for (int t = 0; t < n; t++) {
        const int st = t % KS;
        wait(k_full(st), (uint32_t)((t / KS) & 1), 22);
        if (t >= 2) wait(s_free(t & 1), (uint32_t)(((t - 2) >> 1) & 1), 23);         // the workers hold scores t - 2 in registers
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t d = tmem + (uint32_t)((t & 1) * BN);
        const uint32_t k_lo = desc_lo(sm0 + L_::K + st * L_::K_STAGE);
#pragma unroll
        for (int c = 0; c < HD / 64; c++)
#pragma unroll
          for (int kk = 0; kk < 4; kk++)
            umma_halves(d, q_lo + (uint32_t)((c * L_::Q_SLAB + kk * 32) >> 4), k_lo + (uint32_t)((c * L_::K_SLAB + kk * 32) >> 4),
                        DESC_HI, idesc_s, (c > 0 || kk > 0) ? 1u : 0u);
        umma_commit(s_full(t & 1));
        umma_commit(k_empty(st));
      }
    } else if (lane == 0 && role == 2) {
      constexpr uint32_t idesc_o = instr_desc(BM, HD) | (1u << 16);                   // V is MN-major: hd runs along its rows
      for (int j = 0; j < n; j++) {
        const int st = j % VS;
        wait(v_full(st), (uint32_t)((j / VS) & 1), 25);
        wait(p_ready(j & 1), (uint32_t)((j >> 1) & 1), 24);                          // P of tile j is in shared memory
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t p_lo = desc_lo(sm0 + L_::P + (j & 1) * L_::P_BUF), v_lo = (desc_lo(sm0 + L_::V + st * L_::V_STAGE) & 0xFFFFu) | ((uint32_t)(L_::K_SLAB >> 4) << 16);
#pragma unroll
        for (int kk = 0; kk < 4; kk++)
          umma_halves(tmem + 128u + (uint32_t)((j & 1) * HD), p_lo + (uint32_t)(kk * 2), v_lo + (uint32_t)(kk * (16 * 128 >> 4)), DESC_HI, idesc_o,
                      (j >= 2 || kk > 0) ? 1u : 0u);
        umma_commit(pv_done(j & 1));
        umma_commit(v_empty(st));
      }
    }
    __syncwarp();
  } else {
    // ---- the workers: two groups of four warps; group w takes key tiles w, w + 2, ... and owns a score buffer, a
    // P buffer and an output accumulator.  Thread (quarter, lane) of a group owns row r of the tile: all 64
    // scores of a key tile and its row of the group's output.  Nothing is shared between threads until the end:
    // the groups run half a tile apart, one's exponentials under the other's loads and products. ----
    const int wg = warp >> 2, quarter = warp & 3, r = 32 * quarter + lane;
    const uint32_t lanes = (uint32_t)(quarter * 32) << 16;
    const int pr = p0 + r;                                // this row's position
    const uint32_t s_at = tmem + lanes + (uint32_t)(wg * BN);
    const uint32_t o_at = tmem + lanes + 128u + (uint32_t)(wg * HD);
    float m_ref = -INFINITY, l = 0.f;                     // the maximum the numerators refer to (scaled, log2), the sum
    int mine = 0;                                         // tiles this group has done
    for (int j = wg; j < n; j += NG, mine++) {
      uint32_t sr[64];
      wait(s_full(wg), (uint32_t)(mine & 1), 28);
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      __syncwarp();
      tmem_ld32_nowait(s_at, *reinterpret_cast<uint32_t(*)[32]>(&sr[0]));
      tmem_ld32_nowait(s_at + 32u, *reinterpret_cast<uint32_t(*)[32]>(&sr[32]));
      asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive(s_free(wg));             // the scores are in registers: the buffer may take tile j + 2
      const int kbase = (tile_lo + j) * BN;
      if (window > 0 || kbase + BN - 1 > p0) {
#pragma unroll
        for (int c = 0; c < 64; c++) {
          const int kp = kbase + c;
          if (!(kp <= pr && (window <= 0 || kp > pr - window))) sr[c] = 0xff800000u;     // -inf
        }
      }
      float mx = -INFINITY;
#pragma unroll
      for (int c = 0; c < 64; c++) mx = fmaxf(mx, __uint_as_float(sr[c]));
      mx *= scale_log2;
      // the reference maximum moves only when the true one has run ahead of it by more than 2^TAU
      const bool grow = mx > m_ref + TAU || (m_ref == -INFINITY && mx > -INFINITY);
      if (__any_sync(0xffffffffu, grow)) {
        float factor = 1.f;
        if (grow) {
          factor = m_ref == -INFINITY ? 0.f : ex2_quick(m_ref - mx);
          m_ref = mx;
          l *= factor;
        }
        if (mine > 0) {
          wait(pv_done(wg), (uint32_t)((mine - 1) & 1), 29);                          // every product into this output so far is done
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          __syncwarp();
#pragma unroll 1
          for (int c = 0; c < HD / 32; c++) {
            uint32_t o[32];
            tmem_ld32(o_at + (uint32_t)(32 * c), o);
#pragma unroll
            for (int e = 0; e < 32; e++) o[e] = __float_as_uint(__uint_as_float(o[e]) * factor);
            tmem_st32(o_at + (uint32_t)(32 * c), o);
          }
        }
      }
      const float neg = m_ref == -INFINITY ? 0.f : -m_ref;
      float sum = 0.f;
      uint32_t pk[32];
#pragma unroll
      for (int c = 0; c < 32; c++) {
        const float a = ex2_quick(fmaf(__uint_as_float(sr[2 * c]), scale_log2, neg));
        const float bq = ex2_quick(fmaf(__uint_as_float(sr[2 * c + 1]), scale_log2, neg));
        sum += a + bq;
        pk[c] = pack_bf16(a, bq);
      }
      l += sum;
      if (mine > 0) wait(pv_done(wg), (uint32_t)((mine - 1) & 1), 29);               // the group's P buffer is free
      uint8_t* prow = sm + L_::P + wg * L_::P_BUF + r * 128;
#pragma unroll
      for (int q = 0; q < 8; q++)
        *reinterpret_cast<uint4*>(prow + ((q ^ (r & 7)) << 4)) = make_uint4(pk[4 * q], pk[4 * q + 1], pk[4 * q + 2], pk[4 * q + 3]);
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();                                         // the warp's rows of P are written and fenced
      if (lane == 0) mbar_arrive(p_ready(wg));
    }
    // ---- the two groups' results meet: O = (O_0 2^(m_0 - m) + O_1 2^(m_1 - m)) / (l_0 2^(m_0 - m) + l_1 2^(m_1 - m)) ----
    if (mine > 0) wait(pv_done(wg), (uint32_t)((mine - 1) & 1), 29);
    xch[wg * BM + r] = m_ref;
    xch[(NG + wg) * BM + r] = l;
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    workers_sync();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const float m0 = xch[r], m1 = xch[BM + r];
    const float m_all = fmaxf(m0, m1);
    const float w0 = m0 == -INFINITY ? 0.f : ex2_quick(m0 - m_all), w1 = m1 == -INFINITY ? 0.f : ex2_quick(m1 - m_all);
    const float l_all = xch[NG * BM + r] * w0 + xch[(NG + 1) * BM + r] * w1;
    const bool whole = n_split == 1;                      // else the sums stay unnormalised: another kernel adds the ranges
    const float inv = whole ? 1.0f / l_all : 1.0f;
    const float f0 = w0 * inv, f1 = w1 * inv;
    const bool has0 = n > 0, has1 = n > 1;                // the group had a tile at all (else its accumulator was never written)
    const size_t part_at = whole ? 0 : (((size_t)(t0 + i0 + r) * H + h) * n_split + key_range);
    if (!whole && wg == 0 && r < rows) {
      part_ml[part_at * 2] = has0 ? m_all : -INFINITY;
      part_ml[part_at * 2 + 1] = has0 ? l_all : 0.f;
    }
    __syncwarp();
#pragma unroll 1
    for (int c = 0; c < HD / 64; c++) {                   // the group's half of the output columns, 32 at a time
      const int col = wg * (HD / 2) + 32 * c;
      uint32_t o[32];
      float acc[32];
      if (has0) tmem_ld32(tmem + lanes + 128u + (uint32_t)col, o);
#pragma unroll
      for (int e = 0; e < 32; e++) acc[e] = has0 ? __uint_as_float(o[e]) * f0 : 0.f;
      if (has1) {
        tmem_ld32(tmem + lanes + 128u + (uint32_t)(HD + col), o);
#pragma unroll
        for (int e = 0; e < 32; e++) acc[e] = fmaf(__uint_as_float(o[e]), f1, acc[e]);
      }
      if (!whole) {
        if (r < rows) {
          float4* dst = reinterpret_cast<float4*>(part_o + part_at * HD + col);
#pragma unroll
          for (int q = 0; q < 8; q++) dst[q] = make_float4(acc[4 * q], acc[4 * q + 1], acc[4 * q + 2], acc[4 * q + 3]);
        }
      } else if (r < rows) {
        uint4* dst = reinterpret_cast<uint4*>(out + (size_t)(t0 + i0 + r) * out_ld + (size_t)h * HD + col);
#pragma unroll
        for (int q = 0; q < 4; q++)
          dst[q] = make_uint4(pack_bf16(acc[8 * q], acc[8 * q + 1]), pack_bf16(acc[8 * q + 2], acc[8 * q + 3]),
                              pack_bf16(acc[8 * q + 4], acc[8 * q + 5]), pack_bf16(acc[8 * q + 6], acc[8 * q + 7]));
      }
    }
  }
  }  // b >= 0
  // every agent is done with the item: its copies have landed, its products have completed (the workers read
  // their last results, the loader saw the last commits), tensor memory and shared memory may be written again
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  }  // items
  if (warp == 0)
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TCOLS) : "memory");
}

// The ranges of a row's keys added up: out = sum_z o_z 2^(m_z - m) / sum_z l_z 2^(m_z - m), m the largest m_z of a
// range that had keys (the maxima are in the scaled log2 domain already).  grid (T, ceil(H / 4)), a warp per
// (row, head), a lane per 4 head dims (and their next 128).
constexpr int TC_MAX_SPLIT = 8;
__global__ void __launch_bounds__(128)
attention_tc_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml, __nv_bfloat16* __restrict__ out,
                          int H, int hd, int n_split, int out_ld) {
  tlc_pdl(part_o, part_ml, out);
  const int t = blockIdx.x, h = blockIdx.y * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (h >= H) return;
  const size_t at = ((size_t)t * H + h) * n_split;
  float mz[TC_MAX_SPLIT], lz[TC_MAX_SPLIT], m = -INFINITY;
#pragma unroll
  for (int z = 0; z < TC_MAX_SPLIT; z++) {
    mz[z] = z < n_split ? part_ml[(at + z) * 2] : -INFINITY;
    lz[z] = z < n_split ? part_ml[(at + z) * 2 + 1] : 0.f;
    if (lz[z] > 0.f) m = fmaxf(m, mz[z]);
  }
  float w[TC_MAX_SPLIT], l = 0.f;
#pragma unroll
  for (int z = 0; z < TC_MAX_SPLIT; z++) {
    w[z] = lz[z] > 0.f ? exp2f(mz[z] - m) : 0.f;
    l += lz[z] * w[z];
  }
  const float inv = 1.0f / l;
  for (int d = lane * 4; d < hd; d += 128) {
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int z = 0; z < TC_MAX_SPLIT; z++) {
      if (z < n_split && w[z] != 0.f) {
        const float4 v = *reinterpret_cast<const float4*>(part_o + (at + z) * hd + d);
        acc.x = fmaf(v.x, w[z], acc.x); acc.y = fmaf(v.y, w[z], acc.y); acc.z = fmaf(v.z, w[z], acc.z); acc.w = fmaf(v.w, w[z], acc.w);
      }
    }
    __nv_bfloat16* o = out + (size_t)t * out_ld + (size_t)h * hd + d;
    *reinterpret_cast<uint2*>(o) = make_uint2(pack_bf16(acc.x * inv, acc.y * inv), pack_bf16(acc.z * inv, acc.w * inv));
  }
}

// tensor maps of the cache pages, which stay where they are for the cache's lifetime
struct MapKey {
  const void* p; long long rows; int cols;
  bool operator==(const MapKey& o) const { return p == o.p && rows == o.rows && cols == o.cols; }
};
struct MapHash { size_t operator()(const MapKey& k) const { return (size_t)k.p * 1000003u ^ (size_t)k.rows * 31u ^ (size_t)k.cols; } };
std::unordered_map<MapKey, CUtensorMap, MapHash> g_page_maps;
std::mutex g_page_mu;

int page_map(const void* pages, long long rows, int hd, CUtensorMap* out) {
  MapKey key{pages, rows, hd};
  std::lock_guard<std::mutex> lk(g_page_mu);
  auto it = g_page_maps.find(key);
  if (it != g_page_maps.end()) { *out = it->second; return 0; }
  CUtensorMap m;
  if (int rc = tlc_tensor_map_bf16(pages, rows, hd, hd, 64, BN, &m)) return rc;
  if (g_page_maps.size() > 1024) g_page_maps.clear();
  g_page_maps[key] = m;
  *out = m;
  return 0;
}

template <int HD>
int run(const __nv_bfloat16* q, const __nv_bfloat16* k_pages, const __nv_bfloat16* v_pages, long long n_page_rows,
        const int* block_table, int max_pages, const int* cu_seqlens, const int* slots, const int* start_pos,
        __nv_bfloat16* out, int n_seqs, int n_tiles_bound, int H, int KV, float scale, int window,
        int p_max, int T, int out_ld, int max_blocks, int n_split, float* part_o, float* part_ml, cudaStream_t stream) {
  static bool configured = false;
  const int smem = FaSmem<HD>::total(p_max);
  TLC_REQUIRE(smem <= 220 * 1024, "attention(prefill, tcgen05): %d key tiles need %d bytes of shared memory", p_max, smem);
  if (!configured) {
    if (cudaFuncSetAttribute(attention_prefill_tc_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024) != cudaSuccess)
      return tlc_fail(-2, "attention(prefill, tcgen05): cannot reserve shared memory");
    configured = true;
  }
  CUtensorMap mq, mk, mv;
  if (int rc = tlc_tensor_map_bf16(q, T, (long long)H * HD, (long long)H * HD, 64, BM, &mq)) return rc;
  if (int rc = page_map(k_pages, n_page_rows, HD, &mk)) return rc;
  if (int rc = page_map(v_pages, n_page_rows, HD, &mv)) return rc;
  const long long items = (long long)n_tiles_bound * H * n_split;
  const int blocks = (int)(max_blocks > 0 && max_blocks < items ? max_blocks : items);
  tlc_launch(attention_prefill_tc_kernel<HD>, dim3(blocks), dim3(THREADS), (size_t)smem, stream, mq, mk, mv,
             block_table, max_pages, cu_seqlens, slots, start_pos, out, n_seqs, n_tiles_bound, H, KV, scale * 1.4426950408889634f,
             window, out_ld, n_split, part_o, part_ml, tlc_error_words());
  TLC_CHECK_LAUNCH("attention(prefill, tcgen05)");
  if (n_split > 1) {
    tlc_launch(attention_tc_merge_kernel, dim3(T, (H + 3) / 4), dim3(128), 0, stream, (const float*)part_o, (const float*)part_ml, out, H,
               HD, n_split, out_ld);
    TLC_CHECK_LAUNCH("attention(prefill, tcgen05, merge)");
  }
  return 0;
}

}  // namespace

// How many ranges to cut the keys of every row tile into: more than one when the (tile, head) items leave more than
// half of the SMs idle and the longest sequence has at least 32 key tiles (a piece of a long prompt: 512 new rows
// at position 33,000 of the 1.5B sizes are 40 items of 530 key tiles, 13.2 ms a step; in three ranges 7 ms).
extern "C" int tlc_attention_prefill_tc_splits(int n_tiles_bound, int H, int max_keys) {
  static int sms = 0;
  if (sms == 0) { int dev = 0; cudaGetDevice(&dev); cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev); }
  const long long items = (long long)n_tiles_bound * H;
  const int p_max = (max_keys + BN - 1) / BN;
  if (items <= 0 || items * 2 > sms || p_max < 32) return 1;
  const int n = (int)std::min<long long>(std::min<long long>(TC_MAX_SPLIT, sms / items), p_max / 16);
  return n < 2 ? 1 : n;
}

extern "C" int tlc_attention_prefill_tc_ok(int dtype, int hd, int H, int KV) {
  return dtype == TLC_BF16 && (hd == 64 || hd == 128) && KV > 0 && H % KV == 0 && H <= 65535 && KV <= 65535;
}

// n_tiles_bound: an upper bound of sum_b ceil(n_new_b / 128) (e.g. T / 128 + n_seqs); max_keys: keys of the longest
// sequence after this step; n_pages: pages of the cache (k_pages and v_pages are [n_pages, KV, 64, hd]).
// max_blocks: 0, or how many blocks (hence SMs) the kernel may hold: it then works through its (tile, head) items
// with that many blocks, for callers that run other kernels beside it.
// n_split > 1 (at most 8; tlc_attention_prefill_tc_splits suggests it): the keys of every row tile are cut into
// that many ranges that run as items of their own; part_o [T, H, n_split, hd] and part_ml [T, H, n_split, 2]
// (32-bit) hold the ranges' results until a second kernel has added them up.
extern "C" int tlc_attention_prefill_tc(const void* q, const void* k_pages, const void* v_pages, int n_pages,
                                        const int* block_table, int max_pages, const int* cu_seqlens, const int* slots,
                                        const int* start_pos, void* out, int n_seqs, int n_tiles_bound, int H, int KV,
                                        int hd, float scale, int window, int max_keys, int T, int out_ld, int max_blocks,
                                        int n_split, float* part_o, float* part_ml, cudaStream_t stream) {
  if (n_seqs == 0 || n_tiles_bound == 0 || T == 0) return 0;
  if (out_ld <= 0) out_ld = H * hd;
  TLC_REQUIRE(tlc_attention_prefill_tc_ok(TLC_BF16, hd, H, KV), "attention(prefill, tcgen05): %d heads, %d key/value heads of size %d are not built", H, KV, hd);
  TLC_REQUIRE(out_ld % 8 == 0 && ((uintptr_t)out % 16) == 0 && ((uintptr_t)q % 16) == 0 &&
              ((uintptr_t)k_pages % 16) == 0 && ((uintptr_t)v_pages % 16) == 0, "attention(prefill, tcgen05): rows must start on 16-byte boundaries");
  TLC_REQUIRE(tlc_error_words() != nullptr, "attention(prefill, tcgen05): the library is not set up (tlc_linear_init)");
  const int p_max = (max_keys + BN - 1) / BN;
  TLC_REQUIRE(p_max >= 1 && p_max <= 65535, "attention(prefill, tcgen05): %d keys", max_keys);
  if (n_split < 1) n_split = 1;
  TLC_REQUIRE(n_split <= TC_MAX_SPLIT && (n_split == 1 || (part_o != nullptr && part_ml != nullptr && ((uintptr_t)part_o % 16) == 0)),
              "attention(prefill, tcgen05): %d key ranges need 16-byte aligned scratch (at most %d ranges)", n_split, TC_MAX_SPLIT);
  const long long rows = (long long)n_pages * KV * BN;
  const __nv_bfloat16 *qp = (const __nv_bfloat16*)q, *kp = (const __nv_bfloat16*)k_pages, *vp = (const __nv_bfloat16*)v_pages;
  if (hd == 64)
    return run<64>(qp, kp, vp, rows, block_table, max_pages, cu_seqlens, slots, start_pos, (__nv_bfloat16*)out,
                   n_seqs, n_tiles_bound, H, KV, scale, window, p_max, T, out_ld, max_blocks, n_split, part_o, part_ml, stream);
  return run<128>(qp, kp, vp, rows, block_table, max_pages, cu_seqlens, slots, start_pos, (__nv_bfloat16*)out,
                  n_seqs, n_tiles_bound, H, KV, scale, window, p_max, T, out_ld, max_blocks, n_split, part_o, part_ml, stream);
}
