// bfloat16 linear layers on the 5th-generation tensor cores (sm_100a):
//   out[m, n] (+)= (sum_k a[m, k] * w[n, k]) * colscale[n] + colbias[n],  32-bit accumulation.
//
// The reference multiplies with hand-written kernels of its own: FP32 FMA tiles
// (gpu.cu:1542, matmul_kernel_tiled) and a warp-per-row product (gpu.cu:1008); it has no
// tensor-core path for 16-bit weights.  This file is the B200 form of the same product:
//   * both operands are K-major ([rows, K] with K contiguous), so TMA
//     (cp.async.bulk.tensor.2d, 128-byte swizzle) stages [128 x 64] tiles of each into a
//     ring of shared-memory buffers; out-of-range rows and the K tail arrive as zeros;
//   * one elected thread issues tcgen05.mma (M=128, N=BN = 64, 128 or 256, K=16 per
//     instruction) with the accumulator [128 x BN] in tensor memory, and tcgen05.commit hands
//     each ring slot back to the loader;
//   * four warps read the accumulator back with tcgen05.ld (each warp its 32 lanes = rows,
//     32 columns at a time) and apply the epilogue in registers: column scale and bias (staged
//     once a tile in shared memory), optional add into the 32-bit residual or SwiGLU of
//     interleaved gate|up columns; a lane writes the 32 columns of its row 16 bytes at a time
//     (pieces that stick out of the matrix, or rows off 16-byte boundaries, go through a padded
//     shared-memory tile instead and are written a row of 32 columns per instruction).
// Warp roles: 0 = TMA loader, 1 = MMA issuer and owner of the tensor-memory allocation,
// 2..5 = epilogue.  Every wait on an mbarrier is bounded; a wait that runs out records an
// error code that the host reads, and the kernel frees its tensor memory and returns.
#include "common.cuh"
#include "mbarrier.cuh"
#include "tcgen05.cuh"
#include <atomic>
#include <mutex>
#include <unordered_map>

// gemm_tcgen05_few_rows.cu
int tlc_linear_few_rows_run(const void* a, int lda, const void* w, int ldw, void* out, int out_dtype, int ldo,
                            const float* colscale, const float* colbias, int accumulate, int M, int N, int K,
                            cudaStream_t stream);
int tlc_linear_few_rows_swiglu(const void* a, int lda, const void* w, int ldw, void* out, int out_dtype, int ldo,
                               const float* colscale, const float* colbias, int M, int N, int K, cudaStream_t stream);

namespace {

constexpr int BM = 128;
constexpr int BK = 64;                 // 64 bf16 = 128 bytes = one swizzle row
constexpr int THREADS = 192;
__device__ __forceinline__ uint32_t pack2(float a, float b) {
  __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&v);
}

template <int BN, int STAGES, bool PAIR = false>
struct Smem {
  static constexpr int A_BYTES = BM * BK * 2;
  static constexpr int B_ROWS = PAIR ? BN / 2 : BN;        // weight rows a block stages: each block of a pair half of the tile's
  static constexpr int B_BYTES = B_ROWS * BK * 2;
  static constexpr int TILES = STAGES * (A_BYTES + B_BYTES);
  static constexpr int STAGE_TILE = 1280;                  // floats per epilogue warp: a padded 32 x 33 tile, or 32 x 32 for the copy engine (5 KB: tiles start on 1 KB)
  static constexpr int STAGING = 4 * (STAGE_TILE + 2 * BN) * 4;   // per epilogue warp: that tile, the tile's column scales and biases
  static constexpr int N_BARS = 2 * STAGES + 4;            // full, empty per stage; accumulator full, empty x2
  static constexpr int TOTAL = TILES + STAGING + N_BARS * 8 + 16 + 1024;   // + tmem slot + alignment slack
};

// Persistent: a block walks tiles blockIdx.x, blockIdx.x + gridDim.x, ... (row tiles fastest, so
// that blocks running together share a weight tile in L2).  The shared-memory ring runs on across
// tiles; the accumulator alternates between two halves of tensor memory so that the epilogue of
// one tile overlaps the products of the next.
// With SWIGLU the weight rows come in groups of 16 = 8 gate rows followed by their 8 up rows;
// the epilogue writes silu(gate) * up, half as many columns ([M, N/2], row stride ldo).
// With PAIR two blocks (a cluster of two) share a tile of 256 rows x BN columns: each stages its 128 rows of the
// activations and its BN / 2 rows of the weights, the block of rank 0 issues tcgen05.mma.cta_group::2 (M = 256)
// over both blocks' shared memory, and each finds its 128 rows of the result in its own tensor memory.  A block
// then reads (128 + BN / 2) x 64 operand values for 128 x BN x 64 products where a single block reads
// (128 + BN) x 64: a third less traffic into and out of shared memory, which bounds the single-block tile.
template <typename TO, int BN, int STAGES, bool SWIGLU, bool PAIR>
__global__ void __launch_bounds__(THREADS, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                    TO* __restrict__ out, int ldo, const float* __restrict__ colscale,
                    const float* __restrict__ colbias, int accumulate, int M, int N, int K, ErrWords* err,
                    int splits, float* __restrict__ part, unsigned* __restrict__ arrivals,
                    const __grid_constant__ CUtensorMap map_o, int tma_out) {
  // The set-up and the first weight tiles do not depend on the previous kernel of the stream: they go ahead of
  // the wait on it.  The loader waits before its first activation tile, the epilogue warps before they touch
  // `out`; the issuer reads shared memory only.
  asm volatile("griddepcontrol.launch_dependents;");
  using S = Smem<BN, STAGES, PAIR>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* a_tiles = smem;
  uint8_t* b_tiles = smem + STAGES * S::A_BYTES;
  float* staging = (float*)(smem + S::TILES);
  uint64_t* bars = (uint64_t*)(smem + S::TILES + S::STAGING);
  uint32_t* tmem_slot = (uint32_t*)(bars + S::N_BARS);
  const uint32_t full0 = smem_u32(bars), empty0 = smem_u32(bars + STAGES);
  const uint32_t acc_full0 = smem_u32(bars + 2 * STAGES), acc_empty0 = smem_u32(bars + 2 * STAGES + 2);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long wait_limit = mbar_wait_limit(err);
  constexpr int TM = PAIR ? 2 * BM : BM;               // rows of a tile
  const uint32_t rank = PAIR ? cluster_rank() : 0u;    // which block of the pair
  const int walker = PAIR ? (int)blockIdx.x >> 1 : (int)blockIdx.x;      // blocks, or pairs, walk the tiles
  const int walkers = PAIR ? (int)gridDim.x >> 1 : (int)gridDim.x;
  const int m_tiles = (M + TM - 1) / TM, n_tiles = (N + BN - 1) / BN;
  // splits > 1: a tile's K-steps are shared by `splits` blocks; each leaves its partial accumulator in `part`
  // [splits, M, N] and the last one to arrive (arrivals[tile * 4 + quarter], back at zero afterwards) adds
  // them in order and finishes the tile.  Tile index = split * (tiles of the output) + output tile.
  const int out_tiles = m_tiles * n_tiles;
  const int total_tiles = out_tiles * splits;
  const int num_k = (K + BK - 1) / BK;
  const int k_per = (num_k + splits - 1) / splits;     // every split has at least one step (the launcher sees to it)

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; s++) { mbar_init(full0 + 8 * s, 1); mbar_init(empty0 + 8 * s, 1); }
    for (int s = 0; s < 2; s++) { mbar_init(acc_full0 + 8 * s, 1); mbar_init(acc_empty0 + 8 * s, PAIR ? 8 : 4); }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {   // the whole warp (of both blocks of a pair) allocates two accumulators of BN columns
    if constexpr (PAIR) {
      asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(2 * BN)
                   : "memory");
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    } else {
      asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(2 * BN)
                   : "memory");
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  if constexpr (PAIR) cluster_sync();                  // the other block's mbarriers are initialised too
  else __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {                                   // ---- TMA loader ----
      int it = 0, issued = 0;
      bool ok = true;
      bool waited = false;                             // on the previous kernel of the stream
      int3 pending_a[STAGES];                          // activation tiles (stage, k, m) held back until then
      int n_pending = 0;
      const int my_tiles = walker < total_tiles ? (total_tiles - 1 - walker) / walkers + 1 : 0;
      const int first_run = my_tiles * (num_k - (splits - 1) * k_per);   // stage fills this block issues at least
      // a pair's copies all count on the mbarriers of the block of rank 0, whose issuer waits for them
      const uint32_t full_bar0 = PAIR ? cluster_address(full0, 0) : full0;
      auto load = [&](uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1) {
        if constexpr (PAIR) tma_load_2d_pair(dst, map, bar, c0, c1);
        else tma_load_2d(dst, map, bar, c0, c1);
      };
      for (int tile = walker; tile < total_tiles && ok; tile += walkers) {
        const int ot = tile % out_tiles, sp = tile / out_tiles;
        const int m0 = (ot % m_tiles) * TM + (int)rank * BM, n0 = (ot / m_tiles) * BN + (int)rank * S::B_ROWS;
        const int k_end = min(num_k, (sp + 1) * k_per);
        for (int k = sp * k_per; k < k_end; k++, it++) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          ok = mbar_wait(empty0 + 8 * s, ph ^ 1, err, 1, wait_limit);
          if (!ok) break;
          if (rank == 0) mbar_expect_tx(full0 + 8 * s, (PAIR ? 2 : 1) * (S::A_BYTES + S::B_BYTES));
          load(smem_u32(b_tiles + s * S::B_BYTES), &map_b, full_bar0 + 8 * s, k * BK, n0);
          if (!waited) {
            // the weight tiles of the first stages are on their way; the activations need the previous kernel
            if (it + 1 < STAGES && it + 1 < first_run) { pending_a[n_pending++] = make_int3(s, k * BK, m0); issued = it + 1; continue; }
            asm volatile("griddepcontrol.wait;" ::: "memory");
            waited = true;
            for (int i = 0; i < n_pending; i++)
              load(smem_u32(a_tiles + pending_a[i].x * S::A_BYTES), &map_a, full_bar0 + 8 * pending_a[i].x, pending_a[i].y, pending_a[i].z);
          }
          load(smem_u32(a_tiles + s * S::A_BYTES), &map_a, full_bar0 + 8 * s, k * BK, m0);
          issued = it + 1;
        }
      }
      if (rank == 0 && (!ok || *(volatile int*)&err->flag != 0)) {
        // something went wrong: let the copies still in flight land before the block exits (a pair's count on
        // these mbarriers, and no block of a pair leaves before both have come to the kernel's end)
        for (int i = max(0, issued - STAGES); i < issued; i++)
          mbar_wait(full0 + 8 * (i % STAGES), (i / STAGES) & 1, err, 4, wait_limit);
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && rank == 0) {                      // ---- MMA issuer ----
      constexpr uint32_t idesc = instr_desc(TM, BN);
      int it = 0, local = 0;
      bool ok = true;
      for (int tile = walker; tile < total_tiles && ok; tile += walkers, local++) {
        const int as = local & 1;
        ok = mbar_wait(acc_empty0 + 8 * as, ((local >> 1) & 1) ^ 1, err, 5, wait_limit);   // the epilogue has drained this half
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t d_tmem = tmem + (uint32_t)(as * BN);
        const int sp = tile / out_tiles;
        const int k_begin = sp * k_per, k_end = min(num_k, (sp + 1) * k_per);
        for (int k = k_begin; k < k_end; k++, it++) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          ok = mbar_wait(full0 + 8 * s, ph, err, 2, wait_limit);
          if (!ok) break;
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const uint32_t a_addr = smem_u32(a_tiles + s * S::A_BYTES), b_addr = smem_u32(b_tiles + s * S::B_BYTES);
#pragma unroll
          for (int kk = 0; kk < BK / UMMA_K; kk++) {
            const uint64_t da = smem_desc(a_addr + kk * UMMA_K * 2), db = smem_desc(b_addr + kk * UMMA_K * 2);
            if constexpr (PAIR) umma_pair(d_tmem, da, db, idesc, (k > k_begin || kk > 0) ? 1u : 0u);
            else umma(d_tmem, da, db, idesc, (k > k_begin || kk > 0) ? 1u : 0u);
          }
          // the slot is free (in both blocks of a pair) once these MMAs have read it
          if constexpr (PAIR) umma_commit_pair(empty0 + 8 * s);
          else umma_commit(empty0 + 8 * s);
        }
        if (ok) {                                      // this tile's accumulator is complete
          if constexpr (PAIR) umma_commit_pair(acc_full0 + 8 * as);
          else umma_commit(acc_full0 + 8 * as);
        }
      }
    }
  } else {                                             // ---- epilogue, warps 2..5 ----
    const int quarter = warp & 3;                      // a warp may touch lanes 32*(warp%4) .. +31 only
    float* st = staging + quarter * S::STAGE_TILE;
    float* sc = staging + 4 * S::STAGE_TILE + quarter * 2 * BN;   // [BN] column scales | [BN] column biases of the tile
    int local = 0;
    bool ok = true;
    // a lane can write 32 consecutive columns of its row 16 bytes at a time when rows start on 16-byte boundaries
    const bool rows_aligned = (((uintptr_t)out) & 15) == 0 && ((size_t)ldo * sizeof(TO)) % 16 == 0;
    tlc_wait(out);                                     // `out` may still be read or written by the previous kernel
    for (int tile = walker; tile < total_tiles && ok; tile += walkers, local++) {
      const int as = local & 1;
      const int ot = tile % out_tiles, sp = tile / out_tiles;
      const int m0 = (ot % m_tiles) * TM + (int)rank * BM, n0 = (ot / m_tiles) * BN;
      ok = mbar_wait(acc_full0 + 8 * as, (local >> 1) & 1, err, 3, wait_limit);
      if (!ok) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const int mrow0 = m0 + quarter * 32;
      const bool split = !SWIGLU && splits > 1;
      if (split) {
        // this block's share of the tile's sum goes to scratch; the warp that finds the other shares of its
        // 32 rows already there adds them up and finishes the rows
        const int m = mrow0 + lane;
        const bool vec = (N & 3) == 0;
#pragma unroll 1
        for (int c = 0; c < BN / 32; c++) {
          const int nc0 = n0 + c * 32;
          if (nc0 >= N) break;
          uint32_t r[32];
          tmem_ld32(tmem + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(as * BN + c * 32), r);
          if (m < M) {
            float* dst = part + ((size_t)sp * M + m) * N + nc0;
            if (vec && nc0 + 32 <= N) {
#pragma unroll
              for (int q = 0; q < 8; q++)
                __stcg(reinterpret_cast<float4*>(dst) + q, make_float4(__uint_as_float(r[4 * q]), __uint_as_float(r[4 * q + 1]),
                                                                        __uint_as_float(r[4 * q + 2]), __uint_as_float(r[4 * q + 3])));
            } else {
#pragma unroll
              for (int j = 0; j < 32; j++) if (nc0 + j < N) __stcg(dst + j, __uint_as_float(r[j]));
            }
          }
        }
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(acc_empty0 + 8 * as) : "memory");
        __threadfence();
        __syncwarp();
        unsigned old = 0;
        if (lane == 0) old = atomicInc(arrivals + (size_t)ot * 4 + quarter, (unsigned)(splits - 1));
        old = __shfl_sync(0xffffffffu, old, 0);
        if (old != (unsigned)(splits - 1)) continue;      // another block finishes these rows
        __threadfence();
      }
      const bool scaled = colscale != nullptr || colbias != nullptr;
      if (scaled) {
        // the tile's column scales and biases once into the warp's staging area: every lane needs all of them
        __syncwarp();
        for (int j = lane; j < BN; j += 32) {
          const int n = n0 + j;
          sc[j] = (colscale && n < N) ? colscale[n] : 1.0f;
          sc[BN + j] = (colbias && n < N) ? colbias[n] : 0.0f;
        }
        __syncwarp();
      }
#pragma unroll 1
      for (int c = 0; c < BN / 32; c++) {
        const int nc0 = n0 + c * 32;
        if (nc0 >= N) break;
        uint32_t r[32];
        if (!split) {
          tmem_ld32(tmem + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(as * BN + c * 32), r);
        } else {
          // the shares of all splits, added in the order of the splits
          float v[32];
#pragma unroll
          for (int j = 0; j < 32; j++) v[j] = 0.f;
          const int m = mrow0 + lane;
          if (m < M) {
            const bool vec = (N & 3) == 0 && nc0 + 32 <= N;
            for (int sx = 0; sx < splits; sx++) {
              const float* src = part + ((size_t)sx * M + m) * N + nc0;
              if (vec) {
                float4 x[8];
#pragma unroll
                for (int q = 0; q < 8; q++) x[q] = __ldcg(reinterpret_cast<const float4*>(src) + q);
#pragma unroll
                for (int q = 0; q < 8; q++) { v[4 * q] += x[q].x; v[4 * q + 1] += x[q].y; v[4 * q + 2] += x[q].z; v[4 * q + 3] += x[q].w; }
              } else {
#pragma unroll
                for (int j = 0; j < 32; j++) if (nc0 + j < N) v[j] += __ldcg(src + j);
              }
            }
          }
#pragma unroll
          for (int j = 0; j < 32; j++) r[j] = __float_as_uint(v[j]);
        }
        if (SWIGLU) {
          // A lane holds 32 columns of its row: gates 0..7 | ups 8..15 | gates 16..23 | ups 24..31, i.e. 16
          // features whose gate and up are both in its registers.  It writes 16 consecutive values.
          const int m = mrow0 + lane;
          const int oc0 = nc0 >> 1;
          float o16[16];
#pragma unroll
          for (int f = 0; f < 16; f++) {
            const int gcol = ((f >> 3) << 4) + (f & 7);
            float vg = __uint_as_float(r[gcol]), vu = __uint_as_float(r[gcol + 8]);
            if (scaled) {
              const int jg = c * 32 + gcol;
              vg = vg * sc[jg] + sc[BN + jg];
              vu = vu * sc[jg + 8] + sc[BN + jg + 8];
            }
            o16[f] = silu_quick(vg) * vu;
          }
          if (m < M) {
            TO* dst = out + (size_t)m * ldo + oc0;
            if (nc0 + 32 <= N && (((uintptr_t)dst) & 15) == 0 && sizeof(TO) == 2) {
              uint4 lo, hi;
              lo.x = pack2(o16[0], o16[1]); lo.y = pack2(o16[2], o16[3]); lo.z = pack2(o16[4], o16[5]); lo.w = pack2(o16[6], o16[7]);
              hi.x = pack2(o16[8], o16[9]); hi.y = pack2(o16[10], o16[11]); hi.z = pack2(o16[12], o16[13]); hi.w = pack2(o16[14], o16[15]);
              reinterpret_cast<uint4*>(dst)[0] = lo;
              reinterpret_cast<uint4*>(dst)[1] = hi;
            } else {
#pragma unroll
              for (int f = 0; f < 16; f++) {
                const int gcol = ((f >> 3) << 4) + (f & 7);
                if (nc0 + gcol + 8 < N) dst[f] = from_f32<TO>(o16[f]);
              }
            }
          }
          continue;
        }
        if constexpr (!SWIGLU && sizeof(TO) == 4) {
          if (tma_out && !split) {
            // 32-bit output through the copy engine: the lane writes the 32 columns of its row into a 32 x 32
            // tile of shared memory (128-byte rows, 16-byte pieces swizzled as the tensor map expects) and one
            // bulk tensor copy stores it, or adds it to what is there (the sum is made at the L2: no read of
            // the old values by the SM, no 32 separate lines per store instruction).  The copy clips at M and N.
            if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");   // the tile's last use
            __syncwarp();
            const uint32_t row = smem_u32(st) + (uint32_t)lane * 128u;
#pragma unroll
            for (int q = 0; q < 8; q++) {
              float v0 = __uint_as_float(r[4 * q]), v1 = __uint_as_float(r[4 * q + 1]), v2 = __uint_as_float(r[4 * q + 2]),
                    v3 = __uint_as_float(r[4 * q + 3]);
              if (scaled) {
                const int j = c * 32 + 4 * q;
                v0 = v0 * sc[j] + sc[BN + j]; v1 = v1 * sc[j + 1] + sc[BN + j + 1];
                v2 = v2 * sc[j + 2] + sc[BN + j + 2]; v3 = v3 * sc[j + 3] + sc[BN + j + 3];
              }
              asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(row + (uint32_t)((q ^ (lane & 7)) << 4)), "f"(v0),
                           "f"(v1), "f"(v2), "f"(v3) : "memory");
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
            if (lane == 0 && mrow0 < M) {
              if (accumulate)
                asm volatile("cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.bulk_group [%0, {%2, %3}], [%1];" ::"l"(&map_o),
                             "r"(smem_u32(st)), "r"(nc0), "r"(mrow0) : "memory");
              else
                asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];" ::"l"(&map_o),
                             "r"(smem_u32(st)), "r"(nc0), "r"(mrow0) : "memory");
              asm volatile("cp.async.bulk.commit_group;" ::: "memory");
            }
            continue;
          }
        }
        if (rows_aligned && nc0 + 32 <= N && (nc0 * sizeof(TO)) % 16 == 0) {
          // the whole piece lies inside the matrix: a lane finishes the 32 columns of its row in registers and
          // writes them 16 bytes at a time (no trip through shared memory)
          const int m = mrow0 + lane;
          if (m < M) {
            TO* dst = out + (size_t)m * ldo + nc0;
            float v[32];
#pragma unroll
            for (int j = 0; j < 32; j++) v[j] = __uint_as_float(r[j]);
            if (scaled) {
#pragma unroll
              for (int j = 0; j < 32; j++) v[j] = v[j] * sc[c * 32 + j] + sc[BN + c * 32 + j];
            }
            if (sizeof(TO) == 4) {
              float4* d4 = reinterpret_cast<float4*>(dst);
              if (accumulate) {
                float4 old[8];
#pragma unroll
                for (int q = 0; q < 8; q++) old[q] = d4[q];
#pragma unroll
                for (int q = 0; q < 8; q++) { v[4 * q] += old[q].x; v[4 * q + 1] += old[q].y; v[4 * q + 2] += old[q].z; v[4 * q + 3] += old[q].w; }
              }
#pragma unroll
              for (int q = 0; q < 8; q++) d4[q] = make_float4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
            } else {
              uint4* d4 = reinterpret_cast<uint4*>(dst);
              if (accumulate) {
                uint4 old[4];
#pragma unroll
                for (int q = 0; q < 4; q++) old[q] = d4[q];
#pragma unroll
                for (int q = 0; q < 4; q++) {
                  const uint32_t w4[4] = {old[q].x, old[q].y, old[q].z, old[q].w};
#pragma unroll
                  for (int e = 0; e < 4; e++) {
                    v[8 * q + 2 * e] += __uint_as_float(w4[e] << 16);
                    v[8 * q + 2 * e + 1] += __uint_as_float(w4[e] & 0xffff0000u);
                  }
                }
              }
#pragma unroll
              for (int q = 0; q < 4; q++) {
                uint4 o;
                o.x = pack2(v[8 * q], v[8 * q + 1]); o.y = pack2(v[8 * q + 2], v[8 * q + 3]);
                o.z = pack2(v[8 * q + 4], v[8 * q + 5]); o.w = pack2(v[8 * q + 6], v[8 * q + 7]);
                d4[q] = o;
              }
            }
          }
          continue;
        }
        // registers (row = lane, 32 columns) -> shared (padded) -> rows of 32 consecutive columns
#pragma unroll
        for (int j = 0; j < 32; j++) st[lane * 33 + j] = __uint_as_float(r[j]);
        __syncwarp();
        const int n = nc0 + lane;
        const bool n_ok = n < N;
        const float cs = (colscale && n_ok) ? colscale[n] : 1.0f;
        const float cb = (colbias && n_ok) ? colbias[n] : 0.0f;
        if (accumulate) {
          // all 32 reads of the old values are in flight before the first add
          float old[32];
#pragma unroll
          for (int rr = 0; rr < 32; rr++) {
            const int m = mrow0 + rr;
            old[rr] = (m < M && n_ok) ? to_f32(out[(size_t)m * ldo + n]) : 0.f;
          }
#pragma unroll
          for (int rr = 0; rr < 32; rr++) {
            const int m = mrow0 + rr;
            if (m < M && n_ok) out[(size_t)m * ldo + n] = from_f32<TO>(st[rr * 33 + lane] * cs + cb + old[rr]);
          }
        } else {
#pragma unroll 8
          for (int rr = 0; rr < 32; rr++) {
            const int m = mrow0 + rr;
            if (m < M && n_ok) out[(size_t)m * ldo + n] = from_f32<TO>(st[rr * 33 + lane] * cs + cb);
          }
        }
        __syncwarp();
      }
      // hand the accumulator half back to the MMA issuer (with splits that happened above)
      if (!split) {
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        if (lane == 0) {
          if constexpr (PAIR) mbar_arrive_cluster(cluster_address(acc_empty0 + 8 * as, 0));   // the issuer's block
          else asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(acc_empty0 + 8 * as) : "memory");
        }
      }
    }
    // bulk copies out of the staging tile: shared memory stays until they have read it
    if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  if constexpr (PAIR) {
    cluster_sync();                                    // neither block's memories are in use by the other any more
    if (warp == 1) asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(2 * BN) : "memory");
  } else {
    __syncthreads();
    if (warp == 1) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(2 * BN) : "memory");
  }
}

// ---- host side ---------------------------------------------------------------------------
typedef CUresult (*EncodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiled g_encode = nullptr;
int g_sms = 148;
ErrWords* g_err_dev = nullptr;   // device memory: the flag kernels read + where its host-visible copy lives
int* g_err_host = nullptr;       // host-mapped word, written by a kernel on failure only
std::mutex g_mu;
// Scratch of the products that share a tile's K-steps among blocks: one slot per stream.  Launches of one
// stream are ordered (a kernel touches the scratch only after its wait on its predecessor), so they share a
// slot; launches of different streams (two mixers' output projections side by side, two models) never do.
// A stream beyond the SPLIT_SLOTS-th runs its products without sharing K-steps (a framework's stream pool has
// a few dozen streams, and every captured graph is recorded on one of them).
constexpr int SPLIT_SLOTS = 40;
constexpr size_t SPLIT_SLOT_BYTES = (size_t)8 << 20;       // partial sums of one launch: splits x M x N floats
constexpr int SPLIT_SLOT_COUNTERS = 4096;                   // 4 per output tile
float* g_part = nullptr;
unsigned* g_part_arrivals = nullptr;                        // zero between launches
std::unordered_map<cudaStream_t, int> g_split_slot_of;      // guarded by g_mu
int g_split_override = 0;                                   // test hook: 0 = choose; n = that many splits (1 = none)

struct MapKey {
  const void* p; int rows, k, ld, box_rows;
  bool operator==(const MapKey& o) const { return p == o.p && rows == o.rows && k == o.k && ld == o.ld && box_rows == o.box_rows; }
};
struct MapHash {
  size_t operator()(const MapKey& k) const {
    size_t h = (size_t)k.p;
    for (int v : {k.rows, k.k, k.ld, k.box_rows}) h = h * 1000003u ^ (size_t)v;
    return h;
  }
};
std::unordered_map<MapKey, CUtensorMap, MapHash> g_maps;

int g_pairs = 0;                                            // pairs of blocks the GPU runs at once (0: none)
constexpr int PAIR_BN = 256, PAIR_STAGES = 6;               // the pair's tile is 256 x 256; a stage is 32 KB a block

template <typename TO, int BN, int STAGES, bool SWIGLU = false, bool PAIR = false>
int configure() {
  if (cudaFuncSetAttribute(gemm_tcgen05_kernel<TO, BN, STAGES, SWIGLU, PAIR>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                           Smem<BN, STAGES, PAIR>::TOTAL) != cudaSuccess)
    return tlc_fail(-2, "linear: cannot reserve %d bytes of shared memory", Smem<BN, STAGES, PAIR>::TOTAL);
  return 0;
}

// How many clusters of two blocks of the pair kernel fit on the GPU at once.
int count_pairs() {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * g_sms);
  cfg.blockDim = dim3(THREADS);
  cfg.dynamicSmemBytes = Smem<PAIR_BN, PAIR_STAGES, true>::TOTAL;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  int n = 0;
  if (cudaOccupancyMaxActiveClusters(&n, gemm_tcgen05_kernel<__nv_bfloat16, PAIR_BN, PAIR_STAGES, false, true>, &cfg) != cudaSuccess) {
    cudaGetLastError();
    return 0;
  }
  return n;
}

int init_once() {
  std::lock_guard<std::mutex> lk(g_mu);
  if (g_encode) return 0;
  if (int rc = configure<float, 128, 6>()) return rc;
  if (int rc = configure<__nv_bfloat16, 128, 6>()) return rc;
  if (int rc = configure<float, 256, 4>()) return rc;
  if (int rc = configure<__nv_bfloat16, 256, 4>()) return rc;
  if (int rc = configure<float, 64, 8>()) return rc;
  if (int rc = configure<__nv_bfloat16, 64, 8>()) return rc;
  if (int rc = configure<float, 64, 8, true>()) return rc;
  if (int rc = configure<__nv_bfloat16, 64, 8, true>()) return rc;
  if (int rc = configure<float, 128, 6, true>()) return rc;
  if (int rc = configure<__nv_bfloat16, 128, 6, true>()) return rc;
  if (int rc = configure<float, 256, 4, true>()) return rc;
  if (int rc = configure<__nv_bfloat16, 256, 4, true>()) return rc;
  if (int rc = configure<float, PAIR_BN, PAIR_STAGES, false, true>()) return rc;
  if (int rc = configure<__nv_bfloat16, PAIR_BN, PAIR_STAGES, false, true>()) return rc;
  if (int rc = configure<float, PAIR_BN, PAIR_STAGES, true, true>()) return rc;
  if (int rc = configure<__nv_bfloat16, PAIR_BN, PAIR_STAGES, true, true>()) return rc;
  int dev = 0;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&g_sms, cudaDevAttrMultiProcessorCount, dev);
  if (g_sms <= 0) g_sms = 148;
  g_pairs = count_pairs();
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) != cudaSuccess || !fn)
    return tlc_fail(-3, "linear: the CUDA driver does not export cuTensorMapEncodeTiled");
  int* host_dev_view = nullptr;
  if (cudaHostAlloc((void**)&g_err_host, sizeof(int), cudaHostAllocMapped) != cudaSuccess ||
      cudaHostGetDevicePointer((void**)&host_dev_view, g_err_host, 0) != cudaSuccess ||
      cudaMalloc((void**)&g_err_dev, sizeof(ErrWords)) != cudaSuccess)
    return tlc_fail(-3, "linear: cannot allocate the error words");
  if (cudaMalloc((void**)&g_part, SPLIT_SLOTS * SPLIT_SLOT_BYTES) != cudaSuccess ||
      cudaMalloc((void**)&g_part_arrivals, SPLIT_SLOTS * SPLIT_SLOT_COUNTERS * sizeof(unsigned)) != cudaSuccess ||
      cudaMemset(g_part_arrivals, 0, SPLIT_SLOTS * SPLIT_SLOT_COUNTERS * sizeof(unsigned)) != cudaSuccess)
    return tlc_fail(-3, "linear: cannot allocate the scratch of split products");
  *g_err_host = 0;
  ErrWords init{0, host_dev_view, TLC_WAIT_LIMIT_CYCLES};
  if (cudaMemcpy(g_err_dev, &init, sizeof(init), cudaMemcpyHostToDevice) != cudaSuccess)
    return tlc_fail(-3, "linear: cannot initialise the error words");
  g_encode = (EncodeTiled)fn;
  return 0;
}

int get_map(const void* p, int rows, int k, int ld, int box_rows, CUtensorMap* out) {
  MapKey key{p, rows, k, ld, box_rows};
  std::lock_guard<std::mutex> lk(g_mu);
  auto it = g_maps.find(key);
  if (it != g_maps.end()) { *out = it->second; return 0; }
  cuuint64_t dims[2] = {(cuuint64_t)k, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
  cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUtensorMap m;
  CUresult r = g_encode(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(p), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return tlc_fail(-3, "linear: cuTensorMapEncodeTiled failed with %d (rows %d, k %d, ld %d)", (int)r, rows, k, ld);
  if (g_maps.size() > 4096) g_maps.clear();
  g_maps[key] = m;
  *out = m;
  return 0;
}

// The output as the copy engine sees it: 32-bit values, [M, N] with ldo between rows, boxes of 32 x 32 with the
// 128-byte swizzle.  *ok = 0 where the output cannot go that way (its rows do not start and end on 16-byte
// boundaries, or the test hook is off); *out is then some valid map that the kernel does not use.
int g_tma_out = 1;
int get_out_map(const void* p, int M, int N, int ldo, const CUtensorMap& dummy, CUtensorMap* out, int* ok) {
  *out = dummy;
  *ok = 0;
  // the engine clips at the matrix's edge in pieces of 16 bytes: a row of N values must end on one
  if (!g_tma_out || ((uintptr_t)p & 15) != 0 || (ldo & 3) != 0 || (N & 3) != 0) return 0;
  MapKey key{p, M, N, ldo, -32};
  std::lock_guard<std::mutex> lk(g_mu);
  auto it = g_maps.find(key);
  if (it != g_maps.end()) { *out = it->second; *ok = 1; return 0; }
  cuuint64_t dims[2] = {(cuuint64_t)N, (cuuint64_t)M};
  cuuint64_t strides[1] = {(cuuint64_t)ldo * 4};
  cuuint32_t box[2] = {32, 32};
  cuuint32_t estr[2] = {1, 1};
  CUtensorMap m;
  CUresult r = g_encode(&m, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<void*>(p), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return tlc_fail(-3, "linear: cuTensorMapEncodeTiled failed with %d for the output (M %d, N %d, ldo %d)", (int)r, M, N, ldo);
  if (g_maps.size() > 4096) g_maps.clear();
  g_maps[key] = m;
  *out = m;
  *ok = 1;
  return 0;
}

}  // namespace

// A tensor map of a row-major bfloat16 matrix [rows, cols] with `ld` elements between rows, for boxes of
// box_rows x box_cols elements with the 128-byte swizzle (box_cols = 64).  Not cached: for buffers that live
// for one call.
int tlc_tensor_map_bf16(const void* p, long long rows, long long cols, long long ld, int box_cols, int box_rows,
                        CUtensorMap* out) {
  if (int rc = init_once()) return rc;
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
  cuuint32_t box[2] = {(cuuint32_t)box_cols, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = g_encode(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(p), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    return tlc_fail(-3, "cuTensorMapEncodeTiled failed with %d (rows %lld, cols %lld, ld %lld, box %d x %d)", (int)r, rows, cols,
                    ld, box_rows, box_cols);
  return 0;
}

namespace {

// How many blocks share the K-steps of a tile: more than one when the output has one row of tiles and too few
// of them to occupy the GPU (a batch of 33..128 rows times a narrow matrix) and K is long: a split costs a
// round trip through scratch and an arrival counter, about 5 us, so every split keeps at least 32 K-steps
// (64 x 3072 x 12288: 62 us in one piece, 34 us in three; 64 x 2048 x 4096: 23 us, and 18 us in four, but
// 12 us with the weight-streaming kernel).
int pick_splits(int M, int N, int K, int bn) {
  if (M > BM) return 1;
  const int tiles = (N + bn - 1) / bn, num_k = (K + BK - 1) / BK;
  int s = g_split_override ? g_split_override : (tiles * 2 > g_sms ? 1 : std::min(std::min(g_sms / tiles, num_k / 32), 16));
  s = std::min(s, num_k);
  while (s > 1 && ((size_t)s * M * N * sizeof(float) > SPLIT_SLOT_BYTES || (s - 1) * ((num_k + s - 1) / s) >= num_k)) s--;
  if (tiles * 4 > SPLIT_SLOT_COUNTERS) s = 1;
  return std::max(s, 1);
}

template <typename TO, int BN, int STAGES, bool SWIGLU = false>
int launch(const CUtensorMap& ma, const CUtensorMap& mb, void* out, int ldo, const float* colscale, const float* colbias,
           int accumulate, int M, int N, int K, cudaStream_t stream) {
  using S = Smem<BN, STAGES>;
  auto kern = gemm_tcgen05_kernel<TO, BN, STAGES, SWIGLU, false>;
  int splits = SWIGLU ? 1 : pick_splits(M, N, K, BN);
  int slot = 0;
  if (splits > 1) {
    std::lock_guard<std::mutex> lk(g_mu);
    auto it = g_split_slot_of.find(stream);
    if (it != g_split_slot_of.end()) slot = it->second;
    else if ((int)g_split_slot_of.size() < SPLIT_SLOTS) slot = g_split_slot_of[stream] = (int)g_split_slot_of.size();
    else splits = 1;
  }
  const int tiles = ((N + BN - 1) / BN) * ((M + BM - 1) / BM) * splits;
  float* part = g_part + slot * (SPLIT_SLOT_BYTES / sizeof(float));
  unsigned* arrivals = g_part_arrivals + slot * SPLIT_SLOT_COUNTERS;
  dim3 grid(tiles < g_sms ? tiles : g_sms);
  CUtensorMap mo = ma;
  int tma_out = 0;
  if (std::is_same<TO, float>::value && !SWIGLU && splits == 1)
    if (int rc = get_out_map(out, M, N, ldo, ma, &mo, &tma_out)) return rc;
  tlc_launch(kern, dim3(grid), dim3(THREADS), S::TOTAL, stream, ma, mb, (TO*)out, ldo, colscale, colbias, accumulate, M, N, K, g_err_dev,
             splits, part, arrivals, mo, tma_out);
  TLC_CHECK_LAUNCH("linear(tcgen05)");
  return 0;
}

// Pairs of blocks on tiles of 256 x 256: a cluster of two per tile, as many pairs as the GPU runs at once.
template <typename TO, bool SWIGLU = false>
int launch_pairs(const CUtensorMap& ma, const CUtensorMap& mb, void* out, int ldo, const float* colscale, const float* colbias,
                 int accumulate, int M, int N, int K, cudaStream_t stream) {
  using S = Smem<PAIR_BN, PAIR_STAGES, true>;
  const int tiles = ((N + PAIR_BN - 1) / PAIR_BN) * ((M + 2 * BM - 1) / (2 * BM));
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * std::min(tiles, g_pairs));
  cfg.blockDim = dim3(THREADS);
  cfg.dynamicSmemBytes = S::TOTAL;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = g_tlc_pdl ? 2 : 1;
  CUtensorMap mo = ma;
  int tma_out = 0;
  if (std::is_same<TO, float>::value && !SWIGLU)
    if (int rc = get_out_map(out, M, N, ldo, ma, &mo, &tma_out)) return rc;
  cudaLaunchKernelEx(&cfg, gemm_tcgen05_kernel<TO, PAIR_BN, PAIR_STAGES, SWIGLU, true>, ma, mb, (TO*)out, ldo, colscale, colbias,
                     accumulate, M, N, K, g_err_dev, 1, (float*)nullptr, (unsigned*)nullptr, mo, tma_out);
  TLC_CHECK_LAUNCH("linear(tcgen05, pairs)");
  return 0;
}

}  // namespace

// Error word of the tensor-core kernels: 0, or which bounded wait ran out
// (1 loader, 2 MMA issuer, 3 epilogue, 4 drain).  Reading it does not synchronise.
ErrWords* tlc_error_words() { return g_err_dev; }

extern "C" int tlc_linear_error() { return g_err_host ? *(volatile int*)g_err_host : 0; }
extern "C" void tlc_linear_error_clear() {
  if (g_err_host) *g_err_host = 0;
  if (g_err_dev) cudaMemset(&g_err_dev->flag, 0, sizeof(int));
}

// Prepares everything that must not happen inside a stream capture (driver entry point, the
// error word, shared-memory attributes).  Called once when the library is loaded.
extern "C" int tlc_linear_init() { return init_once(); }

// Test hook: 0 = choose the tile width from the sizes; 64, 128 or 256 = force it.
static int g_tile_override = 0;
extern "C" void tlc_linear_tile_override(int bn) { g_tile_override = bn; }
// Test hook: 0 = choose how many blocks share a tile's K-steps; n = that many where the sizes allow (1 = none).
extern "C" void tlc_linear_split_override(int n) { g_split_override = n; }

// Width of the output tile (rows are always 128).  A block works through ceil(tiles / SMs) tiles one after the
// other, and a tile's time grows with its width, though less than in proportion: per output column a tile of
// 256 moves the least shared memory per flop, one of 128 about 1.45 times and one of 64 about twice as much
// (measured on 2048 x 2048 x 4096: 35 us with 128 tiles of 256 columns, 51 us with 256 tiles of 128).
static int pick_tile(int M, int N) {
  if (g_tile_override) return g_tile_override;
  const long long m_tiles = (M + BM - 1) / BM;
  const int widths[3] = {256, 128, 64};
  const double per_column[3] = {1.0, 1.45, 2.0};
  double best = 0;
  int bn = 128;
  for (int i = 0; i < 3; i++) {
    const long long tiles = m_tiles * ((N + widths[i] - 1) / widths[i]);
    const long long rounds = (tiles + g_sms - 1) / g_sms;
    const double cost = (double)rounds * widths[i] * per_column[i];
    if (i == 0 || cost < best) { best = cost; bn = widths[i]; }
  }
  return bn;
}

// Test hook: 0 = 32-bit outputs never leave through the copy engine (bulk tensor stores and adds).
extern "C" void tlc_linear_tma_out(int on) { g_tma_out = on; }

// Test hook: 0 = pairs of blocks where they pay, 1 = never, 2 = wherever the GPU can run them.
static int g_pair_override = 0;
extern "C" void tlc_linear_pair_override(int mode) { g_pair_override = mode; }
// How many pairs of blocks the GPU runs at once (0: it cannot, and every product runs on single blocks).
extern "C" int tlc_linear_pairs() { return init_once() ? 0 : g_pairs; }

// Pairs of blocks on 256 x 256 tiles: when there are more than 128 rows and single blocks would take tiles
// of 256 columns anyway (wide outputs, many rows).
static bool pick_pairs(int M, int N) {
  if (g_pairs <= 0 || g_pair_override == 1) return false;
  if (g_pair_override == 2) return true;
  return M > BM && !g_tile_override && pick_tile(M, N) == 256;
}

extern "C" int tlc_linear_tcgen05_ok(int a_dtype, int lda, const void* a, int w_dtype, int ldw, const void* w, int K) {
  return a_dtype == TLC_BF16 && w_dtype == TLC_BF16 && K % 8 == 0 && lda % 8 == 0 && ldw % 8 == 0 &&
         ((uintptr_t)a % 16 == 0) && ((uintptr_t)w % 16 == 0);
}

// The fused feed-forward front: out[M, N/2] = silu(gate) * up, where the rows of w come in groups of
// 16 (8 gate rows, then their 8 up rows) and gate/up = (a w^T) * colscale + colbias.  Returns 1 if no
// kernel takes these operands (the caller then runs the product and the activation separately).
extern "C" int tlc_linear_swiglu(const void* a, int a_dtype, int lda, const void* w, int w_dtype, int ldw, void* out,
                                 int out_dtype, int ldo, const float* colscale, const float* colbias, int M, int N, int K,
                                 int min_rows_for_tensor_cores, cudaStream_t stream) {
  if (M == 0 || N == 0) return 0;
  if (N % 16 != 0 || !tlc_linear_tcgen05_ok(a_dtype, lda, a, w_dtype, ldw, w, K)) return 1;
  TLC_REQUIRE(K > 0 && lda >= K && ldw >= K && ldo >= N / 2, "linear: bad sizes M=%d N=%d K=%d lda=%d ldw=%d ldo=%d", M, N, K,
              lda, ldw, ldo);
  if (out_dtype != TLC_F32 && out_dtype != TLC_BF16) return tlc_fail(-1, "linear: unknown output dtype %d", out_dtype);
  if (min_rows_for_tensor_cores <= 128 && tlc_linear_few_rows_ok(a_dtype, lda, a, w_dtype, ldw, w, M, N, K)) {
    if (int rc = init_once()) return rc;
    return tlc_linear_few_rows_swiglu(a, lda, w, ldw, out, out_dtype, ldo, colscale, colbias, M, N, K, stream);
  }
  if (M <= 32 && tlc_linear_skinny_ok(a_dtype, lda, a, w_dtype, ldw, w, M, K))
    return tlc_linear_skinny_swiglu(a, lda, w, ldw, out, out_dtype, ldo, colscale, colbias, M, N, K, stream);
  if (M < min_rows_for_tensor_cores) return 1;
  if (int rc = init_once()) return rc;
  CUtensorMap ma, mb;
  if (int rc = get_map(a, M, K, lda, BM, &ma)) return rc;
  if (pick_pairs(M, N)) {
    if (int rc = get_map(w, N, K, ldw, PAIR_BN / 2, &mb)) return rc;
    return out_dtype == TLC_F32 ? launch_pairs<float, true>(ma, mb, out, ldo, colscale, colbias, 0, M, N, K, stream)
                                : launch_pairs<__nv_bfloat16, true>(ma, mb, out, ldo, colscale, colbias, 0, M, N, K, stream);
  }
  const int bn = pick_tile(M, N);
  if (bn == 256) {
    if (int rc = get_map(w, N, K, ldw, 256, &mb)) return rc;
    return out_dtype == TLC_F32 ? launch<float, 256, 4, true>(ma, mb, out, ldo, colscale, colbias, 0, M, N, K, stream)
                                : launch<__nv_bfloat16, 256, 4, true>(ma, mb, out, ldo, colscale, colbias, 0, M, N, K, stream);
  }
  if (bn == 64) {
    if (int rc = get_map(w, N, K, ldw, 64, &mb)) return rc;
    return out_dtype == TLC_F32 ? launch<float, 64, 8, true>(ma, mb, out, ldo, colscale, colbias, 0, M, N, K, stream)
                                : launch<__nv_bfloat16, 64, 8, true>(ma, mb, out, ldo, colscale, colbias, 0, M, N, K, stream);
  }
  if (int rc = get_map(w, N, K, ldw, 128, &mb)) return rc;
  return out_dtype == TLC_F32 ? launch<float, 128, 6, true>(ma, mb, out, ldo, colscale, colbias, 0, M, N, K, stream)
                              : launch<__nv_bfloat16, 128, 6, true>(ma, mb, out, ldo, colscale, colbias, 0, M, N, K, stream);
}

extern "C" int tlc_linear(const void* a, int a_dtype, int lda, const void* w, int w_dtype, int ldw, void* out,
                          int out_dtype, int ldo, const float* colscale, const float* colbias, int accumulate, int M,
                          int N, int K, int min_rows_for_tensor_cores, cudaStream_t stream) {
  if (M == 0 || N == 0) return 0;
  // Up to 32 rows the weight-streaming kernel is always best.  From 33 to 64 rows it re-reads the
  // activations once per 16 output columns, which only pays while the tiled kernel would have too
  // few tiles to keep the GPU busy (narrow outputs) and too few K-steps to share among blocks.
  // (a threshold above 128 rows keeps every tensor-core kernel out, this one too)
  if (min_rows_for_tensor_cores <= 128 && (out_dtype == TLC_F32 || out_dtype == TLC_BF16) &&
      tlc_linear_few_rows_ok(a_dtype, lda, a, w_dtype, ldw, w, M, N, K)) {
    TLC_REQUIRE(K > 0 && lda >= K && ldw >= K && ldo >= N, "linear: bad sizes M=%d N=%d K=%d lda=%d ldw=%d ldo=%d", M, N, K,
                lda, ldw, ldo);
    if (int rc = init_once()) return rc;
    return tlc_linear_few_rows_run(a, lda, w, ldw, out, out_dtype, ldo, colscale, colbias, accumulate, M, N, K, stream);
  }
  const bool tiled_ok = M >= min_rows_for_tensor_cores && tlc_linear_tcgen05_ok(a_dtype, lda, a, w_dtype, ldw, w, K);
  const bool narrow = N <= 3072 && K < 8192;
  if (tlc_linear_skinny_ok(a_dtype, lda, a, w_dtype, ldw, w, M, K) && (M <= 32 || narrow || !tiled_ok)) {
    TLC_REQUIRE(K > 0 && lda >= K && ldw >= K && ldo >= N, "linear: bad sizes M=%d N=%d K=%d lda=%d ldw=%d ldo=%d", M, N,
                K, lda, ldw, ldo);
    return tlc_linear_skinny(a, lda, w, ldw, out, out_dtype, ldo, colscale, colbias, accumulate, M, N, K, stream);
  }
  if (!tiled_ok)
    return tlc_linear_simt(a, a_dtype, lda, w, w_dtype, ldw, out, out_dtype, ldo, colscale, colbias, accumulate, M, N, K,
                           stream);
  TLC_REQUIRE(K > 0 && lda >= K && ldw >= K && ldo >= N, "linear: bad sizes M=%d N=%d K=%d lda=%d ldw=%d ldo=%d", M, N, K,
              lda, ldw, ldo);
  if (int rc = init_once()) return rc;
  CUtensorMap ma, mb;
  if (out_dtype != TLC_F32 && out_dtype != TLC_BF16) return tlc_fail(-1, "linear: unknown output dtype %d", out_dtype);
  if (int rc = get_map(a, M, K, lda, BM, &ma)) return rc;
  if (pick_pairs(M, N)) {
    if (int rc = get_map(w, N, K, ldw, PAIR_BN / 2, &mb)) return rc;
    return out_dtype == TLC_F32 ? launch_pairs<float>(ma, mb, out, ldo, colscale, colbias, accumulate, M, N, K, stream)
                                : launch_pairs<__nv_bfloat16>(ma, mb, out, ldo, colscale, colbias, accumulate, M, N, K, stream);
  }
  const int bn = pick_tile(M, N);
  if (bn == 256) {
    if (int rc = get_map(w, N, K, ldw, 256, &mb)) return rc;
    return out_dtype == TLC_F32 ? launch<float, 256, 4>(ma, mb, out, ldo, colscale, colbias, accumulate, M, N, K, stream)
                                : launch<__nv_bfloat16, 256, 4>(ma, mb, out, ldo, colscale, colbias, accumulate, M, N, K, stream);
  }
  if (bn == 64) {
    if (int rc = get_map(w, N, K, ldw, 64, &mb)) return rc;
    return out_dtype == TLC_F32 ? launch<float, 64, 8>(ma, mb, out, ldo, colscale, colbias, accumulate, M, N, K, stream)
                                : launch<__nv_bfloat16, 64, 8>(ma, mb, out, ldo, colscale, colbias, accumulate, M, N, K, stream);
  }
  if (int rc = get_map(w, N, K, ldw, 128, &mb)) return rc;
  return out_dtype == TLC_F32 ? launch<float, 128, 6>(ma, mb, out, ldo, colscale, colbias, accumulate, M, N, K, stream)
                              : launch<__nv_bfloat16, 128, 6>(ma, mb, out, ldo, colscale, colbias, accumulate, M, N, K, stream);
}
