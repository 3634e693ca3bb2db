// bfloat16 linear layer for 17..128 rows (decode steps of that many sequences, short prompts) on the 5th-generation tensor cores,
// with the WEIGHTS on the M side of tcgen05.mma:  out[M, N] (+)= (A[M, K] @ W[N, K]^T) * colscale + colbias.
//
// With so few rows the time is the time to stream the weights once.  The product for prompts puts the activations
// on the 128-row side and pads them, and has too few tiles for the GPU where N is small; the weight-streaming
// mma.sync kernel of the smallest batches re-reads the activations for every 16 output columns.  Here a tile is
// 128 weight rows x 32, 64 or 128 activation rows: D[n, m] = sum_k W[n, k] A[m, k], an accumulator of 128 lanes x NB
// columns of tensor memory.  Weight tiles [128, 64] and activation tiles [NB, 64] arrive by TMA (128-byte
// swizzle, rows past the matrices read as zero) in a ring of shared-memory stages; one thread issues the
// products; four warps take the result out of tensor memory, a thread per weight row.
//
// N / 128 tiles do not fill 148 SMs (65 for N = 8240, 16 for N = 2048), so the K-steps of a tile are shared
// among the 2, 4 or 8 blocks of a thread-block CLUSTER: every block leaves its partial sums [NB, 128] in its own
// shared memory, the cluster meets at a barrier, and block r adds up rows r * NB / split ... of all blocks'
// sums, read through distributed shared memory in the order of the ranks (so the result does not depend on
// timing), applies the epilogue and stores.  A second barrier keeps every block's shared memory alive until
// all have read it.  With SWIGLU the weight rows come in groups of 16 = 8 gate rows and their 8 up rows, and the
// block writes silu(gate) * up ([M, N / 2]).
//
// Every mbarrier wait is bounded (codes 31-33 of the error word); a block whose wait ran out still goes to both
// cluster barriers, so that no block of its cluster waits for it.
#include "common.cuh"
#include "mbarrier.cuh"
#include "tcgen05.cuh"
#include <algorithm>

namespace {

constexpr int WM = 128;                 // weight rows of a tile
constexpr int FBK = 64;                 // K of a stage
constexpr int FR_THREADS = 192;         // loader warp, issuer warp, four epilogue warps

template <int NB, int STAGES>
struct FrSmem {
  static constexpr int W_BYTES = WM * FBK * 2;
  static constexpr int X_BYTES = NB * FBK * 2;
  static constexpr int TILES = STAGES * (W_BYTES + X_BYTES);
  static constexpr int PART = NB * WM * 4;                  // the block's sums [NB][128], in the stages' memory once the products are done
  static constexpr int N_BARS = 2 * STAGES + 1;             // full, empty per stage; accumulator complete
  static constexpr int TOTAL = TILES + N_BARS * 8 + 16 + 1024;
  static_assert(PART <= TILES, "the partial sums reuse the stages");
};

// The same shared-memory word in the block of another rank of the cluster, as a generic address: loads through
// it are ordinary loads, which the compiler may have many of in flight (a volatile asm load a value made the sum
// a chain of round trips: 10 us for 32 rows of two blocks).
__device__ __forceinline__ const float* in_rank(const float* p, int rank) {
  unsigned long long q;
  asm("mapa.u64 %0, %1, %2;" : "=l"(q) : "l"((unsigned long long)(uintptr_t)p), "r"(rank));
  return reinterpret_cast<const float*>((uintptr_t)q);
}

template <typename TO, int NB, int STAGES, bool SWIGLU>
__global__ void __launch_bounds__(FR_THREADS, 2)
gemm_few_rows_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                     TO* __restrict__ out, int ldo, const float* __restrict__ colscale,
                     const float* __restrict__ colbias, int accumulate, int M, int N, int K, int split, ErrWords* err) {
  asm volatile("griddepcontrol.launch_dependents;");
  using S = FrSmem<NB, STAGES>;
  extern __shared__ uint8_t fr_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)fr_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* w_tiles = smem;
  uint8_t* x_tiles = smem + STAGES * S::W_BYTES;
  float* part = reinterpret_cast<float*>(smem);
  uint64_t* bars = (uint64_t*)(smem + S::TILES);
  uint32_t* tmem_slot = (uint32_t*)(bars + S::N_BARS);
  const uint32_t full0 = smem_u32(bars), empty0 = smem_u32(bars + STAGES), acc_full = smem_u32(bars + 2 * STAGES);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long wait_limit = mbar_wait_limit(err);
  const int rank = split > 1 ? (int)cluster_rank() : 0;     // clusters are runs of `split` consecutive blocks
  const int n0 = ((int)blockIdx.x / split) * WM;
  const int num_k = (K + FBK - 1) / FBK, k_per = (num_k + split - 1) / split;
  const int k_begin = min(num_k, rank * k_per), k_end = min(num_k, k_begin + k_per);
  const int n_k = k_end - k_begin;                          // this block's K-steps (the last ranks may have none)

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; s++) { mbar_init(full0 + 8 * s, 1); mbar_init(empty0 + 8 * s, 1); }
    mbar_init(acc_full, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(NB) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {                                        // ---- TMA loader ----
      // the weights do not depend on the previous kernel of the stream: the first stages' weight tiles are on
      // their way before the wait on it, the activation tiles follow after it
      bool ok = true, waited = false;
      int issued = 0;
      for (int i = 0; i < n_k && ok; i++) {
        const int s = i % STAGES, k = k_begin + i;
        if (i >= STAGES) ok = mbar_wait(empty0 + 8 * s, (uint32_t)(((i - STAGES) / STAGES) & 1), err, 31, wait_limit);
        if (!ok) break;
        if (!waited && i == min(n_k, STAGES) - 1) {
          // last of the first fills: wait, then hand in the activation tiles of all of them
          mbar_expect_tx(full0 + 8 * s, S::W_BYTES + S::X_BYTES);
          tma_load_2d(smem_u32(w_tiles + s * S::W_BYTES), &map_w, full0 + 8 * s, k * FBK, n0);
          asm volatile("griddepcontrol.wait;" ::: "memory");
          waited = true;
          for (int j = 0; j <= i; j++)
            tma_load_2d(smem_u32(x_tiles + (j % STAGES) * S::X_BYTES), &map_x, full0 + 8 * (j % STAGES), (k_begin + j) * FBK, 0);
        } else if (!waited) {
          mbar_expect_tx(full0 + 8 * s, S::W_BYTES + S::X_BYTES);
          tma_load_2d(smem_u32(w_tiles + s * S::W_BYTES), &map_w, full0 + 8 * s, k * FBK, n0);
        } else {
          mbar_expect_tx(full0 + 8 * s, S::W_BYTES + S::X_BYTES);
          tma_load_2d(smem_u32(w_tiles + s * S::W_BYTES), &map_w, full0 + 8 * s, k * FBK, n0);
          tma_load_2d(smem_u32(x_tiles + s * S::X_BYTES), &map_x, full0 + 8 * s, k * FBK, 0);
        }
        issued = i + 1;
      }
      if (!waited) asm volatile("griddepcontrol.wait;" ::: "memory");
      if (!ok || *(volatile int*)&err->flag != 0) {
        // something went wrong: let the copies still in flight land before the block goes on to its end
        for (int i = max(0, issued - STAGES); i < issued; i++)
          mbar_wait(full0 + 8 * (i % STAGES), (uint32_t)((i / STAGES) & 1), err, 34, wait_limit);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {                                        // ---- MMA issuer ----
      constexpr uint32_t idesc = instr_desc(WM, NB);
      bool ok = true;
      for (int i = 0; i < n_k; i++) {
        const int s = i % STAGES;
        ok = mbar_wait(full0 + 8 * s, (uint32_t)((i / STAGES) & 1), err, 32, wait_limit);
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t w_addr = smem_u32(w_tiles + s * S::W_BYTES), x_addr = smem_u32(x_tiles + s * S::X_BYTES);
#pragma unroll
        for (int kk = 0; kk < FBK / UMMA_K; kk++)
          umma(tmem, smem_desc(w_addr + kk * UMMA_K * 2), smem_desc(x_addr + kk * UMMA_K * 2), idesc, (i > 0 || kk > 0) ? 1u : 0u);
        umma_commit(empty0 + 8 * s);
      }
      if (ok && n_k > 0) umma_commit(acc_full);
      else if (n_k == 0) mbar_arrive(acc_full);             // nothing to wait for: the epilogue takes zeros
    }
  } else {                                                  // ---- epilogue warps 2..5: the block's sums into shared memory ----
    const int quarter = warp & 3;                           // a warp may touch lanes 32 * (warp % 4) .. + 31 only
    const int row = quarter * 32 + lane;                    // weight row of the tile
    asm volatile("griddepcontrol.wait;" ::: "memory");      // `out` may still be read or written by the previous kernel
    mbar_wait(acc_full, 0, err, 33, wait_limit);
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
    for (int c = 0; c < NB / 32; c++) {
      uint32_t r[32];
      tmem_ld32(tmem + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(c * 32), r);
#pragma unroll
      for (int j = 0; j < 32; j++) part[(c * 32 + j) * WM + row] = n_k > 0 ? __uint_as_float(r[j]) : 0.f;
    }
  }
  __syncwarp();                                             // the loader's and the issuer's warps are whole again
  // every block's sums are in its shared memory (the stages are free: every product that read them is complete)
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  if (split > 1) {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
  } else {
    __syncthreads();
  }
  if (warp >= 2) {
    const int row = (warp & 3) * 32 + lane;
    const int rows_per = NB / split;                        // activation rows this block finishes
    const bool second = SWIGLU && (row & 8);                // an up row: its gate row's thread writes the feature
    const int n = n0 + row;
    if (!second && n + (SWIGLU ? 8 : 0) < N) {
      const float cs = colscale ? colscale[n] : 1.0f, cb = colbias ? colbias[n] : 0.0f;
      const float cs2 = (SWIGLU && colscale) ? colscale[n + 8] : 1.0f, cb2 = (SWIGLU && colbias) ? colbias[n + 8] : 0.0f;
      const float* src[8];                                  // the sums of every rank, this thread's weight row
      for (int q = 0; q < 8; q++) src[q] = (q < split ? (split > 1 ? in_rank(part, q) : part) : part) + row;
      constexpr int RB = 4;                                 // rows whose loads are issued together
      for (int m0 = rank * rows_per; m0 < min(M, (rank + 1) * rows_per); m0 += RB) {
        float x[RB][8], x2[RB][8];
#pragma unroll
        for (int i = 0; i < RB; i++)
#pragma unroll
          for (int q = 0; q < 8; q++) {
            const bool in = q < split && m0 + i < M && i < rows_per;
            x[i][q] = in ? src[q][(m0 + i) * WM] : 0.f;
            x2[i][q] = (SWIGLU && in) ? src[q][(m0 + i) * WM + 8] : 0.f;
          }
#pragma unroll
        for (int i = 0; i < RB; i++) {
        const int m = m0 + i;
        if (m >= M || i >= rows_per) break;
        float v = 0.f, v2 = 0.f;
#pragma unroll
        for (int q = 0; q < 8; q++) { v += x[i][q]; v2 += x2[i][q]; }     // in the order of the ranks; absent ranks add zero
        v = v * cs + cb;
        if (SWIGLU) {
          v2 = v2 * cs2 + cb2;
          out[(size_t)m * ldo + (n0 >> 1) + ((row >> 4) << 3) + (row & 7)] = from_f32<TO>(silu_f(v) * v2);
        } else {
          TO* o = out + (size_t)m * ldo + n;
          if (accumulate) v += to_f32(*o);
          *o = from_f32<TO>(v);
        }
        }
      }
    }
  }
  // no block leaves while another may still read its sums
  if (split > 1) {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
  } else {
    __syncthreads();
  }
  if (warp == 1) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(NB) : "memory");
}

int g_few_rows = 1;                     // test hook: 0 = never this kernel
int g_force_split = 0;                  // test hook: blocks per tile (0: chosen)
int g_max_rows = 128;                   // test hook: products of more rows go to the tiles of the prompt product
int g_min_tiles = 0;                    // test hook: outputs of fewer tiles of 128 weight rows stay with the other kernels (0: by the rows)
bool g_configured = false;
int g_max_split[4] = {0, 0, 0, 0};      // [log2 split]: how many clusters of that size run at once (0: that size is not available)

template <typename TO, int NB, int STAGES, bool SWIGLU>
int launch_few(const CUtensorMap& mw, const CUtensorMap& mx, void* out, int ldo, const float* colscale, const float* colbias,
               int accumulate, int M, int N, int K, int split, cudaStream_t stream) {
  using S = FrSmem<NB, STAGES>;
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(gemm_few_rows_kernel<TO, NB, STAGES, SWIGLU>, cudaFuncAttributeMaxDynamicSharedMemorySize, S::TOTAL) != cudaSuccess)
      return tlc_fail(-2, "linear(few rows): cannot reserve %d bytes of shared memory", S::TOTAL);
    attr_set = true;
  }
  const int tiles = (N + WM - 1) / WM;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(tiles * split);
  cfg.blockDim = dim3(FR_THREADS);
  cfg.dynamicSmemBytes = S::TOTAL;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  int na = 0;
  if (split > 1) {
    attr[na].id = cudaLaunchAttributeClusterDimension;
    attr[na].val.clusterDim.x = split;
    attr[na].val.clusterDim.y = 1;
    attr[na].val.clusterDim.z = 1;
    na++;
  }
  if (g_tlc_pdl) {
    attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[na].val.programmaticStreamSerializationAllowed = 1;
    na++;
  }
  cfg.attrs = attr;
  cfg.numAttrs = na;
  cudaLaunchKernelEx(&cfg, gemm_few_rows_kernel<TO, NB, STAGES, SWIGLU>, mw, mx, (TO*)out, ldo, colscale, colbias, accumulate, M, N,
                     K, split, tlc_error_words());
  TLC_CHECK_LAUNCH("linear(few rows)");
  return 0;
}

constexpr int FR_STAGES = 4;

// How many blocks share a tile's K-steps: as many (2, 4, 8) as bring the grid closest to two blocks an SM (what
// fits with four stages) without passing it, each with at least 4 K-steps.
int pick_split(int N, int K, int NB, int sms) {
  const int tiles = (N + WM - 1) / WM, num_k = (K + FBK - 1) / FBK;
  int split = 1;
  while (split < 8 && tiles * split * 2 <= 2 * sms && num_k / (split * 2) >= 4 && NB % (split * 2) == 0) split *= 2;
  return split;
}

template <bool SWIGLU>
int run_few(const void* a, int lda, const void* w, int ldw, void* out, int out_dtype, int ldo, const float* colscale,
            const float* colbias, int accumulate, int M, int N, int K, int force_split, cudaStream_t stream) {
  static int sms = 0;
  if (sms == 0) { int dev = 0; cudaGetDevice(&dev); cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev); }
  const int NB = M <= 32 ? 32 : M <= 64 ? 64 : 128;
  const int split = force_split > 0 ? force_split : pick_split(N, K, NB, sms);
  CUtensorMap mw, mx;
  if (int rc = tlc_tensor_map_bf16(w, N, K, ldw, FBK, WM, &mw)) return rc;
  if (int rc = tlc_tensor_map_bf16(a, M, K, lda, FBK, NB, &mx)) return rc;
  // (with 128 activation rows a stage is 32 KB: three of them, so that two blocks still share an SM)
#define TLC_FEW(TO_, NB_) launch_few<TO_, NB_, (NB_ == 128 ? 3 : FR_STAGES), SWIGLU>(mw, mx, out, ldo, colscale, colbias, accumulate, M, N, K, split, stream)
  if (out_dtype == TLC_F32) return NB == 32 ? TLC_FEW(float, 32) : NB == 64 ? TLC_FEW(float, 64) : TLC_FEW(float, 128);
  if (out_dtype == TLC_BF16) return NB == 32 ? TLC_FEW(__nv_bfloat16, 32) : NB == 64 ? TLC_FEW(__nv_bfloat16, 64) : TLC_FEW(__nv_bfloat16, 128);
#undef TLC_FEW
  return tlc_fail(-1, "linear: unknown output dtype %d", out_dtype);
}

}  // namespace

// Test hooks: whether products of 17..64 rows may take this kernel; a fixed number of blocks per tile (0: chosen).
extern "C" void tlc_linear_few_rows(int on) { g_few_rows = on; }
extern "C" void tlc_linear_few_rows_split(int split) { g_force_split = split; }
extern "C" void tlc_linear_few_rows_min_tiles(int tiles) { g_min_tiles = tiles; }
extern "C" void tlc_linear_few_rows_max_rows(int rows) { g_max_rows = rows; }

// bfloat16 operands with 16-byte aligned rows, 17..64 rows, and an output that is wide enough: from 32 tiles of 128
// weight rows on, from 16 with more than 32 rows.  Measured at 48 and 64 rows, microseconds in a captured loop over
// operand sets larger than the L2: N = 8240, K = 2048: 11.5 against 14.2 for the kernels that run these sizes
// otherwise; N = 8192 with SwiGLU 12.3 against 13.5; N = 2048, K = 4096: 12.0 against 12.0 alone, but inside the
// captured decode step at batch 64 the two products with N = 2048 make 4.08 -> 3.79 ms a step (the
// weight-streaming kernel re-reads 64 rows of activations per 16 columns), at batch 32 and 24 2.40 -> 2.44 and
// 2.13 -> 2.17.  With a forced split (tests) any output of at least one tile qualifies.
extern "C" int tlc_linear_few_rows_ok(int a_dtype, int lda, const void* a, int w_dtype, int ldw, const void* w, int M, int N, int K) {
  // more tiles than two an SM (a vocabulary-sized output: 512 tiles) are better served by the persistent tiles of
  // the product for prompts: 55 us against 62 for 64 x 65,536 x 2,048
  static int sms = 0;
  if (sms == 0) { int dev = 0; cudaGetDevice(&dev); cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev); }
  if (g_force_split == 0 && (N + WM - 1) / WM > 2 * sms) return 0;
  return g_few_rows && a_dtype == TLC_BF16 && w_dtype == TLC_BF16 && M > 16 && M <= g_max_rows && N >= (g_force_split > 0 ? 1 : g_min_tiles > 0 ? g_min_tiles : M > 32 ? 16 : 32) * WM &&
         K % 8 == 0 && lda % 8 == 0 && ldw % 8 == 0 && ((uintptr_t)a % 16 == 0) && ((uintptr_t)w % 16 == 0) &&
         tlc_error_words() != nullptr;
}

int tlc_linear_few_rows_run(const void* a, int lda, const void* w, int ldw, void* out, int out_dtype, int ldo,
                            const float* colscale, const float* colbias, int accumulate, int M, int N, int K,
                            cudaStream_t stream) {
  return run_few<false>(a, lda, w, ldw, out, out_dtype, ldo, colscale, colbias, accumulate, M, N, K, g_force_split, stream);
}

int tlc_linear_few_rows_swiglu(const void* a, int lda, const void* w, int ldw, void* out, int out_dtype, int ldo,
                               const float* colscale, const float* colbias, int M, int N, int K, cudaStream_t stream) {
  return run_few<true>(a, lda, w, ldw, out, out_dtype, ldo, colscale, colbias, 0, M, N, K, g_force_split, stream);
}
