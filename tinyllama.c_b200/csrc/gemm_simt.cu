// Linear layers on the CUDA cores: out[m,n] = (sum_k a[m,k] * w[n,k]) * colscale[n] + colbias[n].
//
// y[r] = sum_c W[r,c] x[c] with W stored [out, in] is the reference's matmul
// (cpu_op.c:121-189 for one row, 253-328 for a batch).  These kernels are the true
// 32-bit path (FFMA, 32-bit accumulation in k order, no tensor cores, no reduced
// matrix mode) and the fall-back for bfloat16 shapes the tensor-core kernel refuses.
// Two shapes: a 64x64 tile kernel for many rows and a warp-per-column kernel for the
// few rows of a decode step, where the weight matrix is streamed once.
#include "common.cuh"

// ---- tiled kernel ---------------------------------------------------------------------
#define BM 64
#define BN 64
#define BK 16

template <typename TA, typename TW, typename TO>
__global__ void __launch_bounds__(256)
gemm_tiled_kernel(const TA* __restrict__ a, int lda, const TW* __restrict__ w, int ldw, TO* __restrict__ out, int ldo,
                  const float* __restrict__ colscale, const float* __restrict__ colbias, int accumulate, int M, int N,
                  int K) {
  tlc_pdl(a, out);
  __shared__ float As[BK][BM + 4];
  __shared__ float Ws[BK][BN + 4];
  const int tid = threadIdx.x;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  const int tm = (tid / 16) * 4, tn = (tid % 16) * 4;
  float acc[4][4] = {};
  // each thread loads 4 elements of each tile: row = tid/4 (0..63), k = (tid%4)*4 .. +3
  const int lr = tid >> 2, lk = (tid & 3) * 4;
  for (int k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
    for (int i = 0; i < 4; i++) {
      const int k = k0 + lk + i;
      const int m = m0 + lr, n = n0 + lr;
      As[lk + i][lr] = (m < M && k < K) ? to_f32(a[(size_t)m * lda + k]) : 0.f;
      Ws[lk + i][lr] = (n < N && k < K) ? to_f32(w[(size_t)n * ldw + k]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < BK; k++) {
      float av[4], wv[4];
#pragma unroll
      for (int i = 0; i < 4; i++) { av[i] = As[k][tm + i]; wv[i] = Ws[k][tn + i]; }
#pragma unroll
      for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) acc[i][j] = fmaf(av[i], wv[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; i++) {
    const int m = m0 + tm + i;
    if (m >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; j++) {
      const int n = n0 + tn + j;
      if (n >= N) continue;
      float v = acc[i][j];
      if (colscale) v *= colscale[n];
      if (colbias) v += colbias[n];
      TO* o = out + (size_t)m * ldo + n;
      if (accumulate) v += to_f32(*o);
      *o = from_f32<TO>(v);
    }
  }
}

// ---- few rows: one warp per output column, the weight row read once ----------------------
template <typename TA, typename TW, typename TO, int MT>
__global__ void __launch_bounds__(256)
gemm_skinny_kernel(const TA* __restrict__ a, int lda, const TW* __restrict__ w, int ldw, TO* __restrict__ out, int ldo,
                   const float* __restrict__ colscale, const float* __restrict__ colbias, int accumulate, int M, int N,
                   int K, int m_base) {
  tlc_pdl(a, out);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n = blockIdx.x * (blockDim.x >> 5) + warp;
  if (n >= N) return;
  const TW* wr = w + (size_t)n * ldw;
  float acc[MT];
#pragma unroll
  for (int m = 0; m < MT; m++) acc[m] = 0.f;
  for (int k = lane; k < K; k += 32) {
    const float wv = to_f32(wr[k]);
#pragma unroll
    for (int m = 0; m < MT; m++)
      if (m_base + m < M) acc[m] = fmaf(to_f32(a[(size_t)(m_base + m) * lda + k]), wv, acc[m]);
  }
#pragma unroll
  for (int m = 0; m < MT; m++) {
    float v = warp_sum(acc[m]);
    if (lane == 0 && m_base + m < M) {
      if (colscale) v *= colscale[n];
      if (colbias) v += colbias[n];
      TO* o = out + (size_t)(m_base + m) * ldo + n;
      if (accumulate) v += to_f32(*o);
      *o = from_f32<TO>(v);
    }
  }
}

// bfloat16 weights and activations, K a multiple of 8 and 16-byte aligned rows: 128-bit loads.
template <typename TO, int MT>
__global__ void __launch_bounds__(256)
gemm_skinny_bf16x8_kernel(const __nv_bfloat16* __restrict__ a, int lda, const __nv_bfloat16* __restrict__ w, int ldw,
                          TO* __restrict__ out, int ldo, const float* __restrict__ colscale,
                          const float* __restrict__ colbias, int accumulate, int M, int N, int K, int m_base) {
  tlc_pdl(a, out);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n = blockIdx.x * (blockDim.x >> 5) + warp;
  if (n >= N) return;
  const uint4* wr = reinterpret_cast<const uint4*>(w + (size_t)n * ldw);
  float acc[MT];
#pragma unroll
  for (int m = 0; m < MT; m++) acc[m] = 0.f;
  const int K8 = K >> 3;
  for (int k8 = lane; k8 < K8; k8 += 32) {
    const uint4 wq = __ldg(wr + k8);
    const __nv_bfloat162* wp = reinterpret_cast<const __nv_bfloat162*>(&wq);
    float wf[8];
#pragma unroll
    for (int i = 0; i < 4; i++) { float2 f = __bfloat1622float2(wp[i]); wf[2 * i] = f.x; wf[2 * i + 1] = f.y; }
#pragma unroll
    for (int m = 0; m < MT; m++) {
      if (m_base + m < M) {
        const uint4 aq = *reinterpret_cast<const uint4*>(a + (size_t)(m_base + m) * lda + (size_t)k8 * 8);
        const __nv_bfloat162* ap = reinterpret_cast<const __nv_bfloat162*>(&aq);
#pragma unroll
        for (int i = 0; i < 4; i++) {
          float2 f = __bfloat1622float2(ap[i]);
          acc[m] = fmaf(f.x, wf[2 * i], acc[m]);
          acc[m] = fmaf(f.y, wf[2 * i + 1], acc[m]);
        }
      }
    }
  }
#pragma unroll
  for (int m = 0; m < MT; m++) {
    float v = warp_sum(acc[m]);
    if (lane == 0 && m_base + m < M) {
      if (colscale) v *= colscale[n];
      if (colbias) v += colbias[n];
      TO* o = out + (size_t)(m_base + m) * ldo + n;
      if (accumulate) v += to_f32(*o);
      *o = from_f32<TO>(v);
    }
  }
}

template <typename TA, typename TW, typename TO>
static int launch_simt(const void* a, int lda, const void* w, int ldw, void* out, int ldo, const float* colscale,
                       const float* colbias, int accumulate, int M, int N, int K, cudaStream_t stream) {
  constexpr int MT = 8;
  if (M <= 16) {
    const bool vec = std::is_same<TA, __nv_bfloat16>::value && std::is_same<TW, __nv_bfloat16>::value && (K % 8 == 0) &&
                     (lda % 8 == 0) && (ldw % 8 == 0) && ((uintptr_t)a % 16 == 0) && ((uintptr_t)w % 16 == 0);
    const unsigned blocks = (unsigned)((N + 7) / 8);
    for (int mb = 0; mb < M; mb += MT) {
      if (vec)
        tlc_launch(gemm_skinny_bf16x8_kernel<TO, MT>, dim3(blocks), dim3(256), 0, stream, 
            (const __nv_bfloat16*)a, lda, (const __nv_bfloat16*)w, ldw, (TO*)out, ldo, colscale, colbias, accumulate, M,
            N, K, mb);
      else
        tlc_launch(gemm_skinny_kernel<TA, TW, TO, MT>, dim3(blocks), dim3(256), 0, stream, (const TA*)a, lda, (const TW*)w, ldw, (TO*)out,
                                                                       ldo, colscale, colbias, accumulate, M, N, K, mb);
    }
  } else {
    dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
    tlc_launch(gemm_tiled_kernel<TA, TW, TO>, dim3(grid), dim3(256), 0, stream, (const TA*)a, lda, (const TW*)w, ldw, (TO*)out, ldo,
                                                            colscale, colbias, accumulate, M, N, K);
  }
  TLC_CHECK_LAUNCH("linear(simt)");
  return 0;
}

extern "C" int tlc_linear_simt(const void* a, int a_dtype, int lda, const void* w, int w_dtype, int ldw, void* out,
                               int out_dtype, int ldo, const float* colscale, const float* colbias, int accumulate,
                               int M, int N, int K, cudaStream_t stream) {
  if (M == 0 || N == 0) return 0;
  TLC_REQUIRE(K > 0 && lda >= K && ldw >= K && ldo >= N, "linear: bad sizes M=%d N=%d K=%d lda=%d ldw=%d ldo=%d", M, N, K,
              lda, ldw, ldo);
  TLC_DISPATCH_DTYPE(a_dtype, TA, TLC_DISPATCH_DTYPE(w_dtype, TW, TLC_DISPATCH_DTYPE(out_dtype, TO,
      return (launch_simt<TA, TW, TO>(a, lda, w, ldw, out, ldo, colscale, colbias, accumulate, M, N, K, stream)))));
  return 0;
}

// ---- few rows, bfloat16, tensor cores as the reducer ----------------------------------------
// A decode step multiplies up to a few dozen rows by every weight matrix; the time is the time
// to stream the weights once.  One block owns 16 output columns (= 16 weight rows); its four
// warps take interleaved 32-wide slices of K.  Each lane reads 16 contiguous bytes of two
// weight rows (g, g+8) and of one activation row per group of 8 rows, and feeds them to
// mma.sync.m16n8k16 with the weight rows as the M side and the activation rows as the N side.
// The contraction index is permuted the same way on both sides (a lane's 8 contiguous values
// serve two instructions), which a dot product does not notice.  Accumulators stay in
// registers; the four warps' partial sums meet in shared memory.
template <int MG> struct SkinnyAcc { float d[MG][2][4]; };

__device__ __forceinline__ void mma_bf16_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                               uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

constexpr int SK_WARPS = 16;          // warps per block, each with its own slices of K
static int g_skinny_pairs = 1;        // 0: never two blocks a tile (for comparisons)

// With SWIGLU a block's 16 weight rows are 8 gate rows followed by their 8 up rows, and the block
// writes silu(gate) * up for its 8 features (out is [M, N/2]).
//
// With PAIR two blocks of a cluster share a tile of 16 columns, each with one half of K: a matrix with few
// rows (N / 16 tiles for 148 SMs that hold two blocks each) and a long K otherwise needs several trips to
// memory on half of the SMs' load slots.  The second block leaves its sums in the first block's shared memory
// (distributed shared memory); the first adds them to its own, always in this order, and stores.
template <typename TO, int MG, int U, bool SWIGLU, bool PAIR>
__global__ void __launch_bounds__(SK_WARPS * 32, ((MG == 1 && U <= 4) || (MG == 2 && U <= 2) || (MG == 4 && U == 1)) ? 2 : 1)
gemm_skinny_mma_kernel(const __nv_bfloat16* __restrict__ a, int lda, const __nv_bfloat16* __restrict__ w, int ldw,
                       TO* __restrict__ out, int ldo, const float* __restrict__ colscale,
                       const float* __restrict__ colbias, int accumulate, int M, int N, int K) {
  static_assert(!(PAIR && SWIGLU), "the paired form has no SwiGLU epilogue");
  // The weights do not depend on the previous kernel of the stream, the activations do: when this
  // kernel is launched early (programmatic dependent launch), the first round of weight loads is
  // in flight while the previous kernel is still finishing; only then does it wait for it.
  asm volatile("griddepcontrol.launch_dependents;");
  __shared__ float red[SK_WARPS][MG < 4 ? MG : 4][32][4];
  __shared__ float other[PAIR ? MG * 128 : 1];                       // the second block's sums, by output value
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int rank = PAIR ? (int)(blockIdx.x & 1) : 0;                 // clusters are pairs of consecutive blocks
  const int n0 = (PAIR ? blockIdx.x >> 1 : blockIdx.x) * 16;
  const int r0 = min(n0 + g, N - 1), r1 = min(n0 + g + 8, N - 1);     // clamped rows are never stored
  const uint4* w0 = reinterpret_cast<const uint4*>(w + (size_t)r0 * ldw);
  const uint4* w1 = reinterpret_cast<const uint4*>(w + (size_t)r1 * ldw);
  float acc[MG][4];
#pragma unroll
  for (int i = 0; i < MG; i++)
#pragma unroll
    for (int j = 0; j < 4; j++) acc[i][j] = 0.f;
  const int K8 = K >> 3;                                             // 16-byte chunks per row
  const int all_steps = (K8 + 3) >> 2;                               // a step is 4 chunks = 32 values of K
  const int half_steps = (all_steps + 1) >> 1;
  const int s_first = PAIR ? rank * half_steps : 0;                  // this block's steps
  const int n_steps = PAIR ? min(all_steps, s_first + half_steps) : all_steps;
  // all of a warp's loads of one round are issued before the first multiply: one trip to memory
  for (int s0 = s_first + warp * U; s0 < n_steps; s0 += SK_WARPS * U) {
    uint4 wa[U], wb[U];
#pragma unroll
    for (int u = 0; u < U; u++) {
      const int c = (s0 + u) * 4 + t;
      const bool in = (s0 + u) < n_steps && c < K8;
      wa[u] = in ? __ldg(w0 + c) : make_uint4(0, 0, 0, 0);
      wb[u] = in ? __ldg(w1 + c) : make_uint4(0, 0, 0, 0);
    }
    if (s0 == s_first + warp * U) tlc_wait(a, out);                            // first round only
    // the activations of every row group, too, before the first multiply
    uint4 xq[MG][U];
#pragma unroll
    for (int u = 0; u < U; u++) {
      const int c = (s0 + u) * 4 + t;
      const bool in = (s0 + u) < n_steps && c < K8;
#pragma unroll
      for (int mg = 0; mg < MG; mg++) {
        const int row = mg * 8 + g;
        xq[mg][u] = (in && row < M) ? *(reinterpret_cast<const uint4*>(a + (size_t)row * lda) + c) : make_uint4(0, 0, 0, 0);
      }
    }
#pragma unroll
    for (int u = 0; u < U; u++) {
#pragma unroll
      for (int mg = 0; mg < MG; mg++) {
        mma_bf16_16816(acc[mg], wa[u].x, wb[u].x, wa[u].y, wb[u].y, xq[mg][u].x, xq[mg][u].y);
        mma_bf16_16816(acc[mg], wa[u].z, wb[u].z, wa[u].w, wb[u].w, xq[mg][u].z, xq[mg][u].w);
      }
    }
  }
  if (s_first + warp * U >= n_steps) tlc_wait(a, out);                         // warps without a round of their own
  // the warps' partial sums meet in shared memory, at most four row groups at a time
  constexpr int RG = MG < 4 ? MG : 4;
#pragma unroll 1
  for (int g0 = 0; g0 < MG; g0 += RG) {
    if (g0 > 0) __syncthreads();
#pragma unroll
    for (int mg = 0; mg < MG; mg++)
      if (mg >= g0 && mg < g0 + RG)
#pragma unroll
        for (int j = 0; j < 4; j++) red[warp][mg - g0][lane][j] = acc[mg][j];
    __syncthreads();
    if (SWIGLU) {
      // one thread per output value: gate (rows 0..7 of the tile) and up (rows 8..15) of one feature and row
      for (int idx = threadIdx.x; idx < RG * 64; idx += blockDim.x) {
        const int mg = idx >> 6, ln = (idx & 63) >> 1, j = idx & 1;
        float vg = 0.f, vu = 0.f;
#pragma unroll
        for (int ww = 0; ww < SK_WARPS; ww++) { vg += red[ww][mg][ln][j]; vu += red[ww][mg][ln][j + 2]; }
        const int ng = n0 + (ln >> 2), nu = ng + 8;
        const int m = (g0 + mg) * 8 + 2 * (ln & 3) + j;
        if (nu < N && m < M) {
          if (colscale) { vg *= colscale[ng]; vu *= colscale[nu]; }
          if (colbias) { vg += colbias[ng]; vu += colbias[nu]; }
          out[(size_t)m * ldo + (n0 >> 1) + (ln >> 2)] = from_f32<TO>(silu_f(vg) * vu);
        }
      }
      continue;
    }
    // one thread per output value: sum the warps' partial sums in warp order, epilogue, store
    if constexpr (PAIR) {
      if (rank == 1) {
        for (int idx = threadIdx.x; idx < RG * 128; idx += blockDim.x) {
          const int mg = idx >> 7, ln = (idx & 127) >> 2, j = idx & 3;
          float v = 0.f;
#pragma unroll
          for (int ww = 0; ww < SK_WARPS; ww++) v += red[ww][mg][ln][j];
          uint32_t dst;                                              // the same word of block 0's `other`
          asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(dst) : "r"((uint32_t)__cvta_generic_to_shared(&other[g0 * 128 + idx])), "r"(0));
          asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(dst), "f"(v) : "memory");
        }
      }
      asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
      asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
      if (rank == 1) continue;
    }
    for (int idx = threadIdx.x; idx < RG * 128; idx += blockDim.x) {
      const int mg = idx >> 7, ln = (idx & 127) >> 2, j = idx & 3;
      float v = 0.f;
#pragma unroll
      for (int ww = 0; ww < SK_WARPS; ww++) v += red[ww][mg][ln][j];
      if constexpr (PAIR) v += other[g0 * 128 + idx];
      const int n = n0 + (ln >> 2) + (j >= 2 ? 8 : 0);
      const int m = (g0 + mg) * 8 + 2 * (ln & 3) + (j & 1);
      if (n < N && m < M) {
        if (colscale) v *= colscale[n];
        if (colbias) v += colbias[n];
        TO* o = out + (size_t)m * ldo + n;
        if (accumulate) v += to_f32(*o);
        *o = from_f32<TO>(v);
      }
    }
  }
}

template <typename TO, int MG, bool SWIGLU>
static void launch_skinny_mg(const __nv_bfloat16* a, int lda, const __nv_bfloat16* w, int ldw, TO* out, int ldo,
                             const float* colscale, const float* colbias, int accumulate, int M, int N, int K,
                             cudaStream_t stream) {
  const unsigned blocks = (unsigned)((N + 15) / 16);
  const int n_steps = ((K >> 3) + 3) >> 2;
  if constexpr (!SWIGLU) {
    // few tiles and more than one round of K: two blocks a tile, each with half of K
    static int sms = 0;
    if (sms == 0) { int dev = 0; cudaGetDevice(&dev); cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev); }
    const int per_round = SK_WARPS * (MG == 2 ? 2 : 4);
    if (g_skinny_pairs && MG <= 2 && (int)blocks <= sms && n_steps > per_round) {     // MG <= 2: two blocks fit on an SM
      cudaLaunchConfig_t cfg = {};
      cfg.gridDim = dim3(2 * blocks);
      cfg.blockDim = dim3(SK_WARPS * 32);
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
      const int half = (n_steps + 1) / 2;
      if (half <= SK_WARPS * 2 || MG == 2)
        cudaLaunchKernelEx(&cfg, gemm_skinny_mma_kernel<TO, MG, 2, false, true>, a, lda, w, ldw, out, ldo, colscale, colbias, accumulate, M, N, K);
      else
        cudaLaunchKernelEx(&cfg, gemm_skinny_mma_kernel<TO, MG, 4, false, true>, a, lda, w, ldw, out, ldo, colscale, colbias, accumulate, M, N, K);
      return;
    }
  }
  // U steps per warp and round: with one row group and U <= 4, or two and U = 2, two blocks fit on an SM
  // (a warp holds the weights and the activations of a round in registers)
  if (MG == 4 && blocks > 296)      // 17..32 rows, many row tiles: one step a round keeps two blocks on an SM
    tlc_launch(gemm_skinny_mma_kernel<TO, MG, 1, SWIGLU, false>, dim3(blocks), dim3(SK_WARPS * 32), 0, stream, a, lda, w, ldw, out, ldo, colscale, colbias, accumulate, M, N, K);
  else if (n_steps <= SK_WARPS * 2 || MG == 2)
    tlc_launch(gemm_skinny_mma_kernel<TO, MG, 2, SWIGLU, false>, dim3(blocks), dim3(SK_WARPS * 32), 0, stream, a, lda, w, ldw, out, ldo, colscale, colbias, accumulate, M, N, K);
  else
    tlc_launch(gemm_skinny_mma_kernel<TO, MG, 4, SWIGLU, false>, dim3(blocks), dim3(SK_WARPS * 32), 0, stream, a, lda, w, ldw, out, ldo, colscale, colbias, accumulate, M, N, K);
}

template <typename TO, bool SWIGLU>
static int launch_skinny_mma(const void* a, int lda, const void* w, int ldw, void* out, int ldo, const float* colscale,
                             const float* colbias, int accumulate, int M, int N, int K, cudaStream_t stream) {
  const __nv_bfloat16* ap = (const __nv_bfloat16*)a;
  const __nv_bfloat16* wp = (const __nv_bfloat16*)w;
  if (M <= 8) launch_skinny_mg<TO, 1, SWIGLU>(ap, lda, wp, ldw, (TO*)out, ldo, colscale, colbias, accumulate, M, N, K, stream);
  else if (M <= 16) launch_skinny_mg<TO, 2, SWIGLU>(ap, lda, wp, ldw, (TO*)out, ldo, colscale, colbias, accumulate, M, N, K, stream);
  else if (M <= 32) launch_skinny_mg<TO, 4, SWIGLU>(ap, lda, wp, ldw, (TO*)out, ldo, colscale, colbias, accumulate, M, N, K, stream);
  else launch_skinny_mg<TO, 8, SWIGLU>(ap, lda, wp, ldw, (TO*)out, ldo, colscale, colbias, accumulate, M, N, K, stream);
  TLC_CHECK_LAUNCH("linear(skinny mma)");
  return 0;
}

// bfloat16 operands with 16-byte aligned rows and at most 64 rows: the weight-streaming kernel.
extern "C" int tlc_linear_skinny_ok(int a_dtype, int lda, const void* a, int w_dtype, int ldw, const void* w, int M, int K) {
  return a_dtype == TLC_BF16 && w_dtype == TLC_BF16 && M <= 64 && K % 8 == 0 && lda % 8 == 0 && ldw % 8 == 0 &&
         ((uintptr_t)a % 16 == 0) && ((uintptr_t)w % 16 == 0);
}

extern "C" int tlc_linear_skinny(const void* a, int lda, const void* w, int ldw, void* out, int out_dtype, int ldo,
                                 const float* colscale, const float* colbias, int accumulate, int M, int N, int K,
                                 cudaStream_t stream) {
  if (out_dtype == TLC_F32)
    return launch_skinny_mma<float, false>(a, lda, w, ldw, out, ldo, colscale, colbias, accumulate, M, N, K, stream);
  if (out_dtype == TLC_BF16)
    return launch_skinny_mma<__nv_bfloat16, false>(a, lda, w, ldw, out, ldo, colscale, colbias, accumulate, M, N, K, stream);
  return tlc_fail(-1, "linear: unknown output dtype %d", out_dtype);
}

extern "C" void tlc_linear_skinny_pairs(int on) { g_skinny_pairs = on; }

extern "C" int tlc_linear_skinny_swiglu(const void* a, int lda, const void* w, int ldw, void* out, int out_dtype, int ldo,
                                        const float* colscale, const float* colbias, int M, int N, int K,
                                        cudaStream_t stream) {
  if (out_dtype == TLC_F32)
    return launch_skinny_mma<float, true>(a, lda, w, ldw, out, ldo, colscale, colbias, 0, M, N, K, stream);
  if (out_dtype == TLC_BF16)
    return launch_skinny_mma<__nv_bfloat16, true>(a, lda, w, ldw, out, ldo, colscale, colbias, 0, M, N, K, stream);
  return tlc_fail(-1, "linear: unknown output dtype %d", out_dtype);
}
