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
        gemm_skinny_bf16x8_kernel<TO, MT><<<blocks, 256, 0, stream>>>(
            (const __nv_bfloat16*)a, lda, (const __nv_bfloat16*)w, ldw, (TO*)out, ldo, colscale, colbias, accumulate, M,
            N, K, mb);
      else
        gemm_skinny_kernel<TA, TW, TO, MT><<<blocks, 256, 0, stream>>>((const TA*)a, lda, (const TW*)w, ldw, (TO*)out,
                                                                       ldo, colscale, colbias, accumulate, M, N, K, mb);
    }
  } else {
    dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
    gemm_tiled_kernel<TA, TW, TO><<<grid, 256, 0, stream>>>((const TA*)a, lda, (const TW*)w, ldw, (TO*)out, ldo,
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
