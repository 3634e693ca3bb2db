// Token selection on the GPU: greedy, and temperature sampling with the filters of
// CodeClaper/tinyllama.c's sampler (sampler.c:107-257), applied in its order:
// repeat / frequency / presence penalties once per unique token of the history window
// (sampler.c:116-144); greedy when temperature <= 1e-6 or when no filter is active
// (sampler.c:146-151); softmax(logits / T) over the whole vocabulary (sampler.c:156-169);
// top-k, min-p relative to the best probability, top-p nucleus (sampler.c:196-221);
// renormalise and draw (sampler.c:237-251).  Greedy is the first maximum (sampler.c:92-102).
//
// The reference sorts a bounded heap; a GPU block instead finds each cut as a threshold
// on the probability's bit pattern (31 counting passes), keeps ties in token-id order and
// draws by inverse CDF over the survivors in token-id order from a uniform number the
// caller supplies, so the result is a pure function of (logits, parameters, u).
#include "common.cuh"

#define SAMP_THREADS 1024

__device__ __forceinline__ float block_max(float v, float* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float t = lane < nw ? red[lane] : -INFINITY;
    t = warp_max(t);
    if (lane == 0) red[32] = t;
  }
  __syncthreads();
  return red[32];
}

// first index of the maximum of v[0..V)
__device__ int block_argmax(const float* v, int V, float* red, int* redi) {
  float best = -INFINITY;
  int bi = 0x7fffffff;
  for (int i = threadIdx.x; i < V; i += blockDim.x) {
    const float x = v[i];
    if (x > best || (x == best && i < bi)) { best = x; bi = i; }
  }
  // NaN-free logits assumed; reduce (value desc, index asc)
  for (int o = 16; o > 0; o >>= 1) {
    const float ob = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ob > best || (ob == best && oi < bi)) { best = ob; bi = oi; }
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  __syncthreads();
  if (lane == 0) { red[warp] = best; redi[warp] = bi; }
  __syncthreads();
  if (warp == 0) {
    best = lane < nw ? red[lane] : -INFINITY;
    bi = lane < nw ? redi[lane] : 0x7fffffff;
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ob > best || (ob == best && oi < bi)) { best = ob; bi = oi; }
    }
    if (lane == 0) redi[32] = bi == 0x7fffffff ? 0 : bi;
  }
  __syncthreads();
  return redi[32];
}

__global__ void __launch_bounds__(SAMP_THREADS) argmax_kernel(const float* __restrict__ logits, int V, int* __restrict__ out) {
  tlc_pdl(logits, out);
  __shared__ float red[33];
  __shared__ int redi[33];
  const int r = block_argmax(logits + (size_t)blockIdx.x * V, V, red, redi);
  if (threadIdx.x == 0) out[blockIdx.x] = r;
}

extern "C" int tlc_argmax(const float* logits, int R, int V, int* out, cudaStream_t stream) {
  if (R == 0) return 0;
  tlc_launch(argmax_kernel, dim3(R), dim3(SAMP_THREADS), 0, stream, logits, V, out);
  TLC_CHECK_LAUNCH("argmax");
  return 0;
}

// number of set flags over the block; every thread gets the count
__device__ unsigned block_count(unsigned c, unsigned* cnt) {
  __syncthreads();
  if (threadIdx.x == 0) *cnt = 0;
  __syncthreads();
  c = __reduce_add_sync(0xffffffffu, c);
  if ((threadIdx.x & 31) == 0) atomicAdd(cnt, c);
  __syncthreads();
  return *cnt;
}

struct SampleParams {
  float temperature, top_p, min_p, repeat_penalty, frequency_penalty, presence_penalty;
  int top_k, n_history;
};

// exclusive prefix sum over the block of one value per thread; returns the thread's prefix
// and the block total through *total.  scan_buf holds blockDim.x/32 + 1 floats.
__device__ float block_exclusive_scan(float v, float* scan_buf, float* total) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  float inc = v;
  for (int o = 1; o < 32; o <<= 1) {
    const float n = __shfl_up_sync(0xffffffffu, inc, o);
    if (lane >= o) inc += n;
  }
  __syncthreads();
  if (lane == 31) scan_buf[warp] = inc;
  __syncthreads();
  if (warp == 0) {
    float w = lane < nw ? scan_buf[lane] : 0.f;
    float winc = w;
    for (int o = 1; o < 32; o <<= 1) {
      const float n = __shfl_up_sync(0xffffffffu, winc, o);
      if (lane >= o) winc += n;
    }
    if (lane < nw) scan_buf[lane] = winc - w;
    if (lane == 31) scan_buf[32] = winc;
  }
  __syncthreads();
  *total = scan_buf[32];
  return scan_buf[warp] + inc - v;
}

// Survivor test shared by all passes: p above the cut, or equal to it and among the first
// `ties` such elements in token-id order (tie ranks are found with a scan where needed).
//
// One block per row.  `work` is a [R, V] 32-bit scratch that receives the penalised logits
// and then the unnormalised probabilities.
__global__ void __launch_bounds__(SAMP_THREADS)
sample_kernel(const float* __restrict__ logits, float* __restrict__ work, const int* __restrict__ history,
              const float* __restrict__ uniforms, SampleParams sp, int V, int* __restrict__ out) {
  tlc_pdl(logits, work, history, uniforms, out);
  __shared__ float red[33];
  __shared__ int redi[33];
  __shared__ float scan_buf[33];
  __shared__ unsigned cnt_s;
  const int row = blockIdx.x;
  const float* lg = logits + (size_t)row * V;
  float* p = work + (size_t)row * V;
  for (int i = threadIdx.x; i < V; i += blockDim.x) p[i] = lg[i];
  __syncthreads();
  // ---- penalties (sampler.c:116-144) ----
  if ((sp.repeat_penalty != 1.0f || sp.frequency_penalty != 0.0f || sp.presence_penalty != 0.0f) && sp.n_history > 0) {
    const int* hist = history + (size_t)row * sp.n_history;
    for (int j = threadIdx.x; j < sp.n_history; j += blockDim.x) {
      const int tid = hist[j];
      if (tid < 0 || tid >= V) continue;
      bool seen = false;
      for (int k = 0; k < j; k++) if (hist[k] == tid) { seen = true; break; }
      if (seen) continue;
      int count = 1;
      for (int k = j + 1; k < sp.n_history; k++) if (hist[k] == tid) count++;
      float v = p[tid];
      v = v <= 0.0f ? v * sp.repeat_penalty : v / sp.repeat_penalty;
      v -= (float)count * sp.frequency_penalty + sp.presence_penalty;
      p[tid] = v;
    }
    __syncthreads();
  }
  const bool no_filter = sp.top_k == 0 && sp.top_p >= 1.0f && sp.min_p <= 1e-6f;
  if (sp.temperature <= 1e-6f || no_filter) {          // sampler.c:146-151
    const int r = block_argmax(p, V, red, redi);
    if (threadIdx.x == 0) out[row] = r;
    return;
  }
  // ---- softmax numerators (sampler.c:156-169) ----
  const float inv_t = 1.0f / sp.temperature;
  float mx = -INFINITY;
  for (int i = threadIdx.x; i < V; i += blockDim.x) mx = fmaxf(mx, p[i] * inv_t);
  mx = block_max(mx, red);
  float s = 0.f;
  for (int i = threadIdx.x; i < V; i += blockDim.x) { const float e = expf(p[i] * inv_t - mx); p[i] = e; s += e; }
  const float total = block_sum(s, red);
  __syncthreads();
  // ---- top-k: bit pattern of the k-th largest probability (all are >= 0) ----
  unsigned cut = 0;            // survivors: bits(p) > cut, or == cut for the first `ties`
  unsigned ties = 0xffffffffu;
  if (sp.top_k > 0 && sp.top_k < V) {
    unsigned prefix = 0;
    for (int bit = 30; bit >= 0; bit--) {
      const unsigned cand = prefix | (1u << bit);
      unsigned c = 0;
      for (int i = threadIdx.x; i < V; i += blockDim.x) c += __float_as_uint(p[i]) >= cand;
      if (block_count(c, &cnt_s) >= (unsigned)sp.top_k) prefix = cand;
    }
    cut = prefix;
    unsigned c = 0;
    for (int i = threadIdx.x; i < V; i += blockDim.x) c += __float_as_uint(p[i]) > cut;
    ties = (unsigned)sp.top_k - block_count(c, &cnt_s);
    // drop what the cut excludes: zero the losers so later passes need one test only
    unsigned seen_ties = 0;      // ties are rare; resolve them in token-id order chunk by chunk
    for (int base = 0; base < V; base += blockDim.x) {
      const int i = base + threadIdx.x;
      const bool is_tie = i < V && __float_as_uint(p[i]) == cut;
      float tot;
      const float before = block_exclusive_scan(is_tie ? 1.f : 0.f, scan_buf, &tot);
      if (i < V) {
        const unsigned b = __float_as_uint(p[i]);
        if (b < cut || (is_tie && seen_ties + (unsigned)before >= ties)) p[i] = 0.f;
      }
      seen_ties += (unsigned)tot;
      __syncthreads();
    }
  }
  // ---- min-p relative to the best probability, whose numerator is exp(0) = 1 (sampler.c:200-210) ----
  if (sp.min_p > 1e-6f) {
    const float thr = sp.min_p * 1.0f;
    for (int i = threadIdx.x; i < V; i += blockDim.x) if (p[i] < thr) p[i] = 0.f;
    __syncthreads();
  }
  // ---- top-p: smallest descending prefix whose normalised mass reaches top_p (sampler.c:213-221) ----
  if (sp.top_p < 1.0f) {
    const float target = sp.top_p * total;            // compare unnormalised masses
    unsigned prefix = 0;
    for (int bit = 30; bit >= 0; bit--) {
      const unsigned cand = prefix | (1u << bit);
      float m = 0.f;
      for (int i = threadIdx.x; i < V; i += blockDim.x) { const float v = p[i]; if (__float_as_uint(v) >= cand) m += v; }
      m = block_sum(m, red);
      if (m >= target) prefix = cand;
      __syncthreads();
    }
    // prefix = the largest cut whose mass at-or-above reaches the target (0: keep every survivor)
    if (prefix != 0) {
      float above = 0.f;
      for (int i = threadIdx.x; i < V; i += blockDim.x) { const float v = p[i]; if (__float_as_uint(v) > prefix) above += v; }
      above = block_sum(above, red);
      const float tv = __uint_as_float(prefix);
      // ties at the cut enter in token-id order until the mass reaches the target
      unsigned need = 0;
      if (above < target) need = (unsigned)ceilf((target - above) / tv);
      if (need == 0 && above < target) need = 1;
      unsigned seen_ties = 0;
      for (int base = 0; base < V; base += blockDim.x) {
        const int i = base + threadIdx.x;
        const bool is_tie = i < V && __float_as_uint(p[i]) == prefix;
        float tot;
        const float before = block_exclusive_scan(is_tie ? 1.f : 0.f, scan_buf, &tot);
        if (i < V) {
          const unsigned b = __float_as_uint(p[i]);
          if (b < prefix || (is_tie && seen_ties + (unsigned)before >= need)) p[i] = 0.f;
        }
        seen_ties += (unsigned)tot;
        __syncthreads();
      }
    }
  }
  // ---- renormalise and draw by inverse CDF in token-id order (sampler.c:237-251) ----
  float m = 0.f;
  for (int i = threadIdx.x; i < V; i += blockDim.x) m += p[i];
  m = block_sum(m, red);
  const float target = uniforms[row] * m;
  if (threadIdx.x == 0) cnt_s = 0xffffffffu;
  __syncthreads();
  float run = 0.f;
  int last_alive = -1;
  for (int base = 0; base < V; base += blockDim.x) {
    const int i = base + threadIdx.x;
    const float v = i < V ? p[i] : 0.f;
    float tot;
    const float before = run + block_exclusive_scan(v, scan_buf, &tot);
    if (v > 0.f) {
      last_alive = i;
      if (target < before + v) atomicMin(&cnt_s, (unsigned)i);
    }
    run += tot;
    __syncthreads();
    const bool found = cnt_s != 0xffffffffu;
    __syncthreads();                       // nobody writes cnt_s again before everybody has read it
    if (found) break;
  }
  if (cnt_s == 0xffffffffu) {     // rounding left the target at the very end: last survivor (sampler.c:253-255)
    if (threadIdx.x == 0) redi[0] = 0;
    __syncthreads();
    if (last_alive >= 0) atomicMax(&redi[0], last_alive);
    __syncthreads();
    if (threadIdx.x == 0) out[row] = redi[0];
    return;
  }
  if (threadIdx.x == 0) out[row] = (int)cnt_s;
}

extern "C" int tlc_sample(const float* logits, float* work, const int* history, const float* uniforms, int R, int V,
                          float temperature, int top_k, float top_p, float min_p, float repeat_penalty,
                          int n_history, float frequency_penalty, float presence_penalty, int* out,
                          cudaStream_t stream) {
  if (R == 0) return 0;
  TLC_REQUIRE(V >= 1, "sample: empty vocabulary");
  TLC_REQUIRE(temperature >= 0.f, "sample: temperature must be >= 0, got %g", temperature);
  TLC_REQUIRE(top_p > 0.f && top_p <= 1.f, "sample: top-p must be in (0, 1], got %g", top_p);
  TLC_REQUIRE(min_p >= 0.f && min_p <= 1.f, "sample: min-p must be in [0, 1], got %g", min_p);
  SampleParams sp{temperature, top_p, min_p, repeat_penalty, frequency_penalty, presence_penalty, top_k,
                  history ? n_history : 0};
  tlc_launch(sample_kernel, dim3(R), dim3(SAMP_THREADS), 0, stream, logits, work, history, uniforms, sp, V, out);
  TLC_CHECK_LAUNCH("sample");
  return 0;
}
