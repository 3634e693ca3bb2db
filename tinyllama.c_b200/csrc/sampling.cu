// Token selection on the GPU: greedy, and temperature sampling with the filters of
// CodeClaper/tinyllama.c's sampler (sampler.c:107-257), applied in its order:
// repeat / frequency / presence penalties once per unique token of the history window
// (sampler.c:116-144); greedy when temperature <= 1e-6 or when no filter is active
// (sampler.c:146-151); softmax(logits / T) over the whole vocabulary (sampler.c:156-169);
// top-k, min-p relative to the best probability, top-p nucleus (sampler.c:196-221);
// renormalise and draw (sampler.c:237-251).  Greedy is the first maximum (sampler.c:92-102).
//
// The reference sorts a bounded heap; a GPU block instead finds each cut as a threshold
// on the probability's bit pattern, keeps ties in token-id order and draws by inverse CDF
// over the survivors in token-id order from a uniform number the caller supplies, so the
// result is a pure function of (logits, parameters, u).  With a top-k of at most 1024 the
// threshold comes from a three-pass radix select and the rest works on the survivors in
// shared memory (sample_topk_kernel); otherwise every cut is found by 31 counting passes
// over the vocabulary (sample_kernel).
#include "common.cuh"

#define SAMP_THREADS 1024

// f(value, index) over a row of V floats, the block's threads striding through it: 16 bytes a load where
// the row allows it (a pass over the vocabulary is bound by the loads one block can keep in flight).
template <typename F>
__device__ __forceinline__ void row_read(const float* __restrict__ p, int V, F f) {
  if ((V & 3) == 0 && (((uintptr_t)p) & 15) == 0) {
    const float4* p4 = reinterpret_cast<const float4*>(p);
#pragma unroll 4
    for (int i = threadIdx.x; i < (V >> 2); i += blockDim.x) {
      const float4 v = p4[i];
      f(v.x, 4 * i); f(v.y, 4 * i + 1); f(v.z, 4 * i + 2); f(v.w, 4 * i + 3);
    }
  } else {
#pragma unroll 4
    for (int i = threadIdx.x; i < V; i += blockDim.x) f(p[i], i);
  }
}

// dst[i] = f(src[i], i) over a row (dst may be src)
template <typename F>
__device__ __forceinline__ void row_map(const float* src, float* dst, int V, F f) {
  if ((V & 3) == 0 && ((((uintptr_t)src) | ((uintptr_t)dst)) & 15) == 0) {
    const float4* s4 = reinterpret_cast<const float4*>(src);
    float4* d4 = reinterpret_cast<float4*>(dst);
#pragma unroll 4
    for (int i = threadIdx.x; i < (V >> 2); i += blockDim.x) {
      float4 v = s4[i];
      v.x = f(v.x, 4 * i); v.y = f(v.y, 4 * i + 1); v.z = f(v.z, 4 * i + 2); v.w = f(v.w, 4 * i + 3);
      d4[i] = v;
    }
  } else {
#pragma unroll 4
    for (int i = threadIdx.x; i < V; i += blockDim.x) dst[i] = f(src[i], i);
  }
}

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

// A row spread over several blocks (a decode step has a few rows of a large vocabulary: one block a row would
// leave the GPU to a handful of SMs).  Each block finds the first maximum of its slice and folds it into the
// row's 64-bit key by atomicMax: the value mapped to an unsigned number of the same order in the high half,
// ~index in the low half, so that the larger value wins and, among equal values, the smaller index.  The block
// that arrives last writes the row's result and sets key and counter back to zero.
// work: R keys (64-bit) followed by R counters (32-bit), all zero between launches.
constexpr int ARGMAX_SLICE = 2048;
__global__ void __launch_bounds__(SAMP_THREADS)
argmax_split_kernel(const float* __restrict__ logits, int V, int* __restrict__ out, unsigned long long* __restrict__ keys,
                    unsigned* __restrict__ counters) {
  tlc_pdl(logits, out, keys, counters);
  __shared__ float red[33];
  __shared__ int redi[33];
  const int r = blockIdx.x, v0 = blockIdx.y * ARGMAX_SLICE, n = min(ARGMAX_SLICE, V - v0);
  const float* row = logits + (size_t)r * V + v0;
  const int bi = block_argmax(row, n, red, redi);
  if (threadIdx.x == 0) {
    const unsigned u = __float_as_uint(row[bi]);
    const unsigned ordered = (u & 0x80000000u) ? ~u : (u | 0x80000000u);
    atomicMax(keys + r, ((unsigned long long)ordered << 32) | (unsigned long long)(0xffffffffu - (unsigned)(v0 + bi)));
    __threadfence();
    if (atomicInc(counters + r, gridDim.y - 1) == gridDim.y - 1) {
      __threadfence();
      const unsigned long long best = atomicExch(keys + r, 0ull);
      out[r] = (int)(0xffffffffu - (unsigned)(best & 0xffffffffull));
    }
  }
}

extern "C" int tlc_argmax(const float* logits, int R, int V, int* out, void* work, cudaStream_t stream) {
  if (R == 0) return 0;
  const int slices = (V + ARGMAX_SLICE - 1) / ARGMAX_SLICE;
  if (work != nullptr && slices > 1 && slices <= 65535 && ((uintptr_t)work % 8) == 0) {
    unsigned long long* keys = (unsigned long long*)work;
    tlc_launch(argmax_split_kernel, dim3(R, slices), dim3(SAMP_THREADS), 0, stream, logits, V, out, keys, (unsigned*)(keys + R));
  } else {
    tlc_launch(argmax_kernel, dim3(R), dim3(SAMP_THREADS), 0, stream, logits, V, out);
  }
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

// The part every sampling kernel starts with: the row's logits into `p`, the penalties
// (sampler.c:116-144), the greedy cases (sampler.c:146-151; returns true when the token is chosen),
// and the softmax numerators exp(l / T - max) in place of the logits with their sum in *total
// (sampler.c:156-169).
__device__ bool sample_prologue(const float* __restrict__ logits, float* __restrict__ work, const int* __restrict__ history,
                                const SampleParams& sp, int V, int* __restrict__ out, float* red, int* redi,
                                float** p_out, float* total_out, unsigned* hist0 = nullptr) {
  const int row = blockIdx.x;
  const float* lg = logits + (size_t)row * V;
  float* p = work + (size_t)row * V;
  *p_out = p;
  row_map(lg, p, V, [](float v, int) { return v; });
  __syncthreads();
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
  if (sp.temperature <= 1e-6f || no_filter) {
    const int r = block_argmax(p, V, red, redi);
    if (threadIdx.x == 0) out[row] = r;
    return true;
  }
  const float inv_t = 1.0f / sp.temperature;
  float mx = -INFINITY;
  row_read(p, V, [&](float v, int) { mx = fmaxf(mx, v * inv_t); });
  mx = block_max(mx, red);
  float s = 0.f;
  if (hist0 != nullptr) {
    // the short-list kernel counts the top digit of the probabilities' bit patterns in the same pass
    row_map(p, p, V, [&](float v, int) {
      const float e = expf(v * inv_t - mx);
      s += e;
      atomicAdd(&hist0[__float_as_uint(e) >> 20], 1u);
      return e;
    });
  } else {
    row_map(p, p, V, [&](float v, int) { const float e = expf(v * inv_t - mx); s += e; return e; });
  }
  *total_out = block_sum(s, red);
  __syncthreads();
  return false;
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
  float* p;
  float total;
  if (sample_prologue(logits, work, history, sp, V, out, red, redi, &p, &total)) return;
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


#define SAMP_KMAX 1024       // survivors of top-k that the short-list kernel holds in shared memory
#define SAMP_BINS 2048       // = 2 * SAMP_THREADS: the digit scan gives every thread two bins

// The same selection when 0 < top_k <= SAMP_KMAX: the k-th largest probability is found by a radix
// select on the bit pattern (three counting passes of 11, 11 and 9 bits instead of 31 of one bit), the at
// most top_k survivors are gathered into shared memory and put in token-id order, and min-p, top-p and the
// draw work on that short list.  Which tokens survive, how ties at a cut are broken (token-id order) and
// the order of the draw are those of the general kernel above; sums over the survivors are taken
// in token-id order.
__global__ void __launch_bounds__(SAMP_THREADS)
sample_topk_kernel(const float* __restrict__ logits, float* __restrict__ work, const int* __restrict__ history,
                   const float* __restrict__ uniforms, SampleParams sp, int V, int* __restrict__ out) {
  tlc_pdl(logits, work, history, uniforms, out);
  __shared__ float red[33];
  __shared__ int redi[33];
  __shared__ float scan_buf[33];
  __shared__ unsigned hist[SAMP_BINS];
  __shared__ float sv[SAMP_KMAX], sv2[SAMP_KMAX];
  __shared__ int si[SAMP_KMAX], si2[SAMP_KMAX];
  __shared__ unsigned s_digit, s_krem, s_count, s_n, s_bits;
  __shared__ int s_pick, s_last;
  const int row = blockIdx.x, tid = threadIdx.x;
  float* p;
  float total;
  for (int j = tid; j < SAMP_BINS; j += blockDim.x) hist[j] = 0;
  __syncthreads();
  if (sample_prologue(logits, work, history, sp, V, out, red, redi, &p, &total, hist)) return;
  // ---- top-k: bit pattern of the k-th largest probability (all are >= 0, so bit 31 is clear) ----
  unsigned prefix = 0, k_rem = (unsigned)sp.top_k, n_at = 0;
#pragma unroll 1
  for (int pass = 0; pass < 3; pass++) {
    const int shift = pass == 0 ? 20 : pass == 1 ? 9 : 0;          // the digit's lowest bit
    const int above = pass == 0 ? 31 : pass == 1 ? 20 : 9;         // bits from here up are settled
    const unsigned mask = pass == 2 ? 511u : 2047u;
    if (pass > 0) {                                                 // the first digit was counted with the numerators
      for (int j = tid; j < SAMP_BINS; j += blockDim.x) hist[j] = 0;
      __syncthreads();
      row_read(p, V, [&](float v, int) {
        const unsigned b = __float_as_uint(v);
        if ((b >> above) == (prefix >> above)) atomicAdd(&hist[(b >> shift) & mask], 1u);
      });
      __syncthreads();
    }
    // from the highest digit down: the digit at which the count reaches what is still wanted
    const int b1 = SAMP_BINS - 1 - 2 * tid, b0 = b1 - 1;
    const unsigned c1 = hist[b1], c0 = hist[b0];
    float tot;
    const unsigned before = (unsigned)block_exclusive_scan((float)(c1 + c0), scan_buf, &tot);   // counts < 2^24: exact
    if (before < k_rem && before + c1 + c0 >= k_rem) {
      if (before + c1 >= k_rem) { s_digit = (unsigned)b1; s_krem = k_rem - before; s_count = c1; }
      else { s_digit = (unsigned)b0; s_krem = k_rem - before - c1; s_count = c0; }
    }
    __syncthreads();
    prefix |= s_digit << shift;
    k_rem = s_krem;
    n_at = s_count;
    __syncthreads();
  }
  const unsigned cut = prefix;      // survivors: bits(p) > cut, and the first k_rem of the n_at elements at the cut
  if (cut != 0 && n_at > k_rem) {
    // more elements tie at the cut than may stay: the first k_rem in token-id order do
    unsigned seen_ties = 0;
    for (int base = 0; base < V; base += blockDim.x) {
      const int i = base + tid;
      const bool is_tie = i < V && __float_as_uint(p[i]) == cut;
      float tot;
      const float before = block_exclusive_scan(is_tie ? 1.f : 0.f, scan_buf, &tot);
      if (is_tie && seen_ties + (unsigned)before >= k_rem) p[i] = 0.f;
      seen_ties += (unsigned)tot;
      __syncthreads();
    }
  }
  // ---- the survivors into shared memory (probabilities of zero can never be drawn: left out) ----
  if (tid == 0) s_n = 0;
  __syncthreads();
  row_read(p, V, [&](float v, int i) {
    const unsigned b = __float_as_uint(v);
    if (b != 0 && b >= cut) {
      const unsigned at = atomicAdd(&s_n, 1u);
      if (at < SAMP_KMAX) { sv[at] = v; si[at] = i; }
    }
  });
  __syncthreads();
  const int n = (int)min(s_n, (unsigned)SAMP_KMAX);
  // token-id order: an element's place is the number of survivors with a smaller id
  if (tid < n) {
    const int mine = si[tid];
    int r = 0;
    for (int j = 0; j < n; j++) r += si[j] < mine;
    sv2[r] = sv[tid];
    si2[r] = mine;
  }
  __syncthreads();
  // ---- min-p relative to the best probability, whose numerator is exp(0) = 1 (sampler.c:200-210) ----
  if (sp.min_p > 1e-6f) {
    if (tid < n && sv2[tid] < sp.min_p) sv2[tid] = 0.f;
    __syncthreads();
  }
  // ---- top-p: smallest descending prefix whose normalised mass reaches top_p (sampler.c:213-221) ----
  if (sp.top_p < 1.0f) {
    const float target = sp.top_p * total;            // compare unnormalised masses
    if (tid == 0) s_bits = 0;
    __syncthreads();
    if (tid < n) {
      const float v = sv2[tid];
      if (v > 0.f) {
        float m = 0.f;
        for (int j = 0; j < n; j++) { const float w = sv2[j]; if (w >= v) m += w; }
        if (m >= target) atomicMax(&s_bits, __float_as_uint(v));
      }
    }
    __syncthreads();
    const unsigned pc = s_bits;     // the largest value whose mass at-or-above reaches the target (0: keep every survivor)
    if (pc != 0) {
      float above = 0.f;
      for (int j = 0; j < n; j++) { const float w = sv2[j]; if (__float_as_uint(w) > pc) above += w; }
      // ties at the cut enter in token-id order until the mass reaches the target
      unsigned need = 0;
      if (above < target) need = (unsigned)ceilf((target - above) / __uint_as_float(pc));
      if (need == 0 && above < target) need = 1;
      bool drop = false;
      if (tid < n) {
        const unsigned b = __float_as_uint(sv2[tid]);
        if (b < pc) drop = true;
        else if (b == pc) {
          unsigned earlier = 0;
          for (int j = 0; j < tid; j++) earlier += __float_as_uint(sv2[j]) == pc;
          drop = earlier >= need;
        }
      }
      __syncthreads();
      if (drop) sv2[tid] = 0.f;
      __syncthreads();
    }
  }
  // ---- renormalise and draw by inverse CDF in token-id order (sampler.c:237-251) ----
  if (tid == 0) { s_pick = 0x7fffffff; s_last = -1; }
  __syncthreads();
  float m = 0.f;
  for (int j = 0; j < n; j++) m += sv2[j];
  const float target = uniforms[row] * m;
  if (tid < n) {
    const float v = sv2[tid];
    if (v > 0.f) {
      float before = 0.f;
      for (int j = 0; j < tid; j++) before += sv2[j];
      if (target < before + v) atomicMin(&s_pick, tid);
      atomicMax(&s_last, tid);
    }
  }
  __syncthreads();
  // rounding may leave the target at the very end: then the last survivor (sampler.c:253-255)
  if (tid == 0) out[row] = si2[s_pick != 0x7fffffff ? s_pick : max(s_last, 0)];
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
  if (top_k > 0 && top_k <= SAMP_KMAX && top_k < V)
    tlc_launch(sample_topk_kernel, dim3(R), dim3(SAMP_THREADS), 0, stream, logits, work, history, uniforms, sp, V, out);
  else
    tlc_launch(sample_kernel, dim3(R), dim3(SAMP_THREADS), 0, stream, logits, work, history, uniforms, sp, V, out);
  TLC_CHECK_LAUNCH("sample");
  return 0;
}
