// Single-token attention as one kernel (bfloat16 cache, head sizes 64, 128, 256).
//
// What the separate kernels do in three launches happens here in one: the rotation of the row's
// queries and of its new key (split-half form, angle = position * inv_freq[i] in 32-bit;
// CodeClaper/tinyllama.c cpu_op.c:637-651), the store of the new key/value row into its page
// (cpu_op.c:995-1008), attention of the row over a split of 128 or 256 keys per block with 32-bit
// scores, statistics and accumulator (cpu_op.c:1010-1062), and the merge of the splits, which
// the last block of a (row, key/value head) to finish does.  A single-token step is a chain of
// short dependent kernels; every launch taken out of the chain shortens the step.
//
// Arrival counting: every block of a (row, kv head) adds one to arrivals[row * KV + kv head]
// with atomicInc modulo the number of splits, so the counter is back at zero when the kernel
// ends and needs no clearing between launches.  It must be zero before the first launch.
#include "common.cuh"

#define FD_NT 512       // threads per block
#define FD_NW (FD_NT / 32)
#define FD_MAXG 8

// HD: head size; GT: compile-time bound of the query heads per key/value head (G <= GT); KEYS: keys
// per block, 128 or (long contexts, so that the grid stays near one wave) 256.
// The block's 512 threads score its keys four (or two) to a key (each takes every fourth 16-byte
// piece of the key row), then take the value rows HD/8 lanes to a row; partial outputs of the
// rows of a warp meet by shuffles, those of the warps in shared memory.
template <int HD, int GT, int KEYS>
__global__ void __launch_bounds__(FD_NT)
attention_decode_fused_kernel(const float* __restrict__ qkv, int ld, int q_off, int k_off, int v_off,
                              __nv_bfloat16* __restrict__ k_pages, __nv_bfloat16* __restrict__ v_pages,
                              const float* __restrict__ inv_freq, int rope_dim, int write_kv,
                              const int* __restrict__ block_table, int max_pages, const int* __restrict__ positions,
                              const int* __restrict__ row_seq, const int* __restrict__ slots, float* __restrict__ part_o,
                              float* __restrict__ part_ml, unsigned* __restrict__ arrivals,
                              __nv_bfloat16* __restrict__ out, int H, int KV, float scale, int window, int n_splits) {
  // Keys and values of earlier positions were stored by earlier steps and are fetched before the
  // wait on the previous kernel; the row's own projection is read after it.
  asm volatile("griddepcontrol.launch_dependents;");
  extern __shared__ float sh[];
  constexpr int TPK = FD_NT / KEYS;          // threads per key while scoring
  constexpr int CH = HD / 8;                 // 16-byte pieces of a row = lanes per value row
  constexpr int CPT = CH / TPK;           // pieces of a key row per scoring thread
  constexpr int ROWS = FD_NT / CH;           // value rows in flight
  constexpr int RPT = KEYS / ROWS;        // value rows per thread
  static_assert(CH % TPK == 0 && KEYS % ROWS == 0 && CH <= 32, "head size");
  const int tid = threadIdx.x, lane = tid & 31, wp = tid >> 5;
  const int t = blockIdx.x, g = blockIdx.y, split = blockIdx.z;
  const int G = H / KV;
  const int pos = positions[t];
  const int n_keys = pos + 1;
  const int start = (window > 0 && n_keys > window) ? n_keys - window : 0;
  const int k0 = split * KEYS;
  const int smem_floats = G * HD + G * KEYS + FD_NW * GT + FD_NW * G * HD;     // floats of dynamic shared memory
  float* ml = part_ml + (((size_t)t * H + (size_t)g * G) * n_splits + split) * 2;
  const bool empty = k0 >= n_keys || k0 + KEYS <= start;     // the same for all threads of the block
  __shared__ int pages[KEYS / TLC_PAGE + 1];
  __shared__ int s_last;
  if (empty) {
    tlc_wait(ml);
    if (tid < G) { ml[(size_t)tid * n_splits * 2] = -INFINITY; ml[(size_t)tid * n_splits * 2 + 1] = 0.f; }
  } else {
    float* qs = sh;                                   // [G][HD]
    float* ps = qs + (size_t)G * HD;                  // [G][KEYS]
    float* red = ps + (size_t)G * KEYS;            // [FD_NW][GT]
    float* os = red + FD_NW * GT;                     // [FD_NW][G][HD]
    __nv_bfloat16* knew = reinterpret_cast<__nv_bfloat16*>(os + (size_t)FD_NW * G * HD);   // [HD]
    __nv_bfloat16* vnew = knew + HD;                                                       // [HD]
    const int* table = block_table + (size_t)slots[row_seq[t]] * max_pages;
    const bool has_new = write_kv && pos >= k0 && pos < k0 + KEYS;   // this block holds the row's own key
    const int key = tid / TPK, piece = tid % TPK;
    const int kp = k0 + key;
    const bool valid = kp >= start && kp < n_keys;
    uint4 kq[CPT];
    const uint4* kr = nullptr;
    if (valid) {
      kr = reinterpret_cast<const uint4*>(k_pages + (((size_t)table[kp / TLC_PAGE] * KV + g) * TLC_PAGE + kp % TLC_PAGE) * HD);
      if (kp != pos) {
#pragma unroll
        for (int i = 0; i < CPT; i++) kq[i] = __ldg(kr + piece + TPK * i);
      }
    }
    if (tid <= KEYS / TLC_PAGE) {
      const int pi = k0 / TLC_PAGE + tid;
      pages[tid] = (pi * TLC_PAGE < n_keys) ? table[pi] : 0;
    }
    // this thread's value rows, too, are on their way before the wait (all but the row's own position)
    const int nk = min(KEYS, n_keys - k0);
    const int dl = tid % CH, rg = tid / CH;
    uint4 vq[RPT];
#pragma unroll
    for (int u = 0; u < RPT; u++) {
      const int j = rg + u * ROWS;
      const int kj = k0 + j;
      const bool use = j < nk && kj >= start && kj != pos;     // outside the window a page may have been given back
      vq[u] = use ? __ldg(reinterpret_cast<const uint4*>(
                              v_pages + (((size_t)table[kj / TLC_PAGE] * KV + g) * TLC_PAGE + kj % TLC_PAGE) * HD) + dl)
                  : make_uint4(0, 0, 0, 0);
    }
    tlc_wait(qkv, kr, k_pages, v_pages, part_o, ml);
    // rotation: the thread of dim d turns that dim of every query head of the group and of the key;
    // all of its loads are issued before the first use
    if (tid < HD) {
      const float* row = qkv + (size_t)t * ld;
      const int half = rope_dim >> 1;
      const int d = tid;
      const bool rot = d < rope_dim;
      const bool lo = d < half;
      const int i = rot ? (lo ? d : d - half) : d;          // first element of the pair (or the dim itself)
      const int j = rot ? i + half : d;                     // second element
      float a[GT + 1], b[GT + 1], vv = 0.f;
#pragma unroll
      for (int hg = 0; hg < GT; hg++) {
        if (hg < G) {
          const float* src = row + q_off + ((size_t)g * G + hg) * HD;
          a[hg] = src[i];
          b[hg] = src[j];
        }
      }
      if (has_new) {
        const float* src = row + k_off + (size_t)g * HD;
        a[GT] = src[i];
        b[GT] = src[j];
        vv = row[v_off + (size_t)g * HD + d];
      }
      float sn = 0.f, cs = 1.f;
      if (rot) sincosf((float)pos * inv_freq[i], &sn, &cs);
#pragma unroll
      for (int hg = 0; hg < GT; hg++) {
        if (hg < G) {
          const float v = rot ? (lo ? a[hg] * cs - b[hg] * sn : a[hg] * sn + b[hg] * cs) : a[hg];
          qs[hg * HD + d] = __bfloat162float(__float2bfloat16_rn(v)) * scale;
        }
      }
      if (has_new) {
        const float v = rot ? (lo ? a[GT] * cs - b[GT] * sn : a[GT] * sn + b[GT] * cs) : a[GT];
        knew[d] = __float2bfloat16_rn(v);
        vnew[d] = __float2bfloat16_rn(vv);
      }
    }
    __syncthreads();
    if (has_new) {
      const size_t at = (((size_t)table[pos / TLC_PAGE] * KV + g) * TLC_PAGE + pos % TLC_PAGE) * HD;
      if (tid < CH) {
        reinterpret_cast<uint4*>(k_pages + at)[tid] = reinterpret_cast<const uint4*>(knew)[tid];
        reinterpret_cast<uint4*>(v_pages + at)[tid] = reinterpret_cast<const uint4*>(vnew)[tid];
      }
      if (kp == pos) {
#pragma unroll
        for (int i = 0; i < CPT; i++) kq[i] = reinterpret_cast<const uint4*>(knew)[piece + TPK * i];
      }
    } else if (valid && kp == pos) {
#pragma unroll
      for (int i = 0; i < CPT; i++) kq[i] = kr[piece + TPK * i];
    }
    float s[GT];
#pragma unroll
    for (int hg = 0; hg < GT; hg++) s[hg] = 0.f;
    if (valid) {
#pragma unroll
      for (int i = 0; i < CPT; i++) {
        const int c = piece + TPK * i;
        const __nv_bfloat162* kb = reinterpret_cast<const __nv_bfloat162*>(&kq[i]);
        float kf[8];
#pragma unroll
        for (int e = 0; e < 4; e++) { const float2 f = __bfloat1622float2(kb[e]); kf[2 * e] = f.x; kf[2 * e + 1] = f.y; }
#pragma unroll
        for (int hg = 0; hg < GT; hg++) {
          if (hg < G) {
            const float4 qa = *reinterpret_cast<const float4*>(qs + hg * HD + c * 8);
            const float4 qb = *reinterpret_cast<const float4*>(qs + hg * HD + c * 8 + 4);
            s[hg] = fmaf(kf[0], qa.x, s[hg]); s[hg] = fmaf(kf[1], qa.y, s[hg]);
            s[hg] = fmaf(kf[2], qa.z, s[hg]); s[hg] = fmaf(kf[3], qa.w, s[hg]);
            s[hg] = fmaf(kf[4], qb.x, s[hg]); s[hg] = fmaf(kf[5], qb.y, s[hg]);
            s[hg] = fmaf(kf[6], qb.z, s[hg]); s[hg] = fmaf(kf[7], qb.w, s[hg]);
          }
        }
      }
    }
    // the key's threads add their pieces (all of them then hold the score)
#pragma unroll
    for (int hg = 0; hg < GT; hg++)
#pragma unroll
      for (int o = 1; o < TPK; o <<= 1) s[hg] += __shfl_xor_sync(0xffffffffu, s[hg], o);
    // maximum and sum over the block's keys, all heads of the group at once
    {
#pragma unroll
      for (int hg = 0; hg < GT; hg++) {
        if (hg < G) {
          const float m = warp_max(valid ? s[hg] : -INFINITY);
          if (lane == 0) red[wp * GT + hg] = m;
        }
      }
      __syncthreads();
      float lsum[GT];
#pragma unroll
      for (int hg = 0; hg < GT; hg++) {
        if (hg < G) {
          float m = red[hg];
#pragma unroll
          for (int w = 1; w < FD_NW; w++) m = fmaxf(m, red[w * GT + hg]);
          const float p = valid ? expf(s[hg] - m) : 0.f;
          if (piece == 0) ps[hg * KEYS + key] = p;
          lsum[hg] = warp_sum(piece == 0 ? p : 0.f);
          s[hg] = m;
        }
      }
      __syncthreads();
#pragma unroll
      for (int hg = 0; hg < GT; hg++)
        if (hg < G && lane == 0) red[wp * GT + hg] = lsum[hg];
      __syncthreads();
      if (tid < G) {
        const int hg = tid;
        float mm = -INFINITY;
#pragma unroll
        for (int i = 0; i < GT; i++) if (i == hg) mm = s[i];
        float l = 0.f;
#pragma unroll
        for (int w = 0; w < FD_NW; w++) l += red[w * GT + hg];
        ml[(size_t)hg * n_splits * 2] = mm;
        ml[(size_t)hg * n_splits * 2 + 1] = l;
      }
    }
    __syncthreads();
    float acc[GT][8];
#pragma unroll
    for (int hg = 0; hg < GT; hg++)
#pragma unroll
      for (int i = 0; i < 8; i++) acc[hg][i] = 0.f;
    {
      // the value row at the row's own position: written above by this block, or (a layer that only reads) by
      // an earlier kernel
#pragma unroll
      for (int u = 0; u < RPT; u++) {
        const int j = rg + u * ROWS;
        const int kj = k0 + j;
        if (j < nk && kj >= start && kj == pos) {
          if (has_new) vq[u] = reinterpret_cast<const uint4*>(vnew)[dl];
          else vq[u] = *(reinterpret_cast<const uint4*>(
                             v_pages + (((size_t)pages[j / TLC_PAGE] * KV + g) * TLC_PAGE + kj % TLC_PAGE) * HD) + dl);
        }
      }
#pragma unroll
      for (int u = 0; u < RPT; u++) {
        const int j = rg + u * ROWS;
        if (j >= nk) continue;
        const __nv_bfloat162* vb = reinterpret_cast<const __nv_bfloat162*>(&vq[u]);
        float vf[8];
#pragma unroll
        for (int i = 0; i < 4; i++) { const float2 f = __bfloat1622float2(vb[i]); vf[2 * i] = f.x; vf[2 * i + 1] = f.y; }
#pragma unroll
        for (int hg = 0; hg < GT; hg++) {
          if (hg < G) {
            const float p = ps[hg * KEYS + j];
#pragma unroll
            for (int i = 0; i < 8; i++) acc[hg][i] = fmaf(p, vf[i], acc[hg][i]);
          }
        }
      }
    }
    // the rows of a warp meet by shuffles, the warps in shared memory
#pragma unroll
    for (int o = CH; o < 32; o <<= 1)
#pragma unroll
      for (int hg = 0; hg < GT; hg++)
#pragma unroll
        for (int i = 0; i < 8; i++) acc[hg][i] += __shfl_xor_sync(0xffffffffu, acc[hg][i], o);
    if (lane < CH) {
#pragma unroll
      for (int hg = 0; hg < GT; hg++) {
        if (hg < G) {
          float* o = os + ((size_t)wp * G + hg) * HD + dl * 8;
          *reinterpret_cast<float4*>(o) = make_float4(acc[hg][0], acc[hg][1], acc[hg][2], acc[hg][3]);
          *reinterpret_cast<float4*>(o + 4) = make_float4(acc[hg][4], acc[hg][5], acc[hg][6], acc[hg][7]);
        }
      }
    }
    __syncthreads();
    for (int idx = tid; idx < G * HD; idx += FD_NT) {
      float v = 0.f;
#pragma unroll
      for (int w = 0; w < FD_NW; w++) v += os[(size_t)w * G * HD + idx];
      const int hg = idx / HD, d = idx % HD;
      part_o[((((size_t)t * H + (size_t)g * G + hg) * n_splits) + split) * HD + d] = v;
    }
  }
  // ---- the last block of this (row, kv head) merges the splits -----------------------------------
  __threadfence();
  __syncthreads();
  if (tid == 0) {
    const unsigned old = atomicInc(arrivals + (size_t)t * KV + g, (unsigned)(n_splits - 1));
    s_last = old == (unsigned)(n_splits - 1);
  }
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  if (2 * G * n_splits <= smem_floats) {
    // statistics of all heads and splits into shared memory (one round trip), weights from them,
    // then the weighted sum with the loads of a thread in flight together
    for (int idx = tid; idx < G * n_splits; idx += FD_NT) {
      const int hg = idx / n_splits, s = idx % n_splits;
      const float2 v = __ldcg(reinterpret_cast<const float2*>(part_ml + (((size_t)t * H + (size_t)g * G + hg) * n_splits + s) * 2));
      sh[2 * idx] = v.x;
      sh[2 * idx + 1] = v.y;
    }
    __syncthreads();
    for (int hg = wp; hg < G; hg += FD_NW) {
      float* e = sh + (size_t)2 * hg * n_splits;
      float m = -INFINITY;
      for (int s = lane; s < n_splits; s += 32) m = fmaxf(m, e[2 * s]);
      m = warp_max(m);
      float l = 0.f;
      for (int s = lane; s < n_splits; s += 32) if (e[2 * s + 1] > 0.f) l += e[2 * s + 1] * expf(e[2 * s] - m);
      l = warp_sum(l);
      const float inv = 1.0f / l;
      for (int s = lane; s < n_splits; s += 32) e[2 * s] = e[2 * s + 1] > 0.f ? expf(e[2 * s] - m) * inv : 0.f;
    }
    __syncthreads();
    for (int idx = tid; idx < G * HD; idx += FD_NT) {
      const int hg = idx / HD, d = idx % HD;
      const size_t th = (size_t)t * H + (size_t)g * G + hg;
      const float* e = sh + (size_t)2 * hg * n_splits;
      const float* po = part_o + th * n_splits * HD + d;
      float acc = 0.f;
      int s = 0;
      for (; s + 8 <= n_splits; s += 8) {
        float v[8];
#pragma unroll
        for (int u = 0; u < 8; u++) v[u] = __ldcg(po + (size_t)(s + u) * HD);
#pragma unroll
        for (int u = 0; u < 8; u++) { const float w = e[2 * (s + u)]; acc = w != 0.f ? fmaf(v[u], w, acc) : acc; }
      }
      for (; s < n_splits; s++) { const float w = e[2 * s]; const float v = __ldcg(po + (size_t)s * HD); acc = w != 0.f ? fmaf(v, w, acc) : acc; }
      out[th * HD + d] = __float2bfloat16_rn(acc);
    }
    return;
  }
  // more splits than shared memory holds statistics for: one head after the other from global memory
  for (int hg = 0; hg < G; hg++) {
    const size_t th = (size_t)t * H + (size_t)g * G + hg;
    const float* mlh = part_ml + th * n_splits * 2;
    float m = -INFINITY;
    for (int s = 0; s < n_splits; s++) m = fmaxf(m, __ldcg(mlh + 2 * s));
    float l = 0.f;
    for (int s = 0; s < n_splits; s++) {
      const float ls = __ldcg(mlh + 2 * s + 1);
      if (ls > 0.f) l += ls * expf(__ldcg(mlh + 2 * s) - m);
    }
    const float inv = 1.0f / l;
    for (int d = tid; d < HD; d += FD_NT) {
      float acc = 0.f;
      for (int s = 0; s < n_splits; s++)
        if (__ldcg(mlh + 2 * s + 1) > 0.f)
          acc = fmaf(__ldcg(part_o + (th * n_splits + s) * HD + d), expf(__ldcg(mlh + 2 * s) - m), acc);
      out[th * HD + d] = __float2bfloat16_rn(acc * inv);
    }
  }
}

static int bound_of(int G) { return G <= 1 ? 1 : G <= 2 ? 2 : G <= 4 ? 4 : 8; }

static size_t fused_smem(int G, int hd, int keys) {
  return ((size_t)G * hd + (size_t)G * keys + (size_t)FD_NW * bound_of(G) + (size_t)FD_NW * G * hd) * sizeof(float) +
         2 * (size_t)hd * sizeof(__nv_bfloat16);
}

// 1 if the fused kernel takes these sizes (the caller falls back to the separate kernels otherwise)
extern "C" int tlc_attention_decode_fused_ok(int H, int KV, int hd) {
  if (KV <= 0 || H % KV != 0 || H / KV > FD_MAXG || KV > 65535) return 0;
  if (hd != 64 && hd != 128 && hd != 256) return 0;
  return fused_smem(H / KV, hd, 256) <= 200 * 1024;
}

template <int HD, int GT, int KEYS, typename... Args>
static cudaError_t launch_fused(dim3 grid, size_t smem, cudaStream_t stream, Args... args) {
  static bool raised[64] = {};          // per device: the kernel may use more than 48 KB of shared memory
  int dev = 0;
  cudaGetDevice(&dev);
  if (smem > 48 * 1024 && dev >= 0 && dev < 64 && !raised[dev]) {
    cudaError_t e = cudaFuncSetAttribute(attention_decode_fused_kernel<HD, GT, KEYS>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    if (e != cudaSuccess) return e;
    raised[dev] = true;
  }
  return tlc_launch(attention_decode_fused_kernel<HD, GT, KEYS>, grid, dim3(FD_NT), smem, stream, args...);
}

// qkv: float32 rows of `ld` elements with the queries, keys and values of the row at q_off, k_off,
// v_off.  scratch: part_o [T, H, n_splits, hd], part_ml [T, H, n_splits, 2] floats with
// n_splits = ceil(max_keys / 128); arrivals: T * KV counters, zero before the first call.
extern "C" int tlc_attention_decode_fused(const float* qkv, int ld, int q_off, int k_off, int v_off, void* k_pages,
                                          void* v_pages, const float* inv_freq, int rope_dim, int write_kv,
                                          const int* block_table, int max_pages, const int* positions,
                                          const int* row_seq, const int* slots, void* out, float* part_o, float* part_ml,
                                          unsigned* arrivals, int T, int H, int KV, int hd, float scale, int window,
                                          int max_keys, cudaStream_t stream) {
  if (T == 0) return 0;
  TLC_REQUIRE(tlc_attention_decode_fused_ok(H, KV, hd), "attention(decode, fused): %d heads, %d key/value heads of size %d are outside the kernel's range", H, KV, hd);
  TLC_REQUIRE(rope_dim % 2 == 0 && rope_dim >= 0 && rope_dim <= hd, "attention(decode, fused): rotated width %d must be even and at most head_dim %d", rope_dim, hd);
  // 128 keys a block while that keeps the grid within about one wave (two blocks an SM), else 256
  int sms = 148, dev = 0;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const long long blocks128 = (long long)T * KV * ((max_keys + 127) / 128);
  const int keys = blocks128 > 2LL * sms ? 256 : 128;
  const int n_splits = (max_keys + keys - 1) / keys;
  TLC_REQUIRE(n_splits >= 1 && n_splits <= 65535, "attention(decode, fused): %d keys are outside the kernel's range", max_keys);
  const size_t smem = fused_smem(H / KV, hd, keys);
  dim3 grid(T, KV, n_splits);
  __nv_bfloat16 *kp = (__nv_bfloat16*)k_pages, *vp = (__nv_bfloat16*)v_pages, *op = (__nv_bfloat16*)out;
  cudaError_t e = cudaSuccess;
#define TLC_FD_LAUNCH(HDV, GTV, KV_)                                                                                    \
  e = launch_fused<HDV, GTV, KV_>(grid, smem, stream, qkv, ld, q_off, k_off, v_off, kp, vp, inv_freq, rope_dim, write_kv, \
                                  block_table, max_pages, positions, row_seq, slots, part_o, part_ml, arrivals, op, H,  \
                                  KV, scale, window, n_splits)
#define TLC_FD_GROUP(HDV, KV_)                                            \
  do {                                                                    \
    switch (bound_of(H / KV)) {                                           \
      case 1: TLC_FD_LAUNCH(HDV, 1, KV_); break;                          \
      case 2: TLC_FD_LAUNCH(HDV, 2, KV_); break;                          \
      case 4: TLC_FD_LAUNCH(HDV, 4, KV_); break;                          \
      default: TLC_FD_LAUNCH(HDV, 8, KV_); break;                         \
    }                                                                     \
  } while (0)
#define TLC_FD_HEAD(HDV)                                                  \
  do { if (keys == 128) TLC_FD_GROUP(HDV, 128); else TLC_FD_GROUP(HDV, 256); } while (0)
  if (hd == 64) TLC_FD_HEAD(64);
  else if (hd == 128) TLC_FD_HEAD(128);
  else TLC_FD_HEAD(256);
#undef TLC_FD_HEAD
#undef TLC_FD_GROUP
#undef TLC_FD_LAUNCH
  if (e != cudaSuccess) return tlc_fail(-2, "attention(decode, fused): %s", cudaGetErrorString(e));
  TLC_CHECK_LAUNCH("attention(decode, fused)");
  return 0;
}
