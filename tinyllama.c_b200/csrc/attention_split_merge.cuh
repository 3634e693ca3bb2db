// The merge of the splits of single-token attention, run by the last block of a (row, key/value
// head) to finish: softmax statistics (maximum, sum) and unnormalised partial outputs of every
// split become the normalised output (CodeClaper/tinyllama.c cpu_op.c:1010-1062 computes the same softmax
// in one piece).  All in 32-bit.
#pragma once
#include "common.cuh"

// part_o [T, H, n_splits, HD], part_ml [T, H, n_splits, 2]; out: rows of out_ld elements, head h at h * HD;
// sh: the block's dynamic shared memory of smem_floats floats (free by now); NT threads.  All threads of
// the block call it.
template <int HD, int NT>
__device__ __forceinline__ void attention_merge_splits(const float* part_o, const float* part_ml, __nv_bfloat16* out,
                                                       float* sh, int smem_floats, int t, int g, int G, int H,
                                                       int n_splits, int out_ld) {
  const int tid = threadIdx.x, lane = tid & 31, wp = tid >> 5;
  constexpr int NW = NT / 32;
  if (2 * G * n_splits <= smem_floats) {
    // statistics of all heads and splits into shared memory (one round trip), weights from them,
    // then the weighted sum with the loads of a thread in flight together
    for (int idx = tid; idx < G * n_splits; idx += NT) {
      const int hg = idx / n_splits, s = idx % n_splits;
      const float2 v = __ldcg(reinterpret_cast<const float2*>(part_ml + (((size_t)t * H + (size_t)g * G + hg) * n_splits + s) * 2));
      sh[2 * idx] = v.x;
      sh[2 * idx + 1] = v.y;
    }
    __syncthreads();
    for (int hg = wp; hg < G; hg += NW) {
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
    for (int idx = tid; idx < G * HD; idx += NT) {
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
      out[(size_t)t * out_ld + ((size_t)g * G + hg) * HD + d] = __float2bfloat16_rn(acc);
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
    for (int d = tid; d < HD; d += NT) {
      float acc = 0.f;
      for (int s = 0; s < n_splits; s++)
        if (__ldcg(mlh + 2 * s + 1) > 0.f)
          acc = fmaf(__ldcg(part_o + (th * n_splits + s) * HD + d), expf(__ldcg(mlh + 2 * s) - m), acc);
      out[(size_t)t * out_ld + ((size_t)g * G + hg) * HD + d] = __float2bfloat16_rn(acc * inv);
    }
  }
}
