// Rotary position encoding with the key/value store, and attention over the paged cache.
//
// CodeClaper/tinyllama.c: split-half rotation of the first rope_dim dims of each head,
// theta_i = 1/base^(2i/r), angle = pos*theta_i (cpu_op.c:637-651); K/V rows written to
// the cache at their absolute position (cpu_op.c:995-1008); causal grouped-query
// attention with kv head h/(H/KV), scale 1/sqrt(head_dim), max-subtracted softmax and an
// optional window of the last w keys (cpu_op.c:1010-1062, 338-349; graph.c:1275).
//
// Here the cache is paged: a sequence's position p lives in page
// block_table[slot][p / 64] at row p % 64; a layer's pages are [page][kv head][64][hd].
// Scores, softmax statistics and the output accumulator are 32-bit.
#include "common.cuh"

// ---- rope + store -----------------------------------------------------------------------
template <typename TI, typename T>
__global__ void rope_kv_store_kernel(const TI* __restrict__ qkv, int ld, int q_off, int k_off, int v_off,
                                     T* __restrict__ q_out, T* __restrict__ k_pages, T* __restrict__ v_pages,
                                     const float* __restrict__ inv_freq, int rope_dim,
                                     const int* __restrict__ positions, const int* __restrict__ row_seq,
                                     const int* __restrict__ slots, const int* __restrict__ block_table, int max_pages,
                                     int H, int KV, int hd, int write_kv) {
  tlc_pdl(qkv, q_out, k_pages, v_pages);
  // the row's angles once: cos and sin of position * inv_freq[i], shared by all heads
  extern __shared__ float rope_cs[];                 // [half] cos | [half] sin
  const int t = blockIdx.x;
  const int pos = positions[t];
  const int half = rope_dim >> 1;
  for (int i = threadIdx.x; i < half; i += blockDim.x) sincosf((float)pos * inv_freq[i], &rope_cs[half + i], &rope_cs[i]);
  __syncthreads();
  const TI* row = qkv + (size_t)t * ld;
  const int n_heads_total = H + 2 * KV;
  int page = -1;
  if (write_kv) page = block_table[(size_t)slots[row_seq[t]] * max_pages + pos / TLC_PAGE];
  const int prow = pos % TLC_PAGE;
  for (int idx = threadIdx.x; idx < n_heads_total * hd; idx += blockDim.x) {
    const int head = idx / hd, d = idx % hd;
    const TI* src;
    int kind;  // 0 q, 1 k, 2 v
    int h;
    if (head < H) { kind = 0; h = head; src = row + q_off + (size_t)h * hd; }
    else if (head < H + KV) { kind = 1; h = head - H; src = row + k_off + (size_t)h * hd; }
    else { kind = 2; h = head - H - KV; src = row + v_off + (size_t)h * hd; }
    if (kind != 0 && !write_kv) continue;
    float v;
    if (kind == 2 || d >= rope_dim) {
      v = to_f32(src[d]);
    } else {
      const int i = d < half ? d : d - half;
      const float cs = rope_cs[i], sn = rope_cs[half + i];
      const float a = to_f32(src[i]), b = to_f32(src[i + half]);
      v = d < half ? a * cs - b * sn : a * sn + b * cs;
    }
    if (kind == 0) {
      q_out[(size_t)t * H * hd + (size_t)h * hd + d] = from_f32<T>(v);
    } else if (page >= 0) {
      T* dst = (kind == 1 ? k_pages : v_pages) + (((size_t)page * KV + h) * TLC_PAGE + prow) * hd + d;
      *dst = from_f32<T>(v);
    }
  }
}

// The same for 32-bit projections whose pieces all lie on 16-byte boundaries (rotated width a multiple of 8, head
// size and offsets multiples of 4): a block takes ROPE_ROWS rows; a thread takes four consecutive dims of a
// head's lower half with their partners in the upper half (two 16-byte loads, two stores), or four dims that
// are only copied (values, dims beyond the rotated width).
#define ROPE_ROWS 4
template <typename T> struct Put4;
template <> struct Put4<float> {
  static __device__ __forceinline__ void put(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
};
template <> struct Put4<__nv_bfloat16> {
  static __device__ __forceinline__ void put(__nv_bfloat16* p, float4 v) {
    __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
    uint2 u;
    u.x = *reinterpret_cast<unsigned*>(&lo);
    u.y = *reinterpret_cast<unsigned*>(&hi);
    *reinterpret_cast<uint2*>(p) = u;
  }
};
template <typename T>
__global__ void __launch_bounds__(256)
rope_kv_store_vec_kernel(const float* __restrict__ qkv, int ld, int q_off, int k_off, int v_off, T* __restrict__ q_out,
                         T* __restrict__ k_pages, T* __restrict__ v_pages, const float* __restrict__ inv_freq,
                         int rope_dim, const int* __restrict__ positions, const int* __restrict__ row_seq,
                         const int* __restrict__ slots, const int* __restrict__ block_table, int max_pages, int n_rows,
                         int H, int KV, int hd, int write_kv) {
  tlc_pdl(qkv, q_out, k_pages, v_pages);
  extern __shared__ float rope_cs[];                 // per row: [half] cos | [half] sin
  __shared__ int s_page[ROPE_ROWS], s_prow[ROPE_ROWS];
  const int t0 = blockIdx.x * ROPE_ROWS;
  const int rows = min(ROPE_ROWS, n_rows - t0);
  const int half = rope_dim >> 1;
  if (threadIdx.x < rows) {
    const int t = t0 + threadIdx.x, pos = positions[t];
    s_page[threadIdx.x] = write_kv ? block_table[(size_t)slots[row_seq[t]] * max_pages + pos / TLC_PAGE] : -1;
    s_prow[threadIdx.x] = pos % TLC_PAGE;
  }
  for (int i = threadIdx.x; i < rows * half; i += blockDim.x) {
    const int r = i / half, j = i - r * half;
    sincosf((float)positions[t0 + r] * inv_freq[j], &rope_cs[r * rope_dim + half + j], &rope_cs[r * rope_dim + j]);
  }
  __syncthreads();
  const int pair_items = half >> 2, tail_items = (hd - rope_dim) >> 2;
  const int per_head = pair_items + tail_items;          // items of a rotated head
  const int n_rot = write_kv ? H + KV : H;               // heads that are rotated (queries, keys)
  const int per_row = n_rot * per_head + (write_kv ? KV * (hd >> 2) : 0);
  for (int idx = threadIdx.x; idx < rows * per_row; idx += blockDim.x) {
    const int r = idx / per_row, it = idx - r * per_row;
    const int t = t0 + r;
    const float* row = qkv + (size_t)t * ld;
    const float* cs = rope_cs + r * rope_dim;
    if (it < n_rot * per_head) {
      const int head = it / per_head, j = it - head * per_head;
      const bool is_q = head < H;
      const int h = is_q ? head : head - H;
      const float* src = row + (is_q ? q_off : k_off) + (size_t)h * hd;
      T* dst = is_q ? q_out + (size_t)t * H * hd + (size_t)h * hd
                    : k_pages + (((size_t)s_page[r] * KV + h) * TLC_PAGE + s_prow[r]) * hd;
      if (j < pair_items) {
        const int d = 4 * j;
        const float4 a = *reinterpret_cast<const float4*>(src + d), b = *reinterpret_cast<const float4*>(src + half + d);
        const float4 c = *reinterpret_cast<const float4*>(cs + d), sn = *reinterpret_cast<const float4*>(cs + half + d);
        Put4<T>::put(dst + d, make_float4(a.x * c.x - b.x * sn.x, a.y * c.y - b.y * sn.y, a.z * c.z - b.z * sn.z, a.w * c.w - b.w * sn.w));
        Put4<T>::put(dst + half + d, make_float4(a.x * sn.x + b.x * c.x, a.y * sn.y + b.y * c.y, a.z * sn.z + b.z * c.z, a.w * sn.w + b.w * c.w));
      } else {
        const int d = rope_dim + 4 * (j - pair_items);
        Put4<T>::put(dst + d, *reinterpret_cast<const float4*>(src + d));
      }
    } else {
      const int iv = it - n_rot * per_head;
      const int h = iv / (hd >> 2), d = 4 * (iv - h * (hd >> 2));
      Put4<T>::put(v_pages + (((size_t)s_page[r] * KV + h) * TLC_PAGE + s_prow[r]) * hd + d,
                   *reinterpret_cast<const float4*>(row + v_off + (size_t)h * hd + d));
    }
  }
}

extern "C" int tlc_rope_kv_store(const void* qkv, int in_dtype, int dtype, int ld, int q_off, int k_off, int v_off, void* q_out,
                                 void* k_pages, void* v_pages, const float* inv_freq, int rope_dim,
                                 const int* positions, const int* row_seq, const int* slots, const int* block_table,
                                 int max_pages, int T, int H, int KV, int hd, int write_kv, cudaStream_t stream) {
  if (T == 0) return 0;
  TLC_REQUIRE(rope_dim % 2 == 0 && rope_dim <= hd, "rope: rotated width %d must be even and at most head_dim %d", rope_dim, hd);
  if (in_dtype == TLC_F32 && rope_dim % 8 == 0 && hd % 4 == 0 && ld % 4 == 0 && q_off % 4 == 0 && k_off % 4 == 0 && v_off % 4 == 0 &&
      ((uintptr_t)qkv % 16) == 0 && ((uintptr_t)q_out % 16) == 0 && ((uintptr_t)k_pages % 16) == 0 && ((uintptr_t)v_pages % 16) == 0 &&
      (size_t)ROPE_ROWS * rope_dim * sizeof(float) <= 40 * 1024) {
    const dim3 grid((T + ROPE_ROWS - 1) / ROPE_ROWS);
    const size_t smem = (size_t)ROPE_ROWS * rope_dim * sizeof(float);
    TLC_DISPATCH_DTYPE(dtype, TT, tlc_launch(rope_kv_store_vec_kernel<TT>, dim3(grid), dim3(256), smem, stream, (const float*)qkv, ld,
        q_off, k_off, v_off, (TT*)q_out, (TT*)k_pages, (TT*)v_pages, inv_freq, rope_dim, positions, row_seq, slots, block_table,
        max_pages, T, H, KV, hd, write_kv));
    TLC_CHECK_LAUNCH("rope_kv_store");
    return 0;
  }
  TLC_DISPATCH_DTYPE(in_dtype, TI, TLC_DISPATCH_DTYPE(dtype, TT, tlc_launch(rope_kv_store_kernel<TI, TT>, dim3(T), dim3(256), (size_t)rope_dim * sizeof(float), stream, 
      (const TI*)qkv, ld, q_off, k_off, v_off, (TT*)q_out, (TT*)k_pages, (TT*)v_pages, inv_freq, rope_dim, positions,
      row_seq, slots, block_table, max_pages, H, KV, hd, write_kv)));
  TLC_CHECK_LAUNCH("rope_kv_store");
  return 0;
}

// ---- attention, one warp per (query row, head) ----------------------------------------------
// Streams the keys 32 at a time: lane j scores key k0+j, the warp keeps a running maximum
// and sum, and every lane owns the output dims lane, lane+32, ...  Any head size up to
// 32*MAXD, any number of heads and groups.
#define ATT_MAXD 8
template <typename T>
__global__ void __launch_bounds__(128)
attention_warp_kernel(const T* __restrict__ q, const T* __restrict__ k_pages, const T* __restrict__ v_pages,
                      const int* __restrict__ block_table, int max_pages, const int* __restrict__ positions,
                      const int* __restrict__ row_seq, const int* __restrict__ slots, T* __restrict__ out, int H, int KV,
                      int hd, float scale, int window, int out_ld) {
  tlc_pdl(q, k_pages, v_pages, out);
  extern __shared__ float qs_all[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x;
  const int h = blockIdx.y * 4 + warp;
  if (h >= H) return;
  float* qs = qs_all + (size_t)warp * hd;
  const int g = h / (H / KV);
  const int pos = positions[t];
  const int* table = block_table + (size_t)slots[row_seq[t]] * max_pages;
  const T* qr = q + ((size_t)t * H + h) * hd;
  for (int d = lane; d < hd; d += 32) qs[d] = to_f32(qr[d]) * scale;
  __syncwarp();
  const int n_keys = pos + 1;
  const int start = (window > 0 && n_keys > window) ? n_keys - window : 0;
  float m = -INFINITY, l = 0.f;
  float acc[ATT_MAXD];
#pragma unroll
  for (int i = 0; i < ATT_MAXD; i++) acc[i] = 0.f;
  for (int k0 = start; k0 < n_keys; k0 += 32) {
    const int kp = k0 + lane;
    float s = -INFINITY;
    if (kp < n_keys) {
      const int page = table[kp / TLC_PAGE];
      const T* kr = k_pages + (((size_t)page * KV + g) * TLC_PAGE + kp % TLC_PAGE) * hd;
      float dot = 0.f;
      for (int d = 0; d < hd; d++) dot = fmaf(to_f32(kr[d]), qs[d], dot);
      s = dot;
    }
    const float m_new = fmaxf(m, warp_max(s));
    const float p = kp < n_keys ? expf(s - m_new) : 0.f;
    const float corr = expf(m - m_new);      // exp(-inf) = 0 on the first chunk
    l = l * corr + warp_sum(p);
#pragma unroll
    for (int i = 0; i < ATT_MAXD; i++) acc[i] *= corr;
    const int nk = min(32, n_keys - k0);
    for (int j = 0; j < nk; j++) {
      const float pj = __shfl_sync(0xffffffffu, p, j);
      const int kj = k0 + j;
      const int page = table[kj / TLC_PAGE];
      const T* vr = v_pages + (((size_t)page * KV + g) * TLC_PAGE + kj % TLC_PAGE) * hd;
#pragma unroll
      for (int i = 0; i < ATT_MAXD; i++) {
        const int d = lane + 32 * i;
        if (d < hd) acc[i] = fmaf(pj, to_f32(vr[d]), acc[i]);
      }
    }
    m = m_new;
  }
  const float inv = 1.0f / l;
  T* o = out + (size_t)t * out_ld + (size_t)h * hd;
#pragma unroll
  for (int i = 0; i < ATT_MAXD; i++) {
    const int d = lane + 32 * i;
    if (d < hd) o[d] = from_f32<T>(acc[i] * inv);
  }
}

extern "C" int tlc_attention(const void* q, int dtype, const void* k_pages, const void* v_pages,
                             const int* block_table, int max_pages, const int* positions, const int* row_seq,
                             const int* slots, void* out, int T, int H, int KV, int hd, float scale, int window,
                             int out_ld, cudaStream_t stream) {
  if (T == 0) return 0;
  if (out_ld <= 0) out_ld = H * hd;                      // elements between rows of out (0: dense)
  TLC_REQUIRE(KV > 0 && H % KV == 0, "attention: %d heads are not a multiple of %d key/value heads", H, KV);
  TLC_REQUIRE(hd <= 32 * ATT_MAXD, "attention: head size %d exceeds the kernel's limit of %d", hd, 32 * ATT_MAXD);
  dim3 grid(T, (H + 3) / 4);
  const size_t smem = (size_t)4 * hd * sizeof(float);
  TLC_DISPATCH_DTYPE(dtype, TT, tlc_launch(attention_warp_kernel<TT>, dim3(grid), dim3(128), smem, stream, 
      (const TT*)q, (const TT*)k_pages, (const TT*)v_pages, block_table, max_pages, positions, row_seq, slots, (TT*)out,
      H, KV, hd, scale, window, out_ld));
  TLC_CHECK_LAUNCH("attention");
  return 0;
}

// ---- attention for one-token steps: keys split across blocks ------------------------------------
// A decode step has one query row per sequence and hundreds or thousands of keys.  The grid is
// (row, kv head, split): a block scores 128 keys of its sequence for all query heads that share
// the kv head (keys and values are read once per group), and writes an unnormalised partial
// output with its running maximum and sum; a second kernel merges the splits.  The split count
// of the grid is an upper bound from the host; a block whose keys lie past the row's length or
// before its window exits at once, so the same launch serves any lengths (and a captured graph).
#define DEC_KEYS 128
#define DEC_MAXG 8
template <typename T>
__global__ void __launch_bounds__(DEC_KEYS)
attention_decode_partial_kernel(const T* __restrict__ q, const T* __restrict__ k_pages, const T* __restrict__ v_pages,
                                const int* __restrict__ block_table, int max_pages, const int* __restrict__ positions,
                                const int* __restrict__ row_seq, const int* __restrict__ slots, float* __restrict__ part_o,
                                float* __restrict__ part_ml, int H, int KV, int hd, float scale, int window, int n_splits) {
  tlc_pdl(q, k_pages, v_pages, part_o, part_ml);
  extern __shared__ float sh[];
  const int t = blockIdx.x, g = blockIdx.y, split = blockIdx.z;
  const int G = H / KV;
  const int pos = positions[t];
  const int n_keys = pos + 1;
  const int start = (window > 0 && n_keys > window) ? n_keys - window : 0;
  const int k0 = split * DEC_KEYS;
  float* ml = part_ml + (((size_t)t * H + (size_t)g * G) * n_splits + split) * 2;   // + hg * n_splits * 2
  if (k0 >= n_keys || k0 + DEC_KEYS <= start) {
    if (threadIdx.x < G) { ml[(size_t)threadIdx.x * n_splits * 2] = -INFINITY; ml[(size_t)threadIdx.x * n_splits * 2 + 1] = 0.f; }
    return;
  }
  float* qs = sh;                          // [G][hd]
  float* ps = sh + (size_t)G * hd;         // [G][DEC_KEYS]
  float* red = ps + (size_t)G * DEC_KEYS;  // [33]
  const int* table = block_table + (size_t)slots[row_seq[t]] * max_pages;
  for (int i = threadIdx.x; i < G * hd; i += blockDim.x)
    qs[i] = to_f32(q[((size_t)t * H + (size_t)g * G) * hd + i]) * scale;
  __syncthreads();
  const int kp = k0 + threadIdx.x;
  const bool valid = kp >= start && kp < n_keys;
  float s[DEC_MAXG];
#pragma unroll
  for (int hg = 0; hg < DEC_MAXG; hg++) s[hg] = 0.f;
  if (valid) {
    const T* kr = k_pages + (((size_t)table[kp / TLC_PAGE] * KV + g) * TLC_PAGE + kp % TLC_PAGE) * hd;
    for (int d = 0; d < hd; d++) {
      const float kv = to_f32(kr[d]);
#pragma unroll
      for (int hg = 0; hg < DEC_MAXG; hg++)
        if (hg < G) s[hg] = fmaf(kv, qs[hg * hd + d], s[hg]);
    }
  }
  // per head: maximum and sum over the block's keys
  for (int hg = 0; hg < G; hg++) {
    const float sv = valid ? s[hg] : -INFINITY;
    float m = warp_max(sv);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = m;
    __syncthreads();
    m = fmaxf(fmaxf(red[0], red[1]), fmaxf(red[2], red[3]));
    const float p = valid ? expf(sv - m) : 0.f;
    ps[hg * DEC_KEYS + threadIdx.x] = p;
    const float l = block_sum(p, red);
    if (threadIdx.x == 0) { ml[(size_t)hg * n_splits * 2] = m; ml[(size_t)hg * n_splits * 2 + 1] = l; }
  }
  __syncthreads();
  const int nk = min(DEC_KEYS, n_keys - k0);
  for (int d = threadIdx.x; d < hd; d += blockDim.x) {
    float acc[DEC_MAXG];
#pragma unroll
    for (int hg = 0; hg < DEC_MAXG; hg++) acc[hg] = 0.f;
    for (int j = 0; j < nk; j++) {
      const int kj = k0 + j;
      if (kj < start) continue;            // outside the window: its page may have been given back
      const float vv = to_f32(v_pages[(((size_t)table[kj / TLC_PAGE] * KV + g) * TLC_PAGE + kj % TLC_PAGE) * hd + d]);
#pragma unroll
      for (int hg = 0; hg < DEC_MAXG; hg++)
        if (hg < G) acc[hg] = fmaf(ps[hg * DEC_KEYS + j], vv, acc[hg]);
    }
#pragma unroll
    for (int hg = 0; hg < DEC_MAXG; hg++)
      if (hg < G) part_o[((((size_t)t * H + (size_t)g * G + hg) * n_splits) + split) * hd + d] = acc[hg];
  }
}

// bfloat16 with a head size of 64, 128 or 256: 16-byte loads.  Scoring: a thread per key reads
// its key row in 16-byte pieces.  Values: hd/8 lanes cover a value row, 128/(hd/8) keys are
// in flight at a time, and the groups' partial outputs meet in shared memory.
template <int HD>
__global__ void __launch_bounds__(DEC_KEYS)
attention_decode_partial_vec_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k_pages,
                                    const __nv_bfloat16* __restrict__ v_pages, const int* __restrict__ block_table,
                                    int max_pages, const int* __restrict__ positions, const int* __restrict__ row_seq,
                                    const int* __restrict__ slots, float* __restrict__ part_o,
                                    float* __restrict__ part_ml, int H, int KV, float scale, int window, int n_splits) {
  // Keys of earlier positions were stored by earlier steps; only the row at the query's own
  // position is written by the kernel before this one.  Everything else is fetched before the
  // wait on that kernel (see tlc_pdl).
  asm volatile("griddepcontrol.launch_dependents;");
  extern __shared__ float sh[];
  constexpr int DL = HD / 8;                 // lanes per value row
  constexpr int GROUPS = DEC_KEYS / DL;      // value rows in flight
  const int t = blockIdx.x, g = blockIdx.y, split = blockIdx.z;
  const int G = H / KV;
  const int pos = positions[t];
  const int n_keys = pos + 1;
  const int start = (window > 0 && n_keys > window) ? n_keys - window : 0;
  const int k0 = split * DEC_KEYS;
  float* ml = part_ml + (((size_t)t * H + (size_t)g * G) * n_splits + split) * 2;
  if (k0 >= n_keys || k0 + DEC_KEYS <= start) {
    tlc_wait(ml);
    if (threadIdx.x < G) { ml[(size_t)threadIdx.x * n_splits * 2] = -INFINITY; ml[(size_t)threadIdx.x * n_splits * 2 + 1] = 0.f; }
    return;
  }
  float* qs = sh;                                   // [G][HD]
  float* ps = qs + (size_t)G * HD;                  // [G][DEC_KEYS]
  float* red = ps + (size_t)G * DEC_KEYS;           // [36]
  float* os = red + 36;                             // [GROUPS][G][HD]
  __shared__ int pages[DEC_KEYS / TLC_PAGE + 1];
  const int* table = block_table + (size_t)slots[row_seq[t]] * max_pages;
  const int kp = k0 + threadIdx.x;
  const bool valid = kp >= start && kp < n_keys;
  uint4 kq[DL];
  const uint4* kr = nullptr;
  if (valid) {
    kr = reinterpret_cast<const uint4*>(k_pages + (((size_t)table[kp / TLC_PAGE] * KV + g) * TLC_PAGE + kp % TLC_PAGE) * HD);
    if (kp != pos) {
#pragma unroll
      for (int d8 = 0; d8 < DL; d8++) kq[d8] = __ldg(kr + d8);
    }
  }
  if (threadIdx.x <= DEC_KEYS / TLC_PAGE) {
    const int pi = k0 / TLC_PAGE + threadIdx.x;
    pages[threadIdx.x] = (pi * TLC_PAGE < n_keys) ? table[pi] : 0;
  }
  tlc_wait(q, kr, v_pages, part_o, ml);     // the row at the query's own position is new: kr, v_pages
  if (valid && kp == pos) {
#pragma unroll
    for (int d8 = 0; d8 < DL; d8++) kq[d8] = kr[d8];
  }
  for (int i = threadIdx.x; i < G * HD; i += blockDim.x)
    qs[i] = __bfloat162float(q[((size_t)t * H + (size_t)g * G) * HD + i]) * scale;
  __syncthreads();
  float s[DEC_MAXG];
#pragma unroll
  for (int hg = 0; hg < DEC_MAXG; hg++) s[hg] = 0.f;
  if (valid) {
#pragma unroll
    for (int d8 = 0; d8 < DL; d8++) {
      const __nv_bfloat162* kb = reinterpret_cast<const __nv_bfloat162*>(&kq[d8]);
      float kf[8];
#pragma unroll
      for (int i = 0; i < 4; i++) { const float2 f = __bfloat1622float2(kb[i]); kf[2 * i] = f.x; kf[2 * i + 1] = f.y; }
#pragma unroll
      for (int hg = 0; hg < DEC_MAXG; hg++) {
        if (hg < G) {
          const float4 qa = *reinterpret_cast<const float4*>(qs + hg * HD + d8 * 8);
          const float4 qb = *reinterpret_cast<const float4*>(qs + hg * HD + d8 * 8 + 4);
          s[hg] = fmaf(kf[0], qa.x, s[hg]); s[hg] = fmaf(kf[1], qa.y, s[hg]);
          s[hg] = fmaf(kf[2], qa.z, s[hg]); s[hg] = fmaf(kf[3], qa.w, s[hg]);
          s[hg] = fmaf(kf[4], qb.x, s[hg]); s[hg] = fmaf(kf[5], qb.y, s[hg]);
          s[hg] = fmaf(kf[6], qb.z, s[hg]); s[hg] = fmaf(kf[7], qb.w, s[hg]);
        }
      }
    }
  }
  // maximum and sum over the block's keys, all heads of the group at once
  {
    float* redm = red;                        // [4 warps][DEC_MAXG]
    const int wp = threadIdx.x >> 5, ln = threadIdx.x & 31;
#pragma unroll
    for (int hg = 0; hg < DEC_MAXG; hg++) {
      if (hg < G) {
        const float m = warp_max(valid ? s[hg] : -INFINITY);
        if (ln == 0) redm[wp * DEC_MAXG + hg] = m;
      }
    }
    __syncthreads();
    float lsum[DEC_MAXG];
#pragma unroll
    for (int hg = 0; hg < DEC_MAXG; hg++) {
      if (hg < G) {
        const float m = fmaxf(fmaxf(redm[hg], redm[DEC_MAXG + hg]), fmaxf(redm[2 * DEC_MAXG + hg], redm[3 * DEC_MAXG + hg]));
        const float p = valid ? expf(s[hg] - m) : 0.f;
        ps[hg * DEC_KEYS + threadIdx.x] = p;
        lsum[hg] = warp_sum(p);
        s[hg] = m;
      }
    }
    __syncthreads();
#pragma unroll
    for (int hg = 0; hg < DEC_MAXG; hg++)
      if (hg < G && ln == 0) redm[wp * DEC_MAXG + hg] = lsum[hg];
    __syncthreads();
    if (threadIdx.x < G) {
      const int hg = threadIdx.x;
      float mm = -INFINITY;
#pragma unroll
      for (int i = 0; i < DEC_MAXG; i++) if (i == hg) mm = s[i];
      ml[(size_t)hg * n_splits * 2] = mm;
      ml[(size_t)hg * n_splits * 2 + 1] = redm[hg] + redm[DEC_MAXG + hg] + redm[2 * DEC_MAXG + hg] + redm[3 * DEC_MAXG + hg];
    }
  }
  __syncthreads();
  const int nk = min(DEC_KEYS, n_keys - k0);
  const int dl = threadIdx.x % DL, grp = threadIdx.x / DL;
  float acc[DEC_MAXG][8];
#pragma unroll
  for (int hg = 0; hg < DEC_MAXG; hg++)
#pragma unroll
    for (int i = 0; i < 8; i++) acc[hg][i] = 0.f;
  // value rows of this thread's group, 16 at a time: all loads are issued before the first use
  constexpr int VB = DL < 16 ? DL : 16;
#pragma unroll 1
  for (int jb = 0; jb < DL; jb += VB) {
    uint4 vq[VB];
#pragma unroll
    for (int u = 0; u < VB; u++) {
      const int j = grp + (jb + u) * GROUPS;
      const int kj = k0 + j;
      const bool use = j < nk && kj >= start;          // outside the window a page may have been given back
      vq[u] = use ? __ldg(reinterpret_cast<const uint4*>(
                              v_pages + (((size_t)pages[j / TLC_PAGE] * KV + g) * TLC_PAGE + kj % TLC_PAGE) * HD) + dl)
                  : make_uint4(0, 0, 0, 0);
    }
#pragma unroll
    for (int u = 0; u < VB; u++) {
      const int j = grp + (jb + u) * GROUPS;
      if (j >= nk) continue;
      const __nv_bfloat162* vb = reinterpret_cast<const __nv_bfloat162*>(&vq[u]);
      float vf[8];
#pragma unroll
      for (int i = 0; i < 4; i++) { const float2 f = __bfloat1622float2(vb[i]); vf[2 * i] = f.x; vf[2 * i + 1] = f.y; }
#pragma unroll
      for (int hg = 0; hg < DEC_MAXG; hg++) {
        if (hg < G) {
          const float p = ps[hg * DEC_KEYS + j];
#pragma unroll
          for (int i = 0; i < 8; i++) acc[hg][i] = fmaf(p, vf[i], acc[hg][i]);
        }
      }
    }
  }
#pragma unroll
  for (int hg = 0; hg < DEC_MAXG; hg++)
    if (hg < G)
#pragma unroll
      for (int i = 0; i < 8; i++) os[((size_t)grp * G + hg) * HD + dl * 8 + i] = acc[hg][i];
  __syncthreads();
  for (int idx = threadIdx.x; idx < G * HD; idx += blockDim.x) {
    float v = 0.f;
#pragma unroll
    for (int gr = 0; gr < GROUPS; gr++) v += os[(size_t)gr * G * HD + idx];
    const int hg = idx / HD, d = idx % HD;
    part_o[((((size_t)t * H + (size_t)g * G + hg) * n_splits) + split) * HD + d] = v;
  }
}

template <typename T>
__global__ void attention_decode_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                              T* __restrict__ out, int hd, int n_splits, int H, int out_ld) {
  tlc_pdl(part_o, part_ml, out);
  const size_t th = blockIdx.x;                       // row * H + head
  T* orow = out + (th / H) * (size_t)out_ld + (th % H) * (size_t)hd;
  const float* ml = part_ml + th * n_splits * 2;
  float m = -INFINITY;
  for (int s = 0; s < n_splits; s++) m = fmaxf(m, ml[2 * s]);
  float l = 0.f;
  for (int s = 0; s < n_splits; s++) if (ml[2 * s + 1] > 0.f) l += ml[2 * s + 1] * expf(ml[2 * s] - m);
  const float inv = 1.0f / l;
  for (int d = threadIdx.x; d < hd; d += blockDim.x) {
    float acc = 0.f;
    for (int s = 0; s < n_splits; s++)
      if (ml[2 * s + 1] > 0.f) acc = fmaf(part_o[(th * n_splits + s) * hd + d], expf(ml[2 * s] - m), acc);
    orow[d] = from_f32<T>(acc * inv);
  }
}

// scratch: part_o [T, H, n_splits, hd] and part_ml [T, H, n_splits, 2] floats, n_splits = ceil(max_keys / 128)
extern "C" int tlc_attention_decode(const void* q, int dtype, const void* k_pages, const void* v_pages,
                                    const int* block_table, int max_pages, const int* positions, const int* row_seq,
                                    const int* slots, void* out, float* part_o, float* part_ml, int T, int H, int KV,
                                    int hd, float scale, int window, int max_keys, int out_ld, cudaStream_t stream) {
  if (T == 0) return 0;
  if (out_ld <= 0) out_ld = H * hd;                      // elements between rows of out (0: dense)
  TLC_REQUIRE(KV > 0 && H % KV == 0, "attention: %d heads are not a multiple of %d key/value heads", H, KV);
  TLC_REQUIRE(H / KV <= DEC_MAXG, "attention(decode): %d query heads per key/value head exceed the kernel's limit of %d", H / KV, DEC_MAXG);
  TLC_REQUIRE(KV <= 65535, "attention(decode): too many key/value heads (%d)", KV);
  const int n_splits = (max_keys + DEC_KEYS - 1) / DEC_KEYS;
  TLC_REQUIRE(n_splits >= 1 && n_splits <= 65535, "attention(decode): %d keys are outside the kernel's range", max_keys);
  const int G = H / KV;
  const size_t smem = ((size_t)G * hd + (size_t)G * DEC_KEYS + 33) * sizeof(float);
  TLC_REQUIRE(smem <= 48 * 1024, "attention(decode): head size %d with %d heads per group needs too much shared memory", hd, G);
  dim3 grid(T, KV, n_splits);
  if (dtype == TLC_BF16 && (hd == 64 || hd == 128 || hd == 256)) {
    const size_t vsmem = ((size_t)G * hd + (size_t)G * DEC_KEYS + 36 + (size_t)(DEC_KEYS / (hd / 8)) * G * hd) * sizeof(float);
    if (vsmem <= 48 * 1024) {
      const __nv_bfloat16 *qp = (const __nv_bfloat16*)q, *kp = (const __nv_bfloat16*)k_pages, *vp = (const __nv_bfloat16*)v_pages;
      if (hd == 64)
        tlc_launch(attention_decode_partial_vec_kernel<64>, dim3(grid), dim3(DEC_KEYS), vsmem, stream, qp, kp, vp, block_table, max_pages, positions, row_seq, slots, part_o, part_ml, H, KV, scale, window, n_splits);
      else if (hd == 128)
        tlc_launch(attention_decode_partial_vec_kernel<128>, dim3(grid), dim3(DEC_KEYS), vsmem, stream, qp, kp, vp, block_table, max_pages, positions, row_seq, slots, part_o, part_ml, H, KV, scale, window, n_splits);
      else
        tlc_launch(attention_decode_partial_vec_kernel<256>, dim3(grid), dim3(DEC_KEYS), vsmem, stream, qp, kp, vp, block_table, max_pages, positions, row_seq, slots, part_o, part_ml, H, KV, scale, window, n_splits);
      tlc_launch(attention_decode_merge_kernel<__nv_bfloat16>, dim3(T * H), dim3(128), 0, stream, part_o, part_ml, (__nv_bfloat16*)out, hd, n_splits, H, out_ld);
      TLC_CHECK_LAUNCH("attention(decode)");
      return 0;
    }
  }
  TLC_DISPATCH_DTYPE(dtype, TT, {
    tlc_launch(attention_decode_partial_kernel<TT>, dim3(grid), dim3(DEC_KEYS), smem, stream, 
        (const TT*)q, (const TT*)k_pages, (const TT*)v_pages, block_table, max_pages, positions, row_seq, slots, part_o,
        part_ml, H, KV, hd, scale, window, n_splits);
    tlc_launch(attention_decode_merge_kernel<TT>, dim3(T * H), dim3(128), 0, stream, part_o, part_ml, (TT*)out, hd, n_splits, H, out_ld);
  });
  TLC_CHECK_LAUNCH("attention(decode)");
  return 0;
}

// ---- single-token attention for callers that cannot allocate ---------------------------------------
// Declared in no_alloc.h (it has no counterpart in the reference).  Same kernels as
// tlc_attention_decode; the split partials live in a fixed array of this library instead of
// buffers the caller provides.
#include "no_alloc.h"

static __device__ __align__(256) float g_decode_scratch[TLC_NO_ALLOC_SCRATCH_FLOATS];
static float* g_decode_scratch_addr[TLC_NO_ALLOC_MAX_DEVICES];      // device address of the array, per device

extern "C" int tlc_attention_decode_no_alloc(const void* q, int dtype, const void* k_pages, const void* v_pages,
                                             const int* block_table, int max_pages, const int* positions,
                                             const int* row_seq, const int* slots, void* out, int T, int H, int KV,
                                             int hd, float scale, int window, int max_keys, cudaStream_t stream) {
  if (T == 0) return 0;
  TLC_REQUIRE(T > 0 && H > 0 && hd > 0 && max_keys > 0, "attention(no alloc): sizes must be positive");
  const long long n_splits = ((long long)max_keys + DEC_KEYS - 1) / DEC_KEYS;
  const long long need = (long long)T * H * n_splits * ((long long)hd + 2);
  TLC_REQUIRE(need <= (long long)TLC_NO_ALLOC_SCRATCH_FLOATS,
              "attention(no alloc): %d rows x %d heads x %lld splits x (head size %d + 2) = %lld floats of partial "
              "results exceed the built-in scratch of %d floats; use tlc_attention_decode with caller buffers",
              T, H, n_splits, hd, need, (int)TLC_NO_ALLOC_SCRATCH_FLOATS);
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return tlc_fail(-2, "attention(no alloc): cudaGetDevice: %s", cudaGetErrorString(e));
  TLC_REQUIRE(dev >= 0 && dev < TLC_NO_ALLOC_MAX_DEVICES, "attention(no alloc): device %d is beyond the %d this library tracks",
              dev, TLC_NO_ALLOC_MAX_DEVICES);
  if (g_decode_scratch_addr[dev] == nullptr) {
    // First call on this device: ask the runtime where this device's copy of the array lives.
    // (In host code the array's name is only a handle, not an address a kernel could use.)
    float* p = nullptr;
    e = cudaGetSymbolAddress((void**)&p, g_decode_scratch);
    if (e != cudaSuccess || p == nullptr)
      return tlc_fail(-2, "attention(no alloc): cudaGetSymbolAddress: %s", cudaGetErrorString(e));
    g_decode_scratch_addr[dev] = p;
  }
  float* part_o = g_decode_scratch_addr[dev];
  float* part_ml = part_o + (size_t)T * H * n_splits * hd;
  return tlc_attention_decode(q, dtype, k_pages, v_pages, block_table, max_pages, positions, row_seq, slots, out, part_o,
                              part_ml, T, H, KV, hd, scale, window, max_keys, 0, stream);
}
