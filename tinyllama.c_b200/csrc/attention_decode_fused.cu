// Single-token attention as one kernel on the tensor cores (bfloat16 cache, head sizes 64, 128, 256,
// up to 8 query heads per key/value head).
//
// One launch does what the separate kernels do in three: the rotation of the row's queries and of
// its new key (split-half form, angle = position * inv_freq[i] in 32-bit; CodeClaper/tinyllama.c
// cpu_op.c:637-651), the store of the new key/value row into its page (cpu_op.c:995-1008), attention of
// the row over its keys with 32-bit scores, statistics and accumulator (cpu_op.c:1010-1062), and the
// merge of the splits, which the last block of a (row, key/value head) to finish does.
//
// The query heads that share a key/value head are the rows of one matrix product (mma.sync m16n8k16,
// rows 8..15 unused): scores = Q [heads, dims] x K^T, output = P [heads, keys] x V, as in the kernel
// for prompts.  A block is four warps; each warp owns every fourth chunk of keys of the block's range,
// brings the chunk's key and value rows into its own part of shared memory with cp.async (the next
// chunks travel while the current one is worked on), and keeps running softmax statistics of its own,
// so the loop has no block-wide barrier.  The warps' results meet in shared memory; with one block per
// (row, key/value head) the block writes the output itself, otherwise partial results go to scratch and
// the last block to arrive merges them.
//
// Arrival counting: every block of a (row, kv head) adds one to arrivals[row * KV + kv head] with
// atomicInc modulo the number of splits, so the counter is back at zero when the kernel ends and needs
// no clearing between launches.  It must be zero before the first launch.
#include <algorithm>
#include "attention_split_merge.cuh"
#include "common.cuh"

#define FM_NW 4
#define FM_NT (FM_NW * 32)
#define FM_MAXG 8

namespace {

__device__ __forceinline__ void fm_cp16(void* smem, const void* gmem, bool pred) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  const int n = pred ? 16 : 0;                       // 0: the 16 bytes are filled with zeros, nothing is read
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(s), "l"(gmem), "r"(n) : "memory");
}
__device__ __forceinline__ void fm_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void fm_wait_group() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ void ldsm_x2(unsigned& r0, unsigned& r1, const void* p) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0, %1}, [%2];" : "=r"(r0), "=r"(r1) : "r"(s));
}
__device__ __forceinline__ void ldsm_x4(unsigned (&r)[4], const void* p) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void ldsm_x4_trans(unsigned (&r)[4], const void* p) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
// d += a x b; rows 8..15 of a are zero (a1 = a3 = 0)
__device__ __forceinline__ void mma_bf16(float (&d)[4], unsigned a0, unsigned a2, unsigned b0, unsigned b1) {
  const unsigned z = 0;
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3]) : "r"(a0), "r"(z), "r"(a2), "r"(z), "r"(b0), "r"(b1));
}
__device__ __forceinline__ unsigned pack_bf16(float lo, float hi) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const unsigned*>(&v);
}

template <int HD, int CK, int STAGES>
struct FmSmem {
  static constexpr int ROWB = HD * 2;                       // bytes of a key or value row
  static constexpr int TILE = CK * ROWB;                    // a chunk of keys (or of values)
  static constexpr int WARP = STAGES * 2 * TILE;            // a warp's stages
  static constexpr int Q = 8 * ROWB;                        // the group's rotated queries, bfloat16
  static constexpr int FIXED = FM_NW * WARP + Q + 2 * ROWB + 2 * FM_NW * 8 * 4;   // + new key, new value, statistics
  static size_t bytes(int passes) { return (size_t)FIXED + (size_t)passes * (FM_NW * CK / TLC_PAGE + 1) * sizeof(int); }
};

// HD: head size; CK: keys of a chunk (a multiple of 16); STAGES: chunks of a warp in shared memory.
// A block takes `passes` rounds of FM_NW chunks, one per warp.  Within a row of shared memory the
// 16-byte pieces are stored at piece ^ (row & 7): ldmatrix then reads eight rows without bank conflicts.
template <int HD, int CK, int STAGES>
__global__ void __launch_bounds__(FM_NT)
attention_decode_fused_kernel(const float* __restrict__ qkv, int ld, int q_off, int k_off, int v_off,
                            __nv_bfloat16* __restrict__ k_pages, __nv_bfloat16* __restrict__ v_pages,
                            const float* __restrict__ inv_freq, int rope_dim, int write_kv,
                            const int* __restrict__ block_table, int max_pages, const int* __restrict__ positions,
                            const int* __restrict__ row_seq, const int* __restrict__ slots, float* __restrict__ part_o,
                            float* __restrict__ part_ml, unsigned* __restrict__ arrivals,
                            __nv_bfloat16* __restrict__ out, int H, int KV, float scale, int window, int n_splits,
                            int passes, int out_ld) {
  // Keys and values of earlier positions were stored by earlier steps and are fetched before the
  // wait on the previous kernel; the row's own projection is read after it.
  asm volatile("griddepcontrol.launch_dependents;");
  using L = FmSmem<HD, CK, STAGES>;
  constexpr int ROWB = L::ROWB, TILE = L::TILE, CPR = HD / 8, NT_S = CK / 8, NT_O = HD / 8;
  static_assert(CK % 16 == 0 && HD % 16 == 0 && CPR <= 32, "chunk and head size");
  extern __shared__ __align__(128) unsigned char smraw[];
  const int tid = threadIdx.x, lane = tid & 31, w = tid >> 5;
  const int t = blockIdx.x, g = blockIdx.y, split = blockIdx.z;
  const int G = H / KV;
  const int pos = positions[t];
  const int n_keys = pos + 1;
  const int start = (window > 0 && n_keys > window) ? n_keys - window : 0;
  const int round = FM_NW * CK;              // keys of one round of the block's warps
  const int span = round * passes;           // keys of this block
  const int kbase = split * span;
  const int n_pg = (span + TLC_PAGE - 1) / TLC_PAGE;
  const int smem_floats = L::FIXED / 4;
  float* ml = part_ml + (((size_t)t * H + (size_t)g * G) * n_splits + split) * 2;
  const bool empty = kbase >= n_keys || kbase + span <= start;     // the same for all threads of the block
  __shared__ int s_last;
  if (empty) {
    tlc_wait(ml);
    if (tid < G) { ml[(size_t)tid * n_splits * 2] = -INFINITY; ml[(size_t)tid * n_splits * 2 + 1] = 0.f; }
  } else {
    unsigned char* wsm = smraw + (size_t)w * L::WARP;                                // this warp's stages
    unsigned char* qsm = smraw + (size_t)FM_NW * L::WARP;                            // [8][HD] bfloat16
    __nv_bfloat16* knew = reinterpret_cast<__nv_bfloat16*>(qsm + L::Q);              // [HD]
    __nv_bfloat16* vnew = knew + HD;                                                 // [HD]
    float* m_s = reinterpret_cast<float*>(vnew + HD);                                // [FM_NW][8]
    float* l_s = m_s + FM_NW * 8;                                                    // [FM_NW][8]
    int* pages = reinterpret_cast<int*>(l_s + FM_NW * 8);                            // [n_pg]
    const int* table = block_table + (size_t)slots[row_seq[t]] * max_pages;
    {
      // the block's pages; before the window a page may have been given back, past the end none is held
      const int pg0 = kbase / TLC_PAGE;
      for (int j = tid; j < n_pg; j += FM_NT) {
        const int pi = pg0 + j;
        pages[j] = (pi * TLC_PAGE < n_keys && (pi + 1) * TLC_PAGE > start) ? table[pi] : 0;
      }
    }
    __syncthreads();
    const bool has_new = write_kv && pos >= kbase && pos < kbase + span;   // this block holds the row's own key
    const int pg_base = kbase / TLC_PAGE * TLC_PAGE;
    auto row_offset = [&](int key) {        // of a key's row in the pages, in elements
      return (((size_t)pages[(key - pg_base) / TLC_PAGE] * KV + g) * TLC_PAGE + key % TLC_PAGE) * HD;
    };
    // this warp's chunks: chunk j starts at base_w + j * round
    const int base_w = kbase + w * CK;
    int j_first = 0;
    if (start - CK - base_w >= 0) j_first = (start - CK - base_w) / round + 1;
    const int j_last = n_keys - 1 - base_w >= 0 ? min(passes - 1, (n_keys - 1 - base_w) / round) : -1;
    // chunk j on its way into its stage (all rows but the row's own position; rows that are no keys of
    // the row are filled with zeros); always closes a group, so that groups can be counted
    auto issue = [&](int j) {
      if (j <= j_last) {
        const int k0 = base_w + j * round;
        unsigned char* Ks = wsm + (size_t)((j - j_first) % STAGES) * (2 * TILE);
        unsigned char* Vs = Ks + TILE;
#pragma unroll 4
        for (int q = lane; q < CK * CPR; q += 32) {
          const int row = q / CPR, c = q % CPR;
          const int key = k0 + row;
          const bool ok = key >= start && key < n_keys && key != pos;
          const size_t off = ok ? row_offset(key) + (size_t)c * 8 : 0;
          const int dst = row * ROWB + ((c ^ (row & 7)) << 4);
          fm_cp16(Ks + dst, k_pages + off, ok);
          fm_cp16(Vs + dst, v_pages + off, ok);
        }
      }
      fm_commit();
    };
#pragma unroll
    for (int s = 0; s < STAGES; s++) issue(j_first + s);
    tlc_wait(qkv, k_pages, v_pages, part_o, ml, out);
    // rotation: the thread of dim d turns that dim of every query head of the group and of the key;
    // all of its loads are issued before the first use
    for (int d = tid; d < HD; d += FM_NT) {
      const float* row = qkv + (size_t)t * ld;
      const int half = rope_dim >> 1;
      const bool rot = d < rope_dim;
      const bool lo = d < half;
      const int i = rot ? (lo ? d : d - half) : d;          // first element of the pair (or the dim itself)
      const int j = rot ? i + half : d;                     // second element
      float a[FM_MAXG + 1], b[FM_MAXG + 1], vv = 0.f;
#pragma unroll
      for (int hg = 0; hg < FM_MAXG; hg++) {
        if (hg < G) {
          const float* src = row + q_off + ((size_t)g * G + hg) * HD;
          a[hg] = src[i];
          b[hg] = src[j];
        }
      }
      if (has_new) {
        const float* src = row + k_off + (size_t)g * HD;
        a[FM_MAXG] = src[i];
        b[FM_MAXG] = src[j];
        vv = row[v_off + (size_t)g * HD + d];
      }
      float sn = 0.f, cs = 1.f;
      if (rot) sincosf((float)pos * inv_freq[i], &sn, &cs);
#pragma unroll
      for (int hg = 0; hg < FM_MAXG; hg++) {
        float v = 0.f;                                      // rows of heads the group does not have stay zero
        if (hg < G) v = rot ? (lo ? a[hg] * cs - b[hg] * sn : a[hg] * sn + b[hg] * cs) : a[hg];
        *reinterpret_cast<__nv_bfloat16*>(qsm + hg * ROWB + (((d >> 3) ^ hg) << 4) + (d & 7) * 2) = __float2bfloat16_rn(v);
      }
      if (has_new) {
        const float v = rot ? (lo ? a[FM_MAXG] * cs - b[FM_MAXG] * sn : a[FM_MAXG] * sn + b[FM_MAXG] * cs) : a[FM_MAXG];
        knew[d] = __float2bfloat16_rn(v);
        vnew[d] = __float2bfloat16_rn(vv);
      }
    }
    __syncthreads();
    if (has_new && tid < CPR) {
      const size_t at = row_offset(pos);
      reinterpret_cast<uint4*>(k_pages + at)[tid] = reinterpret_cast<const uint4*>(knew)[tid];
      reinterpret_cast<uint4*>(v_pages + at)[tid] = reinterpret_cast<const uint4*>(vnew)[tid];
    }
    // ---- this warp's chunks, with running statistics of head lane / 4 ----
    const int hrow = lane >> 2, cpair = (lane & 3) * 2;
    float run_m = -INFINITY, run_l = 0.f;        // run_l: this lane's share of the sum (its key columns)
    float O[NT_O][4];
#pragma unroll
    for (int n = 0; n < NT_O; n++) { O[n][0] = O[n][1] = O[n][2] = O[n][3] = 0.f; }
#pragma unroll 1
    for (int j = j_first; j <= j_last; j++) {
      fm_wait_group<STAGES - 1>();                // all but the STAGES - 1 newest groups: chunk j has arrived
      __syncwarp();
      const int k0 = base_w + j * round;
      unsigned char* Ks = wsm + (size_t)((j - j_first) % STAGES) * (2 * TILE);
      unsigned char* Vs = Ks + TILE;
      if (pos >= k0 && pos < k0 + CK) {
        // the row's own key and value: written above by this block, or (a layer that only reads) by an
        // earlier kernel
        if (lane < CPR) {
          const int row = pos - k0;
          const int dst = row * ROWB + ((lane ^ (row & 7)) << 4);
          const size_t at = row_offset(pos);
          *reinterpret_cast<uint4*>(Ks + dst) = has_new ? reinterpret_cast<const uint4*>(knew)[lane]
                                                        : reinterpret_cast<const uint4*>(k_pages + at)[lane];
          *reinterpret_cast<uint4*>(Vs + dst) = has_new ? reinterpret_cast<const uint4*>(vnew)[lane]
                                                        : reinterpret_cast<const uint4*>(v_pages + at)[lane];
        }
        __syncwarp();
      }
      // scores of the group's heads for the chunk's keys
      float S[NT_S][4];
#pragma unroll
      for (int n = 0; n < NT_S; n++) { S[n][0] = S[n][1] = S[n][2] = S[n][3] = 0.f; }
#pragma unroll
      for (int ks = 0; ks < HD / 16; ks++) {
        unsigned qa0, qa2;
        {
          const int r = lane & 7, c = 2 * ks + ((lane >> 3) & 1);
          ldsm_x2(qa0, qa2, qsm + r * ROWB + ((c ^ r) << 4));
        }
#pragma unroll
        for (int p = 0; p < CK / 16; p++) {
          unsigned kb[4];
          const int mi = lane >> 3;
          const int row = p * 16 + (mi >> 1) * 8 + (lane & 7), c = 2 * ks + (mi & 1);
          ldsm_x4(kb, Ks + row * ROWB + ((c ^ (row & 7)) << 4));
          mma_bf16(S[2 * p], qa0, qa2, kb[0], kb[1]);
          mma_bf16(S[2 * p + 1], qa0, qa2, kb[2], kb[3]);
        }
      }
      // softmax of head `hrow` over this lane's keys, with the running maximum
      float mx = -INFINITY;
#pragma unroll
      for (int n = 0; n < NT_S; n++) {
#pragma unroll
        for (int e = 0; e < 2; e++) {
          const int key = k0 + n * 8 + cpair + e;
          const bool valid = key >= start && key < n_keys;
          S[n][e] = valid ? S[n][e] * scale : -INFINITY;
          mx = fmaxf(mx, S[n][e]);
        }
      }
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
      const float m_new = fmaxf(run_m, mx);
      const float m_use = m_new == -INFINITY ? 0.f : m_new;        // a chunk may hold no key of the row at all
      const float corr = expf(run_m - m_use);                      // 0 while nothing has been seen
      run_m = m_new;
      float lsum = 0.f;
      unsigned pa[NT_S];
#pragma unroll
      for (int n = 0; n < NT_S; n++) {
        const float p0 = expf(S[n][0] - m_use), p1 = expf(S[n][1] - m_use);
        lsum += p0 + p1;
        pa[n] = pack_bf16(p0, p1);
      }
      run_l = run_l * corr + lsum;
#pragma unroll
      for (int n = 0; n < NT_O; n++) { O[n][0] *= corr; O[n][1] *= corr; }
      // output += P x V
#pragma unroll
      for (int kk = 0; kk < CK / 16; kk++) {
#pragma unroll
        for (int dp = 0; dp < HD / 16; dp++) {
          unsigned vb[4];
          const int mi = lane >> 3;
          const int row = kk * 16 + (mi & 1) * 8 + (lane & 7), c = 2 * dp + (mi >> 1);
          ldsm_x4_trans(vb, Vs + row * ROWB + ((c ^ (row & 7)) << 4));
          mma_bf16(O[2 * dp], pa[2 * kk], pa[2 * kk + 1], vb[0], vb[1]);
          mma_bf16(O[2 * dp + 1], pa[2 * kk], pa[2 * kk + 1], vb[2], vb[3]);
        }
      }
      __syncwarp();                               // every lane is done with the stage:
      issue(j + STAGES);                          // the chunk STAGES further on takes it
    }
    fm_wait_group<0>();
    __syncwarp();
    // ---- the warps' results meet ----
    run_l += __shfl_xor_sync(0xffffffffu, run_l, 1);
    run_l += __shfl_xor_sync(0xffffffffu, run_l, 2);
    if ((lane & 3) == 0) { m_s[w * 8 + hrow] = run_m; l_s[w * 8 + hrow] = run_l; }
    float* ow = reinterpret_cast<float*>(wsm);    // [G][HD], in the warp's own stages
    if (hrow < G) {
#pragma unroll
      for (int n = 0; n < NT_O; n++)
        *reinterpret_cast<float2*>(ow + hrow * HD + n * 8 + cpair) = make_float2(O[n][0], O[n][1]);
    }
    __syncthreads();
    for (int idx = tid; idx < G * HD; idx += FM_NT) {
      const int hg = idx / HD, d = idx % HD;
      float M = -INFINITY;
#pragma unroll
      for (int x = 0; x < FM_NW; x++) M = fmaxf(M, m_s[x * 8 + hg]);
      float o = 0.f, l = 0.f;
#pragma unroll
      for (int x = 0; x < FM_NW; x++) {
        const float mw = m_s[x * 8 + hg];
        if (mw > -INFINITY) {
          const float e = expf(mw - M);
          l = fmaf(l_s[x * 8 + hg], e, l);
          o = fmaf(reinterpret_cast<const float*>(smraw + (size_t)x * L::WARP)[hg * HD + d], e, o);
        }
      }
      const size_t th = (size_t)t * H + (size_t)g * G + hg;
      if (n_splits == 1) {
        out[(size_t)t * out_ld + ((size_t)g * G + hg) * HD + d] = __float2bfloat16_rn(o * (1.0f / l));
      } else {
        part_o[(th * n_splits + split) * HD + d] = o;
        if (d == 0) { ml[(size_t)hg * n_splits * 2] = M; ml[(size_t)hg * n_splits * 2 + 1] = l; }
      }
    }
  }
  if (n_splits == 1) return;                      // one block per (row, kv head): it wrote the output itself
  // ---- the last block of this (row, kv head) merges the splits ----
  __threadfence();
  __syncthreads();
  if (tid == 0) {
    const unsigned old = atomicInc(arrivals + (size_t)t * KV + g, (unsigned)(n_splits - 1));
    s_last = old == (unsigned)(n_splits - 1);
  }
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  attention_merge_splits<HD, FM_NT>(part_o, part_ml, out, reinterpret_cast<float*>(smraw), smem_floats, t, g, G, H, n_splits, out_ld);
}

int g_fused_passes = 0;       // > 0: rounds a block takes, for tests (0: chosen from the grid)

template <int HD, int CK, int STAGES, typename... Args>
cudaError_t launch_fused(dim3 grid, int passes, cudaStream_t stream, Args... args) {
  static bool raised[64] = {};          // per device: the kernel uses more than 48 KB of shared memory
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !raised[dev]) {
    cudaError_t e = cudaFuncSetAttribute(attention_decode_fused_kernel<HD, CK, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    if (e != cudaSuccess) return e;
    raised[dev] = true;
  }
  return tlc_launch(attention_decode_fused_kernel<HD, CK, STAGES>, grid, dim3(FM_NT), FmSmem<HD, CK, STAGES>::bytes(passes), stream, args...);
}

}  // namespace

extern "C" int tlc_attention_decode_fused_passes(int passes) { g_fused_passes = passes; return 0; }

// 1 if the kernel takes these sizes (the caller falls back to the separate kernels otherwise)
extern "C" int tlc_attention_decode_fused_ok(int H, int KV, int hd) {
  if (KV <= 0 || H % KV != 0 || H / KV > FM_MAXG || KV > 65535) return 0;
  return hd == 64 || hd == 128 || hd == 256;
}

// qkv: float32 rows of `ld` elements with the queries, keys and values of the row at q_off, k_off,
// v_off.  scratch: part_o [T, H, n_splits, hd], part_ml [T, H, n_splits, 2] floats with
// n_splits <= ceil(max_keys / 128); arrivals: T * KV counters, zero before the first call.
extern "C" int tlc_attention_decode_fused(const float* qkv, int ld, int q_off, int k_off, int v_off, void* k_pages,
                                        void* v_pages, const float* inv_freq, int rope_dim, int write_kv,
                                        const int* block_table, int max_pages, const int* positions,
                                        const int* row_seq, const int* slots, void* out, float* part_o, float* part_ml,
                                        unsigned* arrivals, int T, int H, int KV, int hd, float scale, int window,
                                        int max_keys, int out_ld, cudaStream_t stream) {
  if (T == 0) return 0;
  if (out_ld <= 0) out_ld = H * hd;                      // elements between rows of out (0: dense)
  TLC_REQUIRE(tlc_attention_decode_fused_ok(H, KV, hd), "attention(decode, fused): %d heads, %d key/value heads of size %d are outside the kernel's range", H, KV, hd);
  TLC_REQUIRE(rope_dim % 2 == 0 && rope_dim >= 0 && rope_dim <= hd, "attention(decode, fused): rotated width %d must be even and at most head_dim %d", rope_dim, hd);
  TLC_REQUIRE(max_keys >= 1, "attention(decode, fused): %d keys", max_keys);
  // a round of the block's four warps is 128 keys (64 with heads of 256); a block takes as many rounds as
  // keeps the grid within one block an SM
  int sms = 148, dev = 0;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int round = hd == 256 ? FM_NW * 16 : FM_NW * 32;
  const int pieces = (max_keys + round - 1) / round;
  const long long rows = (long long)T * KV;
  const int want_splits = (int)std::max<long long>(1, std::min<long long>(pieces, sms / rows));
  int passes = (pieces + want_splits - 1) / want_splits;
  if (g_fused_passes > 0) passes = std::min(g_fused_passes, pieces);
  int n_splits = (pieces + passes - 1) / passes;
  // the scratch holds ceil(max_keys / 128) splits of a row
  const int max_splits = (max_keys + 127) / 128;
  if (n_splits > max_splits) { n_splits = max_splits; passes = (pieces + n_splits - 1) / n_splits; n_splits = (pieces + passes - 1) / passes; }
  TLC_REQUIRE(n_splits >= 1 && n_splits <= 65535, "attention(decode, fused): %d keys are outside the kernel's range", max_keys);
  // Two stages per warp (four with heads of 64) even when a warp has one chunk only: with one stage three
  // blocks fit an SM, and the model's step at batch 8 took 1.82 ms instead of 1.44.
  const size_t smem = hd == 64 ? FmSmem<64, 32, 4>::bytes(passes) : hd == 128 ? FmSmem<128, 32, 2>::bytes(passes) : FmSmem<256, 16, 2>::bytes(passes);
  TLC_REQUIRE(smem <= 200 * 1024, "attention(decode, fused): %d keys need %zu bytes of shared memory", max_keys, smem);
  dim3 grid(T, KV, n_splits);
  __nv_bfloat16 *kp = (__nv_bfloat16*)k_pages, *vp = (__nv_bfloat16*)v_pages, *op = (__nv_bfloat16*)out;
  cudaError_t e = cudaSuccess;
#define TLC_FM_LAUNCH(HDV, CKV, STV)                                                                                   \
  e = launch_fused<HDV, CKV, STV>(grid, passes, stream, qkv, ld, q_off, k_off, v_off, kp, vp, inv_freq, rope_dim, write_kv, \
                                block_table, max_pages, positions, row_seq, slots, part_o, part_ml, arrivals, op, H, KV, \
                                scale, window, n_splits, passes, out_ld)
  if (hd == 64) TLC_FM_LAUNCH(64, 32, 4);
  else if (hd == 128) TLC_FM_LAUNCH(128, 32, 2);
  else TLC_FM_LAUNCH(256, 16, 2);
#undef TLC_FM_LAUNCH
  if (e != cudaSuccess) return tlc_fail(-2, "attention(decode, fused): %s", cudaGetErrorString(e));
  TLC_CHECK_LAUNCH("attention(decode)");
  return 0;
}
