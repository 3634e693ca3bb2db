// Attention for the prompts of a step: tiled, tensor cores, keys and values read from the pages.
//
// Same math as the reference's op_attn (cpu_op.c:1010-1062): causal grouped-query attention,
// scale 1/sqrt(head_dim), max-subtracted softmax, optional window.  A block takes 64
// consecutive new rows of one sequence and one query head; it walks the sequence's pages (a
// page is exactly one 64-key tile, contiguous per kv head) from the first visible key to the
// diagonal, keeping a running maximum, sum and output per row (32-bit) while the two products
// Q K^T and P V run on mma.sync.m16n8k16 with bfloat16 operands.  K and V tiles are staged in
// shared memory with cp.async, two tiles in flight; rows are XOR-swizzled in 16-byte chunks so
// that ldmatrix is conflict-free.  Sequences of unequal length are packed back to back; a
// block finds its sequence from cu_seqlens.
#include "common.cuh"

namespace {

constexpr int FA_BM = 64;     // query rows per block (16 per warp)
constexpr int FA_BN = 64;     // keys per tile = one page
static_assert(FA_BN == TLC_PAGE, "a key tile is one page");

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void mma16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

// byte offset of (row, 16-byte chunk) in a [rows][HD] bf16 tile whose chunks are swizzled by row
template <int HD> __device__ __forceinline__ uint32_t tile_off(int row, int chunk) {
  return (uint32_t)(row * HD * 2 + ((chunk ^ (row & 7)) << 4));
}

template <int HD>
__global__ void __launch_bounds__(128)
attention_prefill_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k_pages,
                         const __nv_bfloat16* __restrict__ v_pages, const int* __restrict__ block_table, int max_pages,
                         const int* __restrict__ cu_seqlens, const int* __restrict__ slots,
                         const int* __restrict__ start_pos, __nv_bfloat16* __restrict__ out, int n_seqs, int H, int KV,
                         float scale_log2, int window, int chunk_tiles, int n_chunks_max, float* __restrict__ part_o,
                         float* __restrict__ part_ml, int out_ld) {
  tlc_pdl(q, k_pages, v_pages, out, part_o, part_ml);
  constexpr int CH = HD / 8;                  // 16-byte chunks per row
  constexpr int TILE_BYTES = FA_BN * HD * 2;
  extern __shared__ __align__(128) uint8_t fa_smem[];
  uint8_t* q_s = fa_smem;                     // [64][HD]
  uint8_t* k_s = q_s + FA_BM * HD * 2;        // 2 x [64][HD]
  uint8_t* v_s = k_s + 2 * TILE_BYTES;        // 2 x [64][HD]
  __shared__ int s_seq, s_row0;

  // which sequence, and which of its 64-row tiles, is this block's
  if (threadIdx.x == 0) {
    int tile = blockIdx.x, b = 0, found = -1, row0 = 0;
    for (; b < n_seqs; b++) {
      const int n = cu_seqlens[b + 1] - cu_seqlens[b];
      const int nt = (n + FA_BM - 1) / FA_BM;
      if (tile < nt) { found = b; row0 = tile * FA_BM; break; }
      tile -= nt;
    }
    s_seq = found;
    s_row0 = row0;
  }
  __syncthreads();
  const int b = s_seq;
  if (b < 0) return;
  const int i0 = s_row0;
  const int h = blockIdx.y, g = h / (H / KV);
  const int t0 = cu_seqlens[b], n_new = cu_seqlens[b + 1] - t0;
  const int rows = min(FA_BM, n_new - i0);
  const int p0 = start_pos[b] + i0;                       // position of the block's first row
  const int q_max = p0 + rows - 1;
  const int* table = block_table + (size_t)slots[b] * max_pages;
  const int tile_hi_all = q_max / FA_BN;
  const int tile_lo_all = window > 0 ? max(0, p0 + 1 - window) / FA_BN : 0;
  // Long rows are cut: block z of the row tile takes key tiles [lo + z * chunk, lo + (z + 1) * chunk), so that
  // the last rows of a long prompt do not set the kernel's length; a second kernel merges the pieces.
  const int n_chunks = (tile_hi_all - tile_lo_all) / chunk_tiles + 1;
  const int tile_lo = tile_lo_all + (int)blockIdx.z * chunk_tiles;
  if (tile_lo > tile_hi_all) return;
  const int tile_hi = min(tile_hi_all, tile_lo + chunk_tiles - 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t q_u = (uint32_t)__cvta_generic_to_shared(q_s), k_u = (uint32_t)__cvta_generic_to_shared(k_s),
                 v_u = (uint32_t)__cvta_generic_to_shared(v_s);

  auto load_kv = [&](int tile, int buf) {
    const size_t base = (((size_t)table[tile] * KV + g) * FA_BN) * HD;
    const uint4* ks = reinterpret_cast<const uint4*>(k_pages + base);
    const uint4* vs = reinterpret_cast<const uint4*>(v_pages + base);
    for (int i = threadIdx.x; i < FA_BN * CH; i += 128) {
      const int r = i / CH, c = i % CH;
      cp_async16(k_u + buf * TILE_BYTES + tile_off<HD>(r, c), ks + i);
      cp_async16(v_u + buf * TILE_BYTES + tile_off<HD>(r, c), vs + i);
    }
  };

  // Q tile (rows past the sequence's end are zero), first K/V tile
  for (int i = threadIdx.x; i < FA_BM * CH; i += 128) {
    const int r = i / CH, c = i % CH;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (r < rows) v = *reinterpret_cast<const uint4*>(q + ((size_t)(t0 + i0 + r) * H + h) * HD + c * 8);
    *reinterpret_cast<uint4*>(q_s + tile_off<HD>(r, c)) = v;
  }
  load_kv(tile_lo, 0);
  cp_async_commit();
  __syncthreads();

  // this warp's 16 query rows as A fragments
  uint32_t qa[HD / 16][4];
#pragma unroll
  for (int kk = 0; kk < HD / 16; kk++) {
    const int r = warp * 16 + (lane & 15), c = kk * 2 + (lane >> 4);
    ldsm_x4(q_u + tile_off<HD>(r, c), qa[kk][0], qa[kk][1], qa[kk][2], qa[kk][3]);
  }

  float o[HD / 8][4];
#pragma unroll
  for (int j = 0; j < HD / 8; j++)
#pragma unroll
    for (int i = 0; i < 4; i++) o[j][i] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
  const int gq = lane >> 2, tq = lane & 3;
  const int qpos0 = p0 + warp * 16 + gq, qpos1 = qpos0 + 8;       // positions of this thread's two rows

  for (int tile = tile_lo; tile <= tile_hi; tile++) {
    const int buf = (tile - tile_lo) & 1;
    if (tile + 1 <= tile_hi) load_kv(tile + 1, buf ^ 1);
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();

    // S = Q K^T for 16 rows x 64 keys
    float s[FA_BN / 8][4];
#pragma unroll
    for (int j = 0; j < FA_BN / 8; j++)
#pragma unroll
      for (int i = 0; i < 4; i++) s[j][i] = 0.f;
#pragma unroll
    for (int kk = 0; kk < HD / 16; kk++) {
#pragma unroll
      for (int jp = 0; jp < FA_BN / 16; jp++) {
        // four 8x8 blocks: keys jp*16 + (0..7 | 8..15), head dims kk*16 + (0..7 | 8..15)
        const int r = jp * 16 + (lane & 7) + ((lane >> 4) << 3), c = kk * 2 + ((lane >> 3) & 1);
        uint32_t b0, b1, b2, b3;
        ldsm_x4(k_u + buf * TILE_BYTES + tile_off<HD>(r, c), b0, b1, b2, b3);
        mma16816(s[2 * jp], qa[kk][0], qa[kk][1], qa[kk][2], qa[kk][3], b0, b1);
        mma16816(s[2 * jp + 1], qa[kk][0], qa[kk][1], qa[kk][2], qa[kk][3], b2, b3);
      }
    }
    // mask: causal, window, keys past the page's filled part are covered by the causal test
    const int kbase = tile * FA_BN;
    const bool need_mask = (kbase + FA_BN - 1 > p0) || (window > 0);
    if (need_mask) {
#pragma unroll
      for (int j = 0; j < FA_BN / 8; j++) {
#pragma unroll
        for (int i = 0; i < 4; i++) {
          const int kpos = kbase + j * 8 + 2 * tq + (i & 1);
          const int qp = (i < 2) ? qpos0 : qpos1;
          const bool vis = kpos <= qp && (window <= 0 || kpos > qp - window);
          if (!vis) s[j][i] = -INFINITY;
        }
      }
    }
    // online softmax for the two rows of this thread
#pragma unroll
    for (int r = 0; r < 2; r++) {
      float mx = -INFINITY;
#pragma unroll
      for (int j = 0; j < FA_BN / 8; j++) mx = fmaxf(mx, fmaxf(s[j][2 * r], s[j][2 * r + 1]));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
      const float m_new = fmaxf(m_run[r], mx);
      const float m_use = m_new == -INFINITY ? 0.f : m_new;       // a row with nothing visible yet
      const float corr = exp2f((m_run[r] - m_use) * scale_log2);
      float sum = 0.f;
#pragma unroll
      for (int j = 0; j < FA_BN / 8; j++) {
        const float p0v = exp2f((s[j][2 * r] - m_use) * scale_log2);
        const float p1v = exp2f((s[j][2 * r + 1] - m_use) * scale_log2);
        s[j][2 * r] = p0v;
        s[j][2 * r + 1] = p1v;
        sum += p0v + p1v;
      }
      sum += __shfl_xor_sync(0xffffffffu, sum, 1);
      sum += __shfl_xor_sync(0xffffffffu, sum, 2);
      l_run[r] = l_run[r] * corr + sum;
      m_run[r] = m_new;
#pragma unroll
      for (int j = 0; j < HD / 8; j++) { o[j][2 * r] *= corr; o[j][2 * r + 1] *= corr; }
    }
    // O += P V
#pragma unroll
    for (int kk = 0; kk < FA_BN / 16; kk++) {
      const uint32_t a0 = pack_bf16(s[2 * kk][0], s[2 * kk][1]), a1 = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
      const uint32_t a2 = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]), a3 = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
      for (int jp = 0; jp < HD / 16; jp++) {
        // four 8x8 blocks: keys kk*16 + (0..7 | 8..15), head dims jp*16 + (0..7 | 8..15), transposed on load
        const int r = kk * 16 + (lane & 7) + (((lane >> 3) & 1) << 3), c = jp * 2 + (lane >> 4);
        uint32_t b0, b1, b2, b3;
        ldsm_x4_trans(v_u + buf * TILE_BYTES + tile_off<HD>(r, c), b0, b1, b2, b3);
        mma16816(o[2 * jp], a0, a1, a2, a3, b0, b1);
        mma16816(o[2 * jp + 1], a0, a1, a2, a3, b2, b3);
      }
    }
    __syncthreads();          // everyone is done with this buffer before it is filled again
  }

  if (n_chunks > 1) {
    // a piece of the row: the sums as they are, with the maximum and the denominator they refer to
#pragma unroll
    for (int r = 0; r < 2; r++) {
      const int lr = warp * 16 + gq + 8 * r;
      if (lr < rows) {
        const size_t at = (((size_t)(t0 + i0 + lr) * H + h) * n_chunks_max + blockIdx.z);
        float* orow = part_o + at * HD;
#pragma unroll
        for (int j = 0; j < HD / 8; j++)
          *reinterpret_cast<float2*>(orow + j * 8 + 2 * tq) = make_float2(o[j][2 * r], o[j][2 * r + 1]);
        if (tq == 0) {
          part_ml[at * 2] = m_run[r];
          part_ml[at * 2 + 1] = l_run[r];
        }
      }
    }
    return;
  }
  // normalise and store
#pragma unroll
  for (int r = 0; r < 2; r++) {
    const int lr = warp * 16 + gq + 8 * r;
    if (lr < rows) {
      const float inv = 1.0f / l_run[r];
      __nv_bfloat16* orow = out + (size_t)(t0 + i0 + lr) * out_ld + (size_t)h * HD;
#pragma unroll
      for (int j = 0; j < HD / 8; j++)
        *reinterpret_cast<uint32_t*>(orow + j * 8 + 2 * tq) = pack_bf16(o[j][2 * r] * inv, o[j][2 * r + 1] * inv);
    }
  }
}

// Rows that were cut into pieces: out = sum_z o_z 2^((m_z - m) scale) / sum_z l_z 2^((m_z - m) scale).
// grid (T, ceil(H / 4)); a warp per (row, head), a lane per 4 head dims (and their next 128, 256, ...); at most
// FA_MAX_CHUNKS pieces, all of whose values are in flight together.
constexpr int FA_MAX_CHUNKS = 16;
__global__ void __launch_bounds__(128)
attention_prefill_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                               const int* __restrict__ cu_seqlens, const int* __restrict__ row_seq,
                               const int* __restrict__ start_pos, __nv_bfloat16* __restrict__ out, int H, int hd,
                               float scale_log2, int window, int chunk_tiles, int n_chunks_max, int out_ld) {
  tlc_pdl(part_o, part_ml, out);
  const int t = blockIdx.x, h = blockIdx.y * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (h >= H) return;
  const int b = row_seq[t];
  const int t0 = cu_seqlens[b], n_new = cu_seqlens[b + 1] - t0;
  const int i0 = ((t - t0) / FA_BM) * FA_BM;
  const int rows = min(FA_BM, n_new - i0);
  const int p0 = start_pos[b] + i0;
  const int tile_hi = (p0 + rows - 1) / FA_BN;
  const int tile_lo = window > 0 ? max(0, p0 + 1 - window) / FA_BN : 0;
  const int n_chunks = (tile_hi - tile_lo) / chunk_tiles + 1;
  if (n_chunks <= 1) return;                         // the row was written whole
  const size_t at = ((size_t)t * H + h) * n_chunks_max;
  float2 ml[FA_MAX_CHUNKS];
#pragma unroll
  for (int z = 0; z < FA_MAX_CHUNKS; z++)
    ml[z] = z < n_chunks ? *reinterpret_cast<const float2*>(part_ml + (at + z) * 2) : make_float2(-INFINITY, 0.f);
  float m = -INFINITY;
#pragma unroll
  for (int z = 0; z < FA_MAX_CHUNKS; z++) if (ml[z].y > 0.f) m = fmaxf(m, ml[z].x);
  float w[FA_MAX_CHUNKS], l = 0.f;
#pragma unroll
  for (int z = 0; z < FA_MAX_CHUNKS; z++) {
    w[z] = ml[z].y > 0.f ? exp2f((ml[z].x - m) * scale_log2) : 0.f;
    l += ml[z].y * w[z];
  }
  const float inv = 1.0f / l;
  for (int d = lane * 4; d < hd; d += 128) {
    float4 v[FA_MAX_CHUNKS];
#pragma unroll
    for (int z = 0; z < FA_MAX_CHUNKS; z++)
      v[z] = (z < n_chunks && w[z] != 0.f) ? *reinterpret_cast<const float4*>(part_o + (at + z) * hd + d) : make_float4(0.f, 0.f, 0.f, 0.f);
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int z = 0; z < FA_MAX_CHUNKS; z++) {
      acc.x = fmaf(v[z].x, w[z], acc.x); acc.y = fmaf(v[z].y, w[z], acc.y);
      acc.z = fmaf(v[z].z, w[z], acc.z); acc.w = fmaf(v[z].w, w[z], acc.w);
    }
    uint2 o2;
    o2.x = pack_bf16(acc.x * inv, acc.y * inv);
    o2.y = pack_bf16(acc.z * inv, acc.w * inv);
    *reinterpret_cast<uint2*>(out + (size_t)t * out_ld + (size_t)h * hd + d) = o2;
  }
}

template <int HD> int fa_configure() {
  const int smem = (FA_BM + 4 * FA_BN) * HD * 2;
  if (cudaFuncSetAttribute(attention_prefill_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess)
    return tlc_fail(-2, "attention(prefill): cannot reserve %d bytes of shared memory", smem);
  return 0;
}

}  // namespace

extern "C" int tlc_attention_prefill_init() {
  if (int rc = fa_configure<64>()) return rc;
  return fa_configure<128>();
}

extern "C" int tlc_attention_prefill_ok(int dtype, int hd) { return dtype == TLC_BF16 && (hd == 64 || hd == 128); }

// How many pieces the key range of a row tile is cut into, for `max_tiles` key tiles at most: none while the
// grid fills the GPU anyway, else pieces of 8 tiles.
extern "C" int tlc_attention_prefill_chunks(int n_tiles_bound, int H, int max_tiles, int* chunk_tiles) {
  const int piece = 8;
  *chunk_tiles = max_tiles > 0 ? max_tiles : 1;
  if (max_tiles <= piece || (long long)n_tiles_bound * H >= 1184) return 1;     // 1184 = 148 SMs x 2 blocks x 4 rounds
  // at most FA_MAX_CHUNKS pieces: longer pieces for very long prompts
  int per = piece;
  while ((max_tiles + per - 1) / per > FA_MAX_CHUNKS) per *= 2;
  *chunk_tiles = per;
  return (max_tiles + per - 1) / per;
}

// n_tiles_bound: an upper bound of sum_b ceil(n_new_b / 64) (e.g. T/64 + n_seqs); max_tiles: key tiles of the
// longest sequence after this step; part_o [T, H, n_chunks, hd] and part_ml [T, H, n_chunks, 2] floats and
// row_seq are needed when tlc_attention_prefill_chunks(...) says more than one piece.
extern "C" int tlc_attention_prefill(const void* q, const void* k_pages, const void* v_pages, const int* block_table,
                                     int max_pages, const int* cu_seqlens, const int* slots, const int* start_pos,
                                     void* out, int n_seqs, int n_tiles_bound, int H, int KV, int hd, float scale,
                                     int window, int max_tiles, const int* row_seq, float* part_o, float* part_ml, int T,
                                     int out_ld, cudaStream_t stream) {
  if (n_seqs == 0 || n_tiles_bound == 0) return 0;
  if (out_ld <= 0) out_ld = H * hd;                      // elements between rows of out (0: dense)
  TLC_REQUIRE(out_ld % 4 == 0, "attention(prefill): rows of the output must start on 8-byte boundaries (stride %d)", out_ld);
  TLC_REQUIRE(KV > 0 && H % KV == 0, "attention: %d heads are not a multiple of %d key/value heads", H, KV);
  TLC_REQUIRE(H <= 65535, "attention(prefill): too many heads (%d)", H);
  int chunk_tiles = 1;
  int n_chunks = tlc_attention_prefill_chunks(n_tiles_bound, H, max_tiles, &chunk_tiles);
  if (part_o == nullptr || part_ml == nullptr || row_seq == nullptr) { n_chunks = 1; chunk_tiles = 1 << 30; }
  if (n_chunks == 1) chunk_tiles = 1 << 30;
  TLC_REQUIRE(n_chunks <= 65535, "attention(prefill): too many pieces (%d)", n_chunks);
  dim3 grid(n_tiles_bound, H, n_chunks);
  const float scale_log2 = scale * 1.4426950408889634f;
  const __nv_bfloat16 *qp = (const __nv_bfloat16*)q, *kp = (const __nv_bfloat16*)k_pages, *vp = (const __nv_bfloat16*)v_pages;
  const int smem = (FA_BM + 4 * FA_BN) * hd * 2;
  if (hd == 64)
    tlc_launch(attention_prefill_kernel<64>, dim3(grid), dim3(128), smem, stream, qp, kp, vp, block_table, max_pages, cu_seqlens, slots, start_pos, (__nv_bfloat16*)out, n_seqs, H, KV, scale_log2, window, chunk_tiles, n_chunks, part_o, part_ml, out_ld);
  else if (hd == 128)
    tlc_launch(attention_prefill_kernel<128>, dim3(grid), dim3(128), smem, stream, qp, kp, vp, block_table, max_pages, cu_seqlens, slots, start_pos, (__nv_bfloat16*)out, n_seqs, H, KV, scale_log2, window, chunk_tiles, n_chunks, part_o, part_ml, out_ld);
  else
    return tlc_fail(-1, "attention(prefill): head size %d is not built (64 and 128 are)", hd);
  if (n_chunks > 1)
    tlc_launch(attention_prefill_merge_kernel, dim3(T, (H + 3) / 4), dim3(128), 0, stream, (const float*)part_o,
               (const float*)part_ml, cu_seqlens, row_seq, start_pos, (__nv_bfloat16*)out, H, hd, scale_log2, window,
               chunk_tiles, n_chunks, out_ld);
  TLC_CHECK_LAUNCH("attention(prefill)");
  return 0;
}
