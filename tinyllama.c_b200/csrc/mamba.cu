// Mamba2 mixer kernels: causal depthwise convolution with its per-sequence window,
// the time-step transform, and the selective state scan with its per-sequence state.
//
// CodeClaper/tinyllama.c states the math on the CPU only: convolution over the last K
// raw samples, tap K-1 on the newest, bias, SiLU, then the window shifts and stores the
// raw sample (cpu_op.c:836-889); dt = softplus(dt + bias), dA = exp(dt*A),
// S = S*dA + B*(x*dt), y = sum_n S*C + x*D (cpu_op.c:924-951).  Here a step carries
// several sequences of unequal length packed back to back; a sequence that starts at
// position 0 starts from a zero window and a zero state, any other continues from its
// slot.  Convolution, dt, the decay and the state are 32-bit.
#include "common.cuh"

#define CONV_MAX_TAPS 16

// ---- convolution + SiLU over packed rows, and softplus / decay of dt ---------------------
// In a bfloat16 run (QUICK) x|B|C are operands of the scan's matrix products: they are rounded to bfloat16
// here, whatever type they are stored in, so that a row's values do not depend on which scan reads them (the
// matrix form of long prompts, the row-by-row scan of short ones and of single-token steps).
template <bool BF16_RUN> __device__ __forceinline__ float as_operand(float v) {
  return BF16_RUN ? __bfloat162float(__float2bfloat16_rn(v)) : v;
}

// grid (ceil(T / 8), ceil(Cd/256)): a thread owns one channel of 8 consecutive rows.  It reads the
// raw samples of those rows and of the K-1 rows before them once (all loads issued together), and
// takes a tap from the sequence's stored window only where the row is among the first K-1 of a
// sequence that continues from a slot.  Also writes dt and dA of the rows (first blocks along y).
// With write_state (every sequence of the step starts at position 0, so that no block reads a stored window)
// the block that holds a sequence's last row also leaves the sequence's new window: its last K-1 raw samples,
// zeros before its first row.  A step with a sequence that continues leaves that to mamba_conv_state_kernel,
// which runs when every reader of the old windows has finished.
#define CONV_ROWS 8
template <typename T, typename TO, int K, bool QUICK>
__global__ void __launch_bounds__(256)
mamba_conv_rows_kernel(const T* __restrict__ proj, int ld, int xbc_off, int dt_off,
                  const float* __restrict__ w, const float* __restrict__ bias,
                  const float* __restrict__ dt_bias, const float* __restrict__ A,
                  const float* __restrict__ conv_state, const int* __restrict__ cu_seqlens,
                  const int* __restrict__ row_seq, const int* __restrict__ slots,
                  const int* __restrict__ start_pos, TO* __restrict__ xbc_out,
                  float* __restrict__ dt_out, float* __restrict__ dA_out, int n_rows, int Cd, int Hs,
                  float* state_out, int write_state) {   // state_out is conv_state, written only when nothing reads it
  tlc_pdl(proj, conv_state, xbc_out, dt_out, dA_out, state_out);
  __shared__ int s_i[CONV_ROWS], s_has[CONV_ROWS], s_slot[CONV_ROWS], s_last[CONV_ROWS], s_plain, s_any_last;
  const int t0 = blockIdx.x * CONV_ROWS;
  if (threadIdx.x == 0) { s_plain = 1; s_any_last = 0; }
  __syncthreads();
  if (threadIdx.x < CONV_ROWS) {
    const int t = t0 + threadIdx.x;
    int i = 0, has = 0, slot = 0, last = 0;
    if (t < n_rows) {
      const int b = row_seq[t];
      i = t - cu_seqlens[b];                          // index of the row inside its sequence's new tokens
      has = start_pos[b] > 0;
      slot = slots[b];
      last = write_state && t == cu_seqlens[b + 1] - 1;
    }
    s_i[threadIdx.x] = i;
    s_has[threadIdx.x] = has;
    s_slot[threadIdx.x] = slot;
    s_last[threadIdx.x] = last;
    if (last) s_any_last = 1;
    // plain: all of the block's rows exist and every tap of every row reads a row of this step
    if (t >= n_rows || i < K - 1) s_plain = 0;
  }
  __syncthreads();
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  // The common block is kept free of the window's address arithmetic and of per-row branches: the kernel is bound by
  // its instruction count, not by memory.  Row t0 + r reads raw rows r .. r + K - 1 (raw[0] is row t0 - (K-1)).
  if (c < Cd && s_plain) {
    const T* src = proj + (size_t)(t0 - (K - 1)) * ld + xbc_off + c;
    float raw[CONV_ROWS + K - 1], wk[K];
#pragma unroll
    for (int q = 0; q < CONV_ROWS + K - 1; q++) raw[q] = to_f32(src[(size_t)q * ld]);
#pragma unroll
    for (int k = 0; k < K; k++) wk[k] = w[(size_t)c * K + k];
    const float bv = bias ? bias[c] : 0.f;
    TO* dst = xbc_out + (size_t)t0 * Cd + c;
#pragma unroll
    for (int r = 0; r < CONV_ROWS; r++) {
      float sum = 0.f;
#pragma unroll
      for (int k = 0; k < K; k++) sum = fmaf(raw[r + k], wk[k], sum);
      dst[(size_t)r * Cd] = from_f32<TO>(as_operand<QUICK>(silu_of<QUICK>(sum + bv)));
    }
  } else if (c < Cd) {
    // raw[q] is the sample of packed row t0 - (K-1) + q; rows before the step's first are never used
    float raw[CONV_ROWS + K - 1], wk[K];
#pragma unroll
    for (int q = 0; q < CONV_ROWS + K - 1; q++) {
      const int t = t0 - (K - 1) + q;
      raw[q] = (t >= 0 && t < n_rows) ? to_f32(proj[(size_t)t * ld + xbc_off + c]) : 0.f;
    }
#pragma unroll
    for (int k = 0; k < K; k++) wk[k] = w[(size_t)c * K + k];
    const float bv = bias ? bias[c] : 0.f;
#pragma unroll
    for (int r = 0; r < CONV_ROWS; r++) {
      const int t = t0 + r;
      if (t >= n_rows) break;
      const int i = s_i[r];
      float sum = 0.f;
      if (i >= K - 1) {
        // every tap reads a row of this step: row t - (K-1-k) is raw row r + k (the common case, kept free of the
        // window's address arithmetic: the kernel is bound by its instruction count, not by memory)
#pragma unroll
        for (int k = 0; k < K; k++) sum = fmaf(raw[r + k], wk[k], sum);
      } else {
#pragma unroll
        for (int k = 0; k < K; k++) {
          const int j = i - (K - 1 - k);              // new-token index that tap k reads
          float x;
          if (j >= 0) x = raw[r + k];
          else x = s_has[r] ? conv_state[((size_t)s_slot[r] * (K - 1) + (K - 1 + j)) * Cd + c] : 0.f;
          sum = fmaf(x, wk[k], sum);
        }
      }
      xbc_out[(size_t)t * Cd + c] = from_f32<TO>(as_operand<QUICK>(silu_of<QUICK>(sum + bv)));
    }
  }
  if (s_any_last && c < Cd) {
    for (int r = 0; r < CONV_ROWS; r++) {
      if (!s_last[r]) continue;
      const int t = t0 + r, n = s_i[r] + 1;           // the sequence's last row and its number of rows
      float* st = state_out + (size_t)s_slot[r] * (K - 1) * Cd + c;
#pragma unroll
      for (int j = 0; j < K - 1; j++)                 // window row j is the sequence's row n - (K-1) + j
        st[(size_t)j * Cd] = j >= K - 1 - n ? to_f32(proj[(size_t)(t - (K - 2) + j) * ld + xbc_off + c]) : 0.f;
    }
  }
  if (c < Hs) {
    const float db = dt_bias[c], Ac = A[c];
#pragma unroll
    for (int r = 0; r < CONV_ROWS; r++) {
      const int t = t0 + r;
      if (t >= n_rows) break;
      const float dtv = softplus_f(to_f32(proj[(size_t)t * ld + dt_off + c]) + db);
      dt_out[(size_t)t * Hs + c] = dtv;
      dA_out[(size_t)t * Hs + c] = expf(dtv * Ac);
    }
  }
}

// Any number of taps: grid (T, ceil(Cd/256)), a thread per (row, channel).
template <typename T, typename TO>
__global__ void mamba_conv_kernel(const T* __restrict__ proj, int ld, int xbc_off, int dt_off,
                                  const float* __restrict__ w, const float* __restrict__ bias,
                                  const float* __restrict__ dt_bias, const float* __restrict__ A,
                                  const float* __restrict__ conv_state, const int* __restrict__ cu_seqlens,
                                  const int* __restrict__ row_seq, const int* __restrict__ slots,
                                  const int* __restrict__ start_pos, TO* __restrict__ xbc_out,
                                  float* __restrict__ dt_out, float* __restrict__ dA_out, int Cd, int K, int Hs,
                                  int bf16_run) {
  tlc_pdl(proj, conv_state, xbc_out, dt_out, dA_out);
  const int t = blockIdx.x;
  const int b = row_seq[t];
  const int i = t - cu_seqlens[b];                  // index of this row inside its sequence's new tokens
  const bool has_state = start_pos[b] > 0;
  const float* st = conv_state + (size_t)slots[b] * (K - 1) * Cd;
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c < Cd) {
    float sum = 0.f;
    for (int k = 0; k < K; k++) {
      const int j = i - (K - 1 - k);                // new-token index that tap k reads
      float x;
      if (j >= 0) x = to_f32(proj[(size_t)(t - (K - 1 - k)) * ld + xbc_off + c]);
      else x = has_state ? st[(size_t)(K - 1 + j) * Cd + c] : 0.f;
      sum = fmaf(x, w[(size_t)c * K + k], sum);
    }
    if (bias) sum += bias[c];
    const float v = silu_f(sum);
    xbc_out[(size_t)t * Cd + c] = from_f32<TO>(bf16_run ? as_operand<true>(v) : v);
  }
  if (c < Hs) {
    const float dtv = softplus_f(to_f32(proj[(size_t)t * ld + dt_off + c]) + dt_bias[c]);
    dt_out[(size_t)t * Hs + c] = dtv;
    dA_out[(size_t)t * Hs + c] = expf(dtv * A[c]);
  }
}

// New window of each sequence: its last K-1 raw samples (old window rows where the step
// brought fewer).  One thread owns one (sequence, channel), reads all it needs, then writes.
template <typename T>
__global__ void mamba_conv_state_kernel(const T* __restrict__ proj, int ld, int xbc_off, float* __restrict__ conv_state,
                                        const int* __restrict__ cu_seqlens, const int* __restrict__ slots,
                                        const int* __restrict__ start_pos, int Cd, int K) {
  tlc_pdl(proj, conv_state);
  const int b = blockIdx.x;
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= Cd) return;
  const int t0 = cu_seqlens[b], n = cu_seqlens[b + 1] - t0;
  if (n == 0) return;
  const bool has_state = start_pos[b] > 0;
  float* st = conv_state + (size_t)slots[b] * (K - 1) * Cd;
  float v[CONV_MAX_TAPS];
#pragma unroll
  for (int j = 0; j < CONV_MAX_TAPS; j++) {
    if (j < K - 1) {
      const int idx = n - (K - 1) + j;              // new-token index that lands in window row j
      if (idx >= 0) v[j] = to_f32(proj[(size_t)(t0 + idx) * ld + xbc_off + c]);
      else v[j] = has_state ? st[(size_t)(K - 1 + idx) * Cd + c] : 0.f;
    }
  }
#pragma unroll
  for (int j = 0; j < CONV_MAX_TAPS; j++)
    if (j < K - 1) st[(size_t)j * Cd + c] = v[j];
}

// One-token steps: every sequence brings exactly one row, so a thread owns one (sequence, channel):
// it reads the window, convolves, and writes the shifted window back -- one kernel instead of two.
// KT: the number of taps when it is 2, 3 or 4 (the window then takes KT - 1 registers instead of the limit's 16),
// else 0 and K is read at run time.
template <typename T, int KT>
__global__ void mamba_conv_decode_kernel(const T* __restrict__ proj, int ld, int xbc_off, int dt_off,
                                         const float* __restrict__ w, const float* __restrict__ bias,
                                         const float* __restrict__ dt_bias, const float* __restrict__ A,
                                         float* __restrict__ conv_state, const int* __restrict__ slots,
                                         const int* __restrict__ start_pos, float* __restrict__ xbc_out,
                                         float* __restrict__ dt_out, float* __restrict__ dA_out, int Cd, int K, int Hs,
                                         int bf16_run) {
  constexpr int TAPS = KT > 0 ? KT - 1 : CONV_MAX_TAPS;     // window rows held in registers
  if (KT > 0) K = KT;
  // The window was stored by the step before and the weights never change: both are fetched before the
  // wait on the previous kernel; only the row's projection is read after it.
  asm volatile("griddepcontrol.launch_dependents;");
  const int b = blockIdx.x;                          // row b belongs to sequence b
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  const bool has_state = start_pos[b] > 0;
  float* st = conv_state + (size_t)slots[b] * (K - 1) * Cd;
  float prev[TAPS], wk[TAPS + 1];
  float bv = 0.f, db = 0.f, Ac = 0.f;
  if (c < Cd) {
#pragma unroll
    for (int k = 0; k < TAPS; k++) {
      prev[k] = (k < K - 1 && has_state) ? st[(size_t)k * Cd + c] : 0.f;
      wk[k] = k < K ? w[(size_t)c * K + k] : 0.f;
    }
    wk[TAPS] = TAPS < K ? w[(size_t)c * K + TAPS] : 0.f;
    if (bias) bv = bias[c];
  }
  if (c < Hs) { db = dt_bias[c]; Ac = A[c]; }
  tlc_wait(proj, xbc_out, dt_out, dA_out);
  if (c < Cd) {
    const float cur = to_f32(proj[(size_t)b * ld + xbc_off + c]);
    float sum = bv;
#pragma unroll
    for (int k = 0; k < TAPS; k++)
      if (k < K - 1) sum = fmaf(prev[k], wk[k], sum);
    float wl = 0.f;
#pragma unroll
    for (int k = 0; k <= TAPS; k++) if (k == K - 1) wl = wk[k];
    sum = fmaf(cur, wl, sum);
    const float v = silu_f(sum);
    xbc_out[(size_t)b * Cd + c] = bf16_run ? as_operand<true>(v) : v;
#pragma unroll
    for (int k = 0; k < TAPS; k++) {
      if (k < K - 2) st[(size_t)k * Cd + c] = prev[k + 1];
      else if (k == K - 2) st[(size_t)k * Cd + c] = cur;
    }
  }
  if (c < Hs) {
    const float dtv = softplus_f(to_f32(proj[(size_t)b * ld + dt_off + c]) + db);
    dt_out[(size_t)b * Hs + c] = dtv;
    dA_out[(size_t)b * Hs + c] = expf(dtv * Ac);
  }
}

#define TLC_CONV_ROWS_Q(KT, QK)                                                                                        \
  tlc_launch(mamba_conv_rows_kernel<TT, TO, KT, QK>, dim3(grid8), dim3(256), 0, stream, (const TT*)proj, ld, xbc_off,  \
             dt_off, w, bias, dt_bias, A, conv_state, cu_seqlens, row_seq, slots, start_pos, (TO*)xbc_out, dt_out,     \
             dA_out, T, Cd, Hs, conv_state, fused_state)
#define TLC_CONV_ROWS(KT) do { if (quick) TLC_CONV_ROWS_Q(KT, true); else TLC_CONV_ROWS_Q(KT, false); } while (0)
// xbc_dtype: the element type of xbc_out [T, Cd].  Single-token steps and the 32-bit scans take float; the scan
// of prompts in matrix form takes its operands in bfloat16 and gets them in that type at once.
extern "C" int tlc_mamba_conv(const void* proj, int dtype, int ld, int xbc_off, int dt_off, const float* w,
                              const float* bias, const float* dt_bias, const float* A, float* conv_state,
                              const int* cu_seqlens, const int* row_seq, const int* slots, const int* start_pos,
                              void* xbc_out, int xbc_dtype, float* dt_out, float* dA_out, int T, int B, int Cd, int K,
                              int Hs, int single_rows, int quick, int all_fresh, cudaStream_t stream) {
  if (T == 0) return 0;
  // every sequence starts at position 0: nothing reads a stored window, and the rows' kernel writes the new ones
  const int fused_state = all_fresh && K >= 2 && K <= 4;
  TLC_REQUIRE(K >= 1 && K - 1 <= CONV_MAX_TAPS, "mamba_conv: %d taps exceed the kernel's limit of %d", K, CONV_MAX_TAPS + 1);
  TLC_REQUIRE(Hs <= Cd, "mamba_conv: more heads (%d) than conv channels (%d)", Hs, Cd);
  dim3 grid(T, (Cd + 255) / 256);
  dim3 grid8((T + CONV_ROWS - 1) / CONV_ROWS, (Cd + 255) / 256);
  dim3 grid2(B, (Cd + 255) / 256);
  if (single_rows && T == B) {
    TLC_REQUIRE(xbc_dtype == TLC_F32, "mamba_conv: single-token steps write 32-bit x|B|C");
#define TLC_CONV_DECODE(KT)                                                                                          \
  tlc_launch(mamba_conv_decode_kernel<TT, KT>, dim3(grid2), dim3(256), 0, stream, (const TT*)proj, ld, xbc_off, dt_off, w,  \
             bias, dt_bias, A, conv_state, slots, start_pos, (float*)xbc_out, dt_out, dA_out, Cd, K, Hs, quick)
    TLC_DISPATCH_DTYPE(dtype, TT, {
      if (K == 4) TLC_CONV_DECODE(4);
      else if (K == 3) TLC_CONV_DECODE(3);
      else if (K == 2) TLC_CONV_DECODE(2);
      else TLC_CONV_DECODE(0);
    });
#undef TLC_CONV_DECODE
    TLC_CHECK_LAUNCH("mamba_conv(decode)");
    return 0;
  }
  TLC_DISPATCH_DTYPE(dtype, TT, TLC_DISPATCH_DTYPE(xbc_dtype, TO, {
    if (K == 4) TLC_CONV_ROWS(4);
    else if (K == 3) TLC_CONV_ROWS(3);
    else if (K == 2) TLC_CONV_ROWS(2);
    else
      tlc_launch(mamba_conv_kernel<TT, TO>, dim3(grid), dim3(256), 0, stream, (const TT*)proj, ld, xbc_off, dt_off, w, bias,
                 dt_bias, A, conv_state, cu_seqlens, row_seq, slots, start_pos, (TO*)xbc_out, dt_out, dA_out, Cd, K, Hs, quick);
    if (K > 1 && !fused_state)
      tlc_launch(mamba_conv_state_kernel<TT>, dim3(grid2), dim3(256), 0, stream, (const TT*)proj, ld, xbc_off, conv_state,
                 cu_seqlens, slots, start_pos, Cd, K);
  }));
  TLC_CHECK_LAUNCH("mamba_conv");
  return 0;
}

// ---- selective scan ---------------------------------------------------------------------------
// The scan runs over *segments* of consecutive rows.  In the plain mode a segment is a whole
// sequence: it starts from its slot's state (zero at position 0) and leaves its final state there.
// Long prompts are cut into chunks that run in parallel, in three passes:
//   1. every chunk from a zero state, keeping only its final state  S_c           (mode 1)
//   2. per sequence, in chunk order: S_in[c] = S_in[c-1] * decay[c-1] + S_[c-1]    (state pass)
//   3. every chunk again from its true incoming state S_in[c], now writing y      (mode 3)
// which is the same recurrence, because the state is linear in its initial value.
//
// grid (segment, Hs, ceil(P / (4*RP))), 128 threads: each warp owns RP rows p of one head's state
// [P, N], each lane the columns lane, lane+32, ... (NPL of them) in registers.  Rows run in
// order; the inputs of SCAN_TT rows are staged in shared memory at a time.
#define SCAN_TT 8
#define SCAN_PLAIN 0
#define SCAN_CHUNK_STATE 1
#define SCAN_CHUNK_OUT 3
template <int NPL, int RP>
__global__ void __launch_bounds__(128)
ssm_scan_kernel(const float* __restrict__ xbc, const float* __restrict__ dt, const float* __restrict__ dA,
                const float* __restrict__ Dskip, float* __restrict__ state, float* __restrict__ chunk_state,
                const int* __restrict__ seg_start, const int* __restrict__ seg_seq,
                const int* __restrict__ seq_seg_start, const int* __restrict__ slots,
                const int* __restrict__ start_pos, float* __restrict__ y, float* __restrict__ chunk_decay, int mode,
                int Hs, int P, int N, int G, int Cd) {
  // In the plain mode the state this block starts from was written by an earlier step, not by
  // the kernel before this one: it is fetched before the wait on that kernel (see tlc_pdl).
  asm volatile("griddepcontrol.launch_dependents;");
  if (mode != SCAN_PLAIN) tlc_wait(xbc, dt, dA, state, chunk_state, y, chunk_decay);
  extern __shared__ float sm[];
  const int seg = blockIdx.x, h = blockIdx.y;
  const int b = seg_seq ? seg_seq[seg] : seg;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int rows_per_block = 4 * RP;
  const int p_blk = blockIdx.z * rows_per_block;
  const int p_base = p_blk + warp * RP;
  const int Di = Hs * P;
  const int g = h / (Hs / G);
  const int t0 = seg_start[seg], n_tok = seg_start[seg + 1] - t0;
  if (n_tok == 0) return;
  float* S_slot = state + (((size_t)slots[b] * Hs + h) * P) * N;
  float* S_chunk = chunk_state ? chunk_state + (((size_t)seg * Hs + h) * P) * N : nullptr;
  const float* S_init = nullptr;
  if (mode == SCAN_PLAIN) { if (start_pos[b] > 0) S_init = S_slot; }
  else if (mode == SCAN_CHUNK_OUT) S_init = S_chunk;
  float* S_final = nullptr;
  if (mode == SCAN_PLAIN) S_final = S_slot;
  else if (mode == SCAN_CHUNK_STATE) S_final = S_chunk;
  else if (seg + 1 == seq_seg_start[b + 1]) S_final = S_slot;        // the sequence's last chunk
  const bool want_y = mode != SCAN_CHUNK_STATE;
  // A lane owns the columns lane, lane + 32, ... of its rows, or (VEC: more than 64 columns, a multiple of 4)
  // four consecutive columns 4 lane + 128 jj, which it loads and stores 16 bytes at a time.
  const bool VEC = NPL % 4 == 0 && N % 4 == 0;
  auto col = [&](int j) { return VEC ? 4 * lane + 128 * (j >> 2) + (j & 3) : lane + 32 * j; };
  float s[RP][NPL];
#pragma unroll
  for (int r = 0; r < RP; r++) {
    const int p = p_base + r;
    if (VEC) {
#pragma unroll
      for (int jj = 0; jj < NPL / 4; jj++) {
        const int n = 4 * lane + 128 * jj;
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (S_init && p < P && n < N) v = *reinterpret_cast<const float4*>(S_init + (size_t)p * N + n);
        s[r][4 * jj] = v.x; s[r][4 * jj + 1] = v.y; s[r][4 * jj + 2] = v.z; s[r][4 * jj + 3] = v.w;
      }
    } else {
#pragma unroll
      for (int j = 0; j < NPL; j++) {
        const int n = lane + 32 * j;
        s[r][j] = (S_init && p < P && n < N) ? S_init[(size_t)p * N + n] : 0.f;
      }
    }
  }
  if (mode == SCAN_PLAIN) tlc_wait(xbc, dt, dA, y);
  // shared staging: per row  B[N] | C[N] | x[rows_per_block] | dt | dA
  const int per_tok = 2 * N + rows_per_block + 2;
  const float Dh = Dskip[h];
  for (int tt0 = 0; tt0 < n_tok; tt0 += SCAN_TT) {
    const int nt = min(SCAN_TT, n_tok - tt0);
    __syncthreads();
    for (int k = 0; k < nt; k++) {
      const float* row = xbc + (size_t)(t0 + tt0 + k) * Cd;
      float* dst = sm + (size_t)k * per_tok;
      const float* Bg = row + Di + (size_t)g * N;
      const float* Cg = row + Di + (size_t)G * N + (size_t)g * N;
      for (int e = threadIdx.x; e < N; e += blockDim.x) {
        dst[e] = Bg[e];
        dst[N + e] = want_y ? Cg[e] : 0.f;
      }
      if (threadIdx.x < rows_per_block) {
        const int p = p_blk + threadIdx.x;
        dst[2 * N + threadIdx.x] = p < P ? row[(size_t)h * P + p] : 0.f;
      } else if (threadIdx.x == 32 + rows_per_block) {
        dst[2 * N + rows_per_block] = dt[(size_t)(t0 + tt0 + k) * Hs + h];
      } else if (threadIdx.x == 64 + rows_per_block) {
        dst[2 * N + rows_per_block + 1] = dA[(size_t)(t0 + tt0 + k) * Hs + h];
      }
    }
    __syncthreads();
    for (int k = 0; k < nt; k++) {
      const float* tk = sm + (size_t)k * per_tok;
      const float dtv = tk[2 * N + rows_per_block], dAv = tk[2 * N + rows_per_block + 1];
      float Bv[NPL], Cv[NPL];
#pragma unroll
      for (int j = 0; j < NPL; j++) {
        const int n = col(j);
        Bv[j] = n < N ? tk[n] : 0.f;
        Cv[j] = n < N ? tk[N + n] : 0.f;
      }
      if (want_y) {
#pragma unroll
        for (int r = 0; r < RP; r++) {
          const float xv = tk[2 * N + warp * RP + r];
          const float xdt = xv * dtv;
          float sum = 0.f;
#pragma unroll
          for (int j = 0; j < NPL; j++) {
            const float sv = fmaf(s[r][j], dAv, Bv[j] * xdt);
            s[r][j] = sv;
            sum = fmaf(sv, Cv[j], sum);
          }
          sum = warp_sum(sum);
          const int p = p_base + r;
          if (lane == 0 && p < P) y[(size_t)(t0 + tt0 + k) * Di + (size_t)h * P + p] = sum + xv * Dh;
        }
      } else {
#pragma unroll
        for (int r = 0; r < RP; r++) {
          const float xdt = tk[2 * N + warp * RP + r] * dtv;
#pragma unroll
          for (int j = 0; j < NPL; j++) s[r][j] = fmaf(s[r][j], dAv, Bv[j] * xdt);
        }
      }
    }
  }
  if (mode == SCAN_CHUNK_STATE && blockIdx.z == 0 && threadIdx.x == 0) {
    float d = 1.f;                         // decay of the whole chunk: the product of its rows' decays
    for (int k = 0; k < n_tok; k++) d *= dA[(size_t)(t0 + k) * Hs + h];
    chunk_decay[(size_t)seg * Hs + h] = d;
  }
  if (S_final) {
#pragma unroll
    for (int r = 0; r < RP; r++) {
      const int p = p_base + r;
      if (VEC) {
#pragma unroll
        for (int jj = 0; jj < NPL / 4; jj++) {
          const int n = 4 * lane + 128 * jj;
          if (p < P && n < N)
            *reinterpret_cast<float4*>(S_final + (size_t)p * N + n) =
                make_float4(s[r][4 * jj], s[r][4 * jj + 1], s[r][4 * jj + 2], s[r][4 * jj + 3]);
        }
      } else {
#pragma unroll
        for (int j = 0; j < NPL; j++) {
          const int n = lane + 32 * j;
          if (p < P && n < N) S_final[(size_t)p * N + n] = s[r][j];
        }
      }
    }
  }
}

// Pass 2: carries the state through a sequence's chunks.  chunk_state[c] holds the chunk's own
// contribution on entry and the state *before* the chunk on exit.  grid (B, Hs, blocks over P*N).
// With write_final the state after the last chunk goes to the sequence's slot.
__global__ void __launch_bounds__(256)
ssm_state_pass_kernel(const float* __restrict__ chunk_decay, float* __restrict__ state,
                      float* __restrict__ chunk_state, const int* __restrict__ seq_seg_start,
                      const int* __restrict__ slots, const int* __restrict__ start_pos, int Hs, int PN, int write_final) {
  tlc_pdl(chunk_decay, state, chunk_state);
  const int b = blockIdx.x, h = blockIdx.y;
  const int e = blockIdx.z * blockDim.x + threadIdx.x;
  const int c0 = seq_seg_start[b], c1 = seq_seg_start[b + 1];
  if (c1 - c0 <= 0 || e >= PN) return;
  float* slot = state + ((size_t)slots[b] * Hs + h) * PN + e;
  float s = start_pos[b] > 0 ? *slot : 0.f;
  constexpr int BATCH = 16;                // chunks whose values are fetched together
  for (int cb = c0; cb < c1; cb += BATCH) {
    float own[BATCH], decay[BATCH];
#pragma unroll
    for (int i = 0; i < BATCH; i++) {
      const int c = cb + i;
      own[i] = c < c1 ? chunk_state[((size_t)c * Hs + h) * PN + e] : 0.f;
      decay[i] = c < c1 ? chunk_decay[(size_t)c * Hs + h] : 1.f;
    }
#pragma unroll
    for (int i = 0; i < BATCH; i++) {
      const int c = cb + i;
      if (c < c1) {
        chunk_state[((size_t)c * Hs + h) * PN + e] = s;
        s = fmaf(s, decay[i], own[i]);
      }
    }
  }
  if (write_final) *slot = s;
}

// The same with four state elements a thread (16-byte loads and stores), for state sizes that are multiples of 4.
__global__ void __launch_bounds__(256)
ssm_state_pass_vec_kernel(const float* __restrict__ chunk_decay, float* __restrict__ state,
                          float* __restrict__ chunk_state, const int* __restrict__ seq_seg_start,
                          const int* __restrict__ slots, const int* __restrict__ start_pos, int Hs, int PN, int write_final) {
  tlc_pdl(chunk_decay, state, chunk_state);
  const int b = blockIdx.x, h = blockIdx.y;
  const int e = 4 * (blockIdx.z * blockDim.x + threadIdx.x);
  const int c0 = seq_seg_start[b], c1 = seq_seg_start[b + 1];
  if (c1 - c0 <= 0 || e >= PN) return;
  float4* slot = reinterpret_cast<float4*>(state + ((size_t)slots[b] * Hs + h) * PN + e);
  float4 s = start_pos[b] > 0 ? *slot : make_float4(0.f, 0.f, 0.f, 0.f);
  constexpr int BATCH = 16;                // chunks whose values are fetched together
  for (int cb = c0; cb < c1; cb += BATCH) {
    float4 own[BATCH];
    float decay[BATCH];
#pragma unroll
    for (int i = 0; i < BATCH; i++) {
      const int c = cb + i;
      own[i] = c < c1 ? *reinterpret_cast<const float4*>(chunk_state + ((size_t)c * Hs + h) * PN + e) : make_float4(0.f, 0.f, 0.f, 0.f);
      decay[i] = c < c1 ? chunk_decay[(size_t)c * Hs + h] : 1.f;
    }
#pragma unroll
    for (int i = 0; i < BATCH; i++) {
      const int c = cb + i;
      if (c < c1) {
        *reinterpret_cast<float4*>(chunk_state + ((size_t)c * Hs + h) * PN + e) = s;
        s = make_float4(fmaf(s.x, decay[i], own[i].x), fmaf(s.y, decay[i], own[i].y), fmaf(s.z, decay[i], own[i].z),
                        fmaf(s.w, decay[i], own[i].w));
      }
    }
  }
  if (write_final) *slot = s;
}

int tlc_ssm_state_pass_launch(const float* chunk_decay, float* state, float* chunk_state, const int* seq_seg_start,
                              const int* slots, const int* start_pos, int B, int Hs, int PN, int write_final,
                              cudaStream_t stream) {
  if (PN % 4 == 0 && ((uintptr_t)state % 16) == 0 && ((uintptr_t)chunk_state % 16) == 0) {
    dim3 grid(B, Hs, (PN / 4 + 255) / 256);
    tlc_launch(ssm_state_pass_vec_kernel, grid, dim3(256), 0, stream, chunk_decay, state, chunk_state, seq_seg_start, slots,
               start_pos, Hs, PN, write_final);
    TLC_CHECK_LAUNCH("ssm_state_pass");
    return 0;
  }
  dim3 grid(B, Hs, (PN + 255) / 256);
  tlc_launch(ssm_state_pass_kernel, grid, dim3(256), 0, stream, chunk_decay, state, chunk_state, seq_seg_start, slots,
             start_pos, Hs, PN, write_final);
  TLC_CHECK_LAUNCH("ssm_state_pass");
  return 0;
}

template <int NPL>
static int launch_scan(const float* xbc, const float* dt, const float* dA, const float* Dskip, float* state,
                       float* chunk_state, const int* seg_start, const int* seg_seq, const int* seq_seg_start,
                       const int* slots, const int* start_pos, float* y, float* chunk_decay, int mode, int n_seg, int Hs,
                       int P, int N, int G, int Cd, cudaStream_t stream) {
  constexpr int RP = 4;
  dim3 grid(n_seg, Hs, (P + 4 * RP - 1) / (4 * RP));
  const size_t smem = (size_t)SCAN_TT * (2 * N + 4 * RP + 2) * sizeof(float);
  tlc_launch(ssm_scan_kernel<NPL, RP>, dim3(grid), dim3(128), smem, stream, xbc, dt, dA, Dskip, state, chunk_state, seg_start, seg_seq,
                                                        seq_seg_start, slots, start_pos, y, chunk_decay, mode, Hs, P, N, G,
                                                        Cd);
  TLC_CHECK_LAUNCH("ssm_scan");
  return 0;
}

static int scan_dispatch(const float* xbc, const float* dt, const float* dA, const float* Dskip, float* state,
                         float* chunk_state, const int* seg_start, const int* seg_seq, const int* seq_seg_start,
                         const int* slots, const int* start_pos, float* y, float* chunk_decay, int mode, int n_seg,
                         int Hs, int P, int N, int G, int Cd, cudaStream_t stream) {
#define TLC_SCAN(NPL) launch_scan<NPL>(xbc, dt, dA, Dskip, state, chunk_state, seg_start, seg_seq, seq_seg_start, slots, start_pos, y, chunk_decay, mode, n_seg, Hs, P, N, G, Cd, stream)
  if (N <= 32) return TLC_SCAN(1);
  if (N <= 64) return TLC_SCAN(2);
  if (N <= 128) return TLC_SCAN(4);
  return TLC_SCAN(8);
#undef TLC_SCAN
}

static int scan_checks(int Hs, int N, int G) {
  TLC_REQUIRE(G > 0 && Hs % G == 0, "ssm_scan: %d heads are not a multiple of %d groups", Hs, G);
  TLC_REQUIRE(N >= 1 && N <= 256, "ssm_scan: state size %d is outside the kernel's range 1..256", N);
  TLC_REQUIRE(Hs <= 65535, "ssm_scan: too many heads (%d)", Hs);
  return 0;
}

extern "C" int tlc_ssm_scan(const float* xbc, const float* dt, const float* dA, const float* Dskip, float* state,
                            const int* cu_seqlens, const int* slots, const int* start_pos, float* y, int B, int Hs,
                            int P, int N, int G, int Cd, cudaStream_t stream) {
  if (B == 0) return 0;
  if (int rc = scan_checks(Hs, N, G)) return rc;
  return scan_dispatch(xbc, dt, dA, Dskip, state, nullptr, cu_seqlens, nullptr, nullptr, slots, start_pos, y, nullptr,
                       SCAN_PLAIN, B, Hs, P, N, G, Cd, stream);
}

// The same scan with every sequence cut into chunks that run in parallel.  seg_start [n_seg + 1]:
// first row of every chunk; seg_seq [n_seg]: its sequence; seq_seg_start [B + 1]: first chunk of
// every sequence; chunk_state: scratch [n_seg, Hs, P, N] + [n_seg, Hs] floats.
extern "C" int tlc_ssm_scan_chunked(const float* xbc, const float* dt, const float* dA, const float* Dskip,
                                    float* state, float* chunk_state, const int* seg_start, const int* seg_seq,
                                    const int* seq_seg_start, const int* slots, const int* start_pos, float* y,
                                    int B, int n_seg, int Hs, int P, int N, int G, int Cd, cudaStream_t stream) {
  if (B == 0 || n_seg == 0) return 0;
  if (int rc = scan_checks(Hs, N, G)) return rc;
  float* chunk_decay = chunk_state + (size_t)n_seg * Hs * P * N;
  if (int rc = scan_dispatch(xbc, dt, dA, Dskip, state, chunk_state, seg_start, seg_seq, seq_seg_start, slots, start_pos,
                             y, chunk_decay, SCAN_CHUNK_STATE, n_seg, Hs, P, N, G, Cd, stream)) return rc;
  if (int rc = tlc_ssm_state_pass_launch(chunk_decay, state, chunk_state, seq_seg_start, slots, start_pos, B, Hs, P * N, 0,
                                         stream)) return rc;
  return scan_dispatch(xbc, dt, dA, Dskip, state, chunk_state, seg_start, seg_seq, seq_seg_start, slots, start_pos, y,
                       chunk_decay, SCAN_CHUNK_OUT, n_seg, Hs, P, N, G, Cd, stream);
}
