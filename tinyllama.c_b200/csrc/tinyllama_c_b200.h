/* tinyllama_c_b200.h -- the C interface of libtinyllama_c_b200.so (CUDA kernels for sm_100a).
 *
 * CodeClaper/tinyllama.c's programming interface is a pair of headers: core.h:19-52 (engine_open,
 * session_create, ...) and graph.h:51-109 (the op builders and graph_execute).  This header plays that
 * role for the kernel library: every function the shared library exports is declared here, every .cu
 * file includes it (so the compiler holds each definition to its declaration), and the Python package
 * loads the library with ctypes from a table that a test compares with these prototypes.
 *
 * Conventions
 *   * Every pointer is DEVICE memory unless its comment says "host".  Nothing here allocates on behalf of
 *     the caller except the set-up functions (tlc_*_init), which must run before any stream capture.
 *   * A function that launches work returns 0, or a negative code after storing a message that
 *     tlc_last_error() returns (thread-local).  Nothing exits, traps or prints.
 *   * dtype codes: TLC_F32 = 0 (float), TLC_BF16 = 1 (bfloat16).  A "ld" argument is a row stride in
 *     elements.  All launches go to the given stream and return without waiting.
 *   * A batch is packed: row t of the step belongs to sequence row_seq[t] (0..B-1), which owns rows
 *     cu_seqlens[b] .. cu_seqlens[b+1]-1, sits in cache slot slots[b] and began this step at position
 *     start_pos[b]; positions[t] is the row's absolute position.  All of these are int32.
 *   * Keys and values live in pages of TLC_PAGE positions: [n_pages, KV, TLC_PAGE, hd]; block_table
 *     [n_slots, max_pages] gives the page of every TLC_PAGE positions of a slot.
 *   * Softmax, norms, rotation angles, decay factors, states and all accumulators are 32-bit.
 */
#ifndef TINYLLAMA_C_B200_H
#define TINYLLAMA_C_B200_H

#include <cuda_runtime_api.h>

#define TLC_F32 0
#define TLC_BF16 1
#define TLC_PAGE 64

#ifdef __cplusplus
extern "C" {
#endif

/* ---- library state ------------------------------------------------------------------------------- */
/* Message of the last failed call of this thread. */
const char* tlc_last_error(void);
/* 1: launches carry the programmatic-serialization attribute (a kernel's blocks are scheduled while its
 * predecessor drains); 0: plain stream order.  The embedding kernel never carries it: it is the boundary
 * between steps (see tlc_embed). */
void tlc_set_pdl(int on);
/* Set-up of the tensor-core products, of prompt attention and of the chunked scan (shared-memory
 * attributes, the driver's tensor-map encoder, the error words, scratch).  Once per process, before any
 * stream capture. */
int tlc_linear_init(void);
int tlc_attention_prefill_init(void);
int tlc_ssd_init(void);
/* Error word of kernels whose waits are bounded: 0, or the code of the wait that ran out (1 loader,
 * 2 issuer, 3 epilogue, 4 drain, 5 accumulator of the tcgen05 product; 9 the self-test).  Reading does
 * not synchronise; clear sets it back to 0. */
int tlc_linear_error(void);
void tlc_linear_error_clear(void);
/* How many clock cycles a bounded wait may spin before it gives up (0: the default, about a second). */
int tlc_wait_limit_cycles(long long cycles);
/* Self-test of the error channel: one block waits, bounded, on a barrier that nobody arrives at, records
 * code 9 when the wait runs out, and returns.  It never traps and never spins beyond the limit. */
int tlc_selftest_bounded_wait(cudaStream_t stream);

/* ---- embedding, norms, activations (elementwise.cu) ---------------------------------------------- */
/* out[t] = table[tokens[t]] * scale; out float [T, D].  The first kernel of a step: it is launched with a
 * full dependency on all earlier work of the stream, which is what lets later kernels of the step fetch
 * cache contents of earlier steps ahead of their own dependency wait. */
int tlc_embed(const int* tokens, const void* table, int table_dtype, int T, int D, int V, float scale,
              float* out, cudaStream_t stream);
/* out[r] = x[rows ? rows[r] : r] / sqrt(mean(x^2) + eps) * w;  x float [*, D], out [R, D] of out_dtype. */
int tlc_rmsnorm(const float* x, const int* rows, const float* w, float eps, int R, int D, void* out,
                int out_dtype, cudaStream_t stream);
/* Gate y (+ y2, where y2 is not NULL: an input that comes as two summands) by silu(z) and RMS-normalise per group,
 * in either order; w NULL: gate only.  out [T, Di] with row stride out_ld, multiplied by out_scale. */
int tlc_gated_rmsnorm(const float* y, const float* y2, const void* z, int z_dtype, int ldz, const float* w, float eps, int T,
                      int Di, int n_groups, int norm_before_gate, void* out, int out_dtype, int out_ld,
                      float out_scale, cudaStream_t stream);
/* out[T, F] = silu(gate) * up; gu holds gate | up as halves, or (interleave) 8 gates then their 8 ups. */
int tlc_swiglu(const void* gu, int in_dtype, int ld, int F, int T, void* out, int dtype, int interleave,
               cudaStream_t stream);
int tlc_gather_rows(const float* x, const int* rows, int R, int D, float* out, cudaStream_t stream);

/* ---- linear layers (gemm_tcgen05.cu, gemm_simt.cu) ----------------------------------------------------
 * out[m, n] (+)= (sum_k a[m, k] w[n, k]) * colscale[n] + colbias[n];  a [M, K], w [N, K], 32-bit sums.
 * tlc_linear chooses: bfloat16 operands go to the tcgen05 kernel (TMA -> shared memory -> tensor memory)
 * from min_rows_for_tensor_cores rows on, to the weight-streaming mma.sync kernel below that; float
 * operands run on the CUDA cores in true 32-bit arithmetic (tlc_linear_simt). */
int tlc_linear(const void* a, int a_dtype, int lda, const void* w, int w_dtype, int ldw, void* out,
               int out_dtype, int ldo, const float* colscale, const float* colbias, int accumulate, int M,
               int N, int K, int min_rows_for_tensor_cores, cudaStream_t stream);
/* out[M, N/2] = silu(gate) * up where the rows of w come in groups of 16 (8 gate rows, their 8 up rows).
 * Returns 1 when no fused kernel takes the operands (run tlc_linear and tlc_swiglu instead). */
int tlc_linear_swiglu(const void* a, int a_dtype, int lda, const void* w, int w_dtype, int ldw, void* out,
                      int out_dtype, int ldo, const float* colscale, const float* colbias, int M, int N, int K,
                      int min_rows_for_tensor_cores, cudaStream_t stream);
int tlc_linear_simt(const void* a, int a_dtype, int lda, const void* w, int w_dtype, int ldw, void* out,
                    int out_dtype, int ldo, const float* colscale, const float* colbias, int accumulate,
                    int M, int N, int K, cudaStream_t stream);
// The product for 17..64 rows (weights on the 128-row side of tcgen05.mma, K shared among the blocks of a cluster).
void tlc_linear_few_rows(int on);          // 0: never this kernel (for comparisons)
void tlc_linear_few_rows_split(int split); // 0: the number of blocks per tile is chosen; 1, 2, 4, 8: fixed (for tests)
void tlc_linear_few_rows_min_tiles(int tiles);   // outputs of fewer tiles of 128 weight rows stay with the other kernels (0: 16 tiles with more than 32 rows, else 32)
void tlc_linear_few_rows_max_rows(int rows);     // products of more rows go to the tiles of the prompt product (128; for comparisons)
int tlc_linear_few_rows_ok(int a_dtype, int lda, const void* a, int w_dtype, int ldw, const void* w, int M, int N, int K);
void tlc_linear_tma_out(int on);        // 0: the tensor-core product's 32-bit outputs never leave through the copy engine (for comparisons)
void tlc_linear_skinny_pairs(int on);   // 0: the skinny product never splits K over a pair of blocks (for comparisons)
int tlc_linear_skinny_ok(int a_dtype, int lda, const void* a, int w_dtype, int ldw, const void* w, int M, int K);
int tlc_linear_skinny(const void* a, int lda, const void* w, int ldw, void* out, int out_dtype, int ldo,
                      const float* colscale, const float* colbias, int accumulate, int M, int N, int K,
                      cudaStream_t stream);
int tlc_linear_skinny_swiglu(const void* a, int lda, const void* w, int ldw, void* out, int out_dtype, int ldo,
                             const float* colscale, const float* colbias, int M, int N, int K,
                             cudaStream_t stream);
int tlc_linear_tcgen05_ok(int a_dtype, int lda, const void* a, int w_dtype, int ldw, const void* w, int K);
/* Test hooks: force the tile width (0, 64, 128, 256) / how many blocks share a tile's K-steps (0 = choose). */
void tlc_linear_tile_override(int bn);
void tlc_linear_split_override(int n);
/* Test hook: pairs of blocks on 256 x 256 tiles (tcgen05.mma.cta_group::2): 0 = where they pay, 1 = never,
 * 2 = wherever the GPU can run them. */
void tlc_linear_pair_override(int mode);
/* How many pairs of blocks the GPU runs at once; 0 if it runs none (every product then takes single blocks). */
int tlc_linear_pairs(void);

/* ---- attention (attention.cu, attention_decode_fused.cu, attention_prefill.cu) ------------------- */
/* Rotates q and k (split-half pairs over the first rope_dim dims, angle = position * inv_freq[i]); writes
 * q to q_out [T, H*hd] and, when write_kv, k and v into the pages of their sequences. */
int tlc_rope_kv_store(const void* qkv, int in_dtype, int dtype, int ld, int q_off, int k_off, int v_off,
                      void* q_out, void* k_pages, void* v_pages, const float* inv_freq, int rope_dim,
                      const int* positions, const int* row_seq, const int* slots, const int* block_table,
                      int max_pages, int T, int H, int KV, int hd, int write_kv, cudaStream_t stream);
/* Causal grouped-query attention of every row over its sequence's pages (keys 0..position, or the last
 * `window`); any sizes, both element types; a warp per (row, head). */
int tlc_attention(const void* q, int dtype, const void* k_pages, const void* v_pages, const int* block_table,
                  int max_pages, const int* positions, const int* row_seq, const int* slots, void* out, int T,
                  int H, int KV, int hd, float scale, int window, int out_ld, cudaStream_t stream);
/* Single-token rows: keys split across blocks of 128, partial results in part_o [T, H, splits, hd] and
 * part_ml [T, H, splits, 2], then merged. */
int tlc_attention_decode(const void* q, int dtype, const void* k_pages, const void* v_pages,
                         const int* block_table, int max_pages, const int* positions, const int* row_seq,
                         const int* slots, void* out, float* part_o, float* part_ml, int T, int H, int KV,
                         int hd, float scale, int window, int max_keys, int out_ld, cudaStream_t stream);
/* Single-token rows of a bfloat16 cache in one kernel: rotation of q and the new key, store of the new
 * K/V row, scores and outputs on the tensor cores, merge of the splits by the last block to arrive
 * (arrivals: zeroed counters, at least T*KV, back at zero afterwards). */
int tlc_attention_decode_fused_ok(int H, int KV, int hd);
int tlc_attention_decode_fused_passes(int passes);
int tlc_attention_decode_fused(const float* qkv, int ld, int q_off, int k_off, int v_off, void* k_pages,
                               void* v_pages, const float* inv_freq, int rope_dim, int write_kv,
                               const int* block_table, int max_pages, const int* positions, const int* row_seq,
                               const int* slots, void* out, float* part_o, float* part_ml, unsigned* arrivals,
                               int T, int H, int KV, int hd, float scale, int window, int max_keys, int out_ld,
                               cudaStream_t stream);
/* Prompt rows (consecutive positions from start_pos) of a bfloat16 cache on the tensor cores. */
int tlc_attention_prefill_ok(int dtype, int hd);
int tlc_attention_prefill_chunks(int n_tiles_bound, int H, int max_tiles, int* chunk_tiles /* host */);
int tlc_attention_prefill(const void* q, const void* k_pages, const void* v_pages, const int* block_table,
                          int max_pages, const int* cu_seqlens, const int* slots, const int* start_pos, void* out,
                          int n_seqs, int n_tiles_bound, int H, int KV, int hd, float scale, int window,
                          int max_tiles, const int* row_seq, float* part_o, float* part_ml, int T, int out_ld,
                          cudaStream_t stream);

/* The same on tcgen05.mma (attention_prefill_tc.cu): 128-row tiles, Q and the K and V pages by TMA, scores and
 * output in tensor memory.  n_tiles_bound >= sum_b ceil(n_new_b / 128); n_pages: pages of k_pages / v_pages.
 * Values in pages past a sequence's end must be finite. */
int tlc_attention_prefill_tc_ok(int dtype, int hd, int H, int KV);
int tlc_attention_prefill_tc(const void* q, const void* k_pages, const void* v_pages, int n_pages,
                             const int* block_table, int max_pages, const int* cu_seqlens, const int* slots,
                             const int* start_pos, void* out, int n_seqs, int n_tiles_bound, int H, int KV,
                             int hd, float scale, int window, int max_keys, int T, int out_ld, int max_blocks,
                             int n_split, float* part_o, float* part_ml, cudaStream_t stream);
int tlc_attention_prefill_tc_splits(int n_tiles_bound, int H, int max_keys);   // suggested n_split (1: none)

/* ---- Mamba2 (mamba.cu, mamba_ssd.cu) ----------------------------------------------------------------- */
/* Causal depthwise convolution + SiLU over the x|B|C columns of proj, continuing each sequence's window
 * conv_state [n_slots, K-1, Cd] (updated in place); dt = softplus(dt + dt_bias), dA = exp(dt * A).
 * xbc_out [T, Cd] has the type xbc_dtype: float for single-token steps and the 32-bit scans, bfloat16
 * for the scan of prompts in matrix form (tlc_ssm_scan_ssd). */
int tlc_mamba_conv(const void* proj, int dtype, int ld, int xbc_off, int dt_off, const float* w,
                   const float* bias, const float* dt_bias, const float* A, float* conv_state,
                   const int* cu_seqlens, const int* row_seq, const int* slots, const int* start_pos,
                   void* xbc_out, int xbc_dtype, float* dt_out, float* dA_out, int T, int B, int Cd, int K,
                   int Hs, int single_rows, int quick, int all_fresh, cudaStream_t stream);
/* S = S * dA + B (x dt), y = S.C + x D, row by row from each slot's state [n_slots, Hs, P, N] (zero at
 * position 0), which is updated in place. */
int tlc_ssm_scan(const float* xbc, const float* dt, const float* dA, const float* Dskip, float* state,
                 const int* cu_seqlens, const int* slots, const int* start_pos, float* y, int B, int Hs, int P,
                 int N, int G, int Cd, cudaStream_t stream);
/* The same with sequences cut into chunks (seg_start [n_seg+1], seg_seq [n_seg], seq_seg_start [B+1]) that
 * run in parallel in three 32-bit passes; chunk_state: n_seg*Hs*(P*N+1) floats of scratch. */
int tlc_ssm_scan_chunked(const float* xbc, const float* dt, const float* dA, const float* Dskip, float* state,
                         float* chunk_state, const int* seg_start, const int* seg_seq, const int* seq_seg_start,
                         const int* slots, const int* start_pos, float* y, int B, int n_seg, int Hs, int P, int N,
                         int G, int Cd, cudaStream_t stream);
/* The chunks (of 128 rows at most) in matrix form on the tensor cores, for bfloat16 runs: xbc is bfloat16
 * [T, Cd]; C B^T of every chunk goes through `scratch` (tlc_ssd_scratch_floats floats); one block per
 * (sequence, head, 32 rows of the head) then walks the sequence's chunks in order with the state in its
 * registers, from the slot's state to the slot's state. */
int tlc_ssd_ok(int Hs, int P, int N, int G, int Cd);
/* Test hook: 0 = the walk uses tcgen05.mma with the state in tensor memory where it is built (states of 128
 * or 256 columns) and mma.sync with the state in registers elsewhere; 1 = always the latter. */
void tlc_ssd_walk_override(int mode);
void tlc_ssd_walk_blocks(int blocks);      // the grid of the tcgen05 walk (0: one block an SM at most; for tests)
long long tlc_ssd_scratch_floats(int n_seg, int T, int Hs, int P, int N, int G);
/* y_part [T, Hs*P] and used_part may be NULL.  Where the walk runs on tcgen05 and they are given, the outputs come as
 * two summands: what needs no state (M x + D x) in y_part, the state's share in y, and *used_part = 1.  With a second
 * stream `aux` (NULL: none) the first summand is computed there, beside the walk; `stream` has waited for it when the
 * call returns.  Otherwise *used_part = 0 and y holds the outputs. */
int tlc_ssm_scan_ssd(const void* xbc, const float* dt, const float* A, const float* Dskip, float* state,
                     float* scratch, const int* seg_start, const int* seg_seq, const int* seq_seg_start,
                     const int* slots, const int* start_pos, float* y, float* y_part, int* used_part, int B, int n_seg,
                     int T, int Hs, int P, int N, int G, int Cd, cudaStream_t stream, cudaStream_t aux);

/* ---- sampling (sampling.cu) ------------------------------------------------------------------------ */
/* out[r] = first index of the maximum of logits[r].  work: NULL (one block a row), or 12 * R bytes, 8-byte
 * aligned and zero (R 64-bit keys, R counters), which every launch leaves zero: a row is then spread over
 * blocks of 2,048 values.  Launches that share `work` must not overlap on the GPU. */
int tlc_argmax(const float* logits, int R, int V, int* out, void* work, cudaStream_t stream);
/* Penalties over history [R, n_history] (-1 = empty), temperature, top-k, min-p, top-p, then one draw per
 * row from uniforms [R]; work: R*V floats of scratch. */
int tlc_sample(const float* logits, float* work, const int* history, const float* uniforms, int R, int V,
               float temperature, int top_k, float top_p, float min_p, float repeat_penalty, int n_history,
               float frequency_penalty, float presence_penalty, int* out, cudaStream_t stream);

#ifdef __cplusplus
}
#endif

/* The entry point for callers that must not allocate has a header of its own. */
#include "no_alloc.h"

#endif /* TINYLLAMA_C_B200_H */
