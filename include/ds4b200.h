/* ds4b200.h — C ABI of libds4b200.so: the fused elementwise / row-reduction
 * path of the ds4cuda forward pass, written for NVIDIA B200 (sm_100a).
 *
 * Two families of entry points:
 *
 *  1. `ds4b200_launch_*`  — `extern "C"` names for the reference's C++
 *     launchers (`namespace ds4cuda`, declared in ds4b200_launchers.cuh with
 *     the reference's own signatures).  One token per call, `void`, no checks,
 *     no allocation, no synchronisation: exactly the reference's convention.
 *
 *  2. `ds4b200_*_rows*`   — batched siblings for T-token prefill, explicit
 *     parameters instead of per-layer routing.  They check their arguments and
 *     return 0, or a negative errno (-EINVAL bad argument, -EIO launch error);
 *     ds4b200_last_error() gives the message.  They never allocate or
 *     synchronise either.
 *
 * Every pointer is device memory owned by the caller unless its name starts
 * with `host_`.  `stream` is a `cudaStream_t` passed as `void *` (NULL = the
 * default stream).  The library has no CPU fallback: without a CUDA device the
 * launches fail and the checked entry points return -EIO.
 */
#ifndef DS4B200_H
#define DS4B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- enums and parameter blocks ------------------------------------------ */

enum { DS4B200_TABLE_F16 = 0, DS4B200_TABLE_Q8_0 = 1 };

/* FP8 scale layout.  BLOCK64_POW2 is the reference's rule (cuda/fp8_kv.cu:161-180):
 * one power-of-two scale per 64 elements of the non-rotated prefix, the rotated
 * tail kept in f32.  ROW_AMAX is one scale = max(amax,1e-4)/448 per row over all
 * head_dim elements. */
enum { DS4B200_FP8_BLOCK64_POW2 = 0, DS4B200_FP8_ROW_AMAX = 1 };

/* SwiGLU flavour.  PLAIN: (g*sigmoid(g))*u (cuda/glu.cu:56-75).  CLAMP_REF:
 * gate clamped from above, up clamped both sides (cuda/moe_iq2_pair.cu:352-373).
 * CLAMP_SYM: both clamped both sides. */
enum { DS4B200_GLU_PLAIN = 0, DS4B200_GLU_CLAMP_REF = 1, DS4B200_GLU_CLAMP_SYM = 2 };

/* RoPE parameters after the per-layer routing of cuda/rope.cu:214-250.
 * theta_scale <= 0 asks the kernel to evaluate powf(freq_base, -2/n_rot) on the
 * device, as the reference kernel does (cuda/rope.cu:173). */
typedef struct ds4b200_rope_params {
    float freq_base;
    float theta_scale;
    float freq_scale;
    float ext_factor;
    float attn_factor;
    float corr_low;
    float corr_high;
} ds4b200_rope_params;

/* ---- library state ----------------------------------------------------------- */

const char *ds4b200_version(void);
/* Message of the last failing checked call on this thread ("" if none). */
const char *ds4b200_last_error(void);
/* Bit mask of faults kernels recorded on the current device since the last
 * call (bit 0: a bulk copy into shared memory did not complete in time);
 * reading clears it.  Synchronises the device.  Negative errno on failure. */
int ds4b200_device_status(void);

/* Self-test of the bounded device-side wait: a one-warp kernel waits on a barrier that
 * nothing signals, gives up after max_polls (<= 65536) polls, writes 1 to *gave_up (device
 * int) and ends normally; ds4b200_device_status() then reports bit 0.  Never hangs. */
int ds4b200_selftest_bounded_wait(int max_polls, int *gave_up, void *stream);

/* Host-side routing helpers (no device work).
 * for_layer: the reference's rule, cuda/rope.cu:214-250 (theta_scale left 0). */
void ds4b200_rope_params_for_layer(int il, int n_rot, ds4b200_rope_params *out);
void ds4b200_rope_params_explicit(float freq_base, float yarn_factor, int n_ctx_orig,
                                  int n_rot, ds4b200_rope_params *out);

/* ---- 1. drop-in launchers, C names ---------------------------------------------- */

/* cuda/norm.cuh:24 */
void ds4b200_launch_rms_norm_f32(const float *x, const float *w, float *y, int n,
                                 float eps, void *stream);
/* cuda/norm.cuh:42 */
void ds4b200_launch_rms_norm_batch_f32(const float *x, const float *w, int weight_dim,
                                       float *y, int n_rows, int n_per_row, float eps,
                                       void *stream);
/* cuda/elementwise.cuh:27 */
void ds4b200_launch_add_f32(const float *a, const float *b, float *y, int n, void *stream);
/* cuda/rope.cuh:51 */
void ds4b200_launch_tail_rope_yarn_f32(const float *x_in, float *x_out, int n_heads,
                                       int head_dim, int n_rot, int pos, int il, void *stream);
/* cuda/attn_out.cuh:52 */
void ds4b200_launch_tail_rope_yarn_inverse_f32(const float *x_in, float *x_out, int n_heads,
                                               int head_dim, int n_rot, int pos, int il,
                                               void *stream);
/* cuda/fp8_kv.cuh:62 */
void ds4b200_launch_fp8_kv_quantize_round_trip_f32(const float *kv_in, float *kv_out,
                                                   int n_rows, int head_dim, int n_rot,
                                                   void *stream);
/* cuda/glu.cuh:30 */
void ds4b200_launch_silu_mul_f32(const float *g, const float *u, float *y, int n, void *stream);
/* cuda/embedding.cuh:46 */
void ds4b200_launch_embed_token_f16_to_f32(const uint16_t *token_embd_weight, int token_id,
                                           int n_embd, float *out, void *stream);
/* cuda/hc_sinkhorn.cuh:55 */
void ds4b200_launch_hc_attn_pre_f32(const float *residual_hc, const uint16_t *hc_fn,
                                    const float *hc_scale, const float *hc_base,
                                    float *post_weights, float *comb, float *out,
                                    int n_embd, int n_hc, int sinkhorn_iters, float eps,
                                    void *stream);
/* cuda/hc_sinkhorn.cuh:80 and :99 (the ffn variant forwards to the same chain) */
void ds4b200_launch_hc_attn_pre_v2_f32(const float *residual_hc, const uint16_t *hc_fn,
                                       const float *hc_scale, const float *hc_base,
                                       float *post_weights, float *comb, float *out,
                                       int n_embd, int n_hc, int sinkhorn_iters, float eps,
                                       float *rms_scratch, float *mix_scratch, void *stream);
/* cuda/hc_sinkhorn.cuh:138 */
void ds4b200_launch_hc_post_f32(const float *block_out, const float *residual_hc,
                                const float *post, const float *comb, float *out_hc,
                                int n_hc, int n_embd, void *stream);

/* cuda/output_head.cuh:68 */
void ds4b200_launch_output_hc_head_f32(const float *residual_hc, const uint16_t *output_hc_fn,
                                       const float *output_hc_scale, const float *output_hc_base,
                                       float *out, int n_embd, int n_hc, float eps, void *stream);

/* ---- 2. batched, checked siblings ---------------------------------------------- */

/* y = a + b over n elements (cuda/elementwise.cu:36-43, any n). */
int ds4b200_add_f32(const float *a, const float *b, float *y, int64_t n, void *stream);

/* RMSNorm of n_rows rows of n elements (cuda/norm.cu:126-197) with the chain
 * around it fused: residual_in (nullable) is added first, the sum goes to
 * residual_out (nullable), the normalised row to y_f32 and/or y_bf16 (either
 * nullable, RNE).  weight_dim: 0 unit gain, n shared gain, n*n_rows per-row. */
int ds4b200_rms_norm_rows_f32(const float *x, const float *residual_in, const float *w,
                              int64_t weight_dim, float *y_f32, uint16_t *y_bf16,
                              float *residual_out, int64_t n_rows, int n, float eps,
                              void *stream);

/* The same RMSNorm with the activation quantiser of the Q8_0 matvec that consumes the row
 * fused behind it (cuda/dense_q8.cu:122-152: per 32 elements d = amax/127 as f32,
 * q = clamp(rint(y/d))): xq[n_rows][n] int8, xscale[n_rows][n/32].  y_f32 nullable.
 * n a multiple of 32, at most 8192; 16-byte aligned f32 buffers. */
int ds4b200_rms_norm_q8_0_rows_f32(const float *x, const float *residual_in, const float *w,
                                   int64_t weight_dim, float *y_f32, float *residual_out,
                                   int8_t *xq, float *xscale, int64_t n_rows, int n, float eps,
                                   void *stream);

/* The same RMSNorm leaving the row as the Q8_K blocks the routed experts' IQ2_XXS gate / up dots
 * read, which the reference quantises inside that launcher (cuda/moe_iq2_pair.cu:159-235 called on
 * the normalised row at :404-421): kq[n_rows][n] int8, kscale[n_rows][n/256],
 * kbsums[n_rows][n/256][16].  xq / xscale (the Q8_0 form, both or neither) and y_f32 are nullable:
 * the feed-forward norm of a layer feeds a Q8_0 matvec (shared expert) and the Q8_K dots (routed
 * experts) from the same row.  n a multiple of 256, at most 8192; 16-byte aligned f32 buffers. */
int ds4b200_rms_norm_q8_K_rows_f32(const float *x, const float *residual_in, const float *w,
                                   int64_t weight_dim, float *y_f32, float *residual_out,
                                   int8_t *xq, float *xscale, int8_t *kq, float *kscale,
                                   int16_t *kbsums, int64_t n_rows, int n, float eps, void *stream);

/* The activation quantisers on their own.  Q8_0 split form: n_blocks blocks of 32 f32 ->
 * int8 + one f32 scale each (cuda/dense_q8.cu:122-152).  Q8_K: n_blocks blocks of 256 ->
 * int8, one f32 scale and 16 int16 partial sums each (cuda/moe_iq2_pair.cu:159-235; on equal
 * magnitudes the first element decides the sign of the scale). */
int ds4b200_quantize_q8_0_rows_f32(const float *x, int8_t *xq, float *xscale, int64_t n_blocks,
                                   void *stream);
int ds4b200_quantize_q8_K_rows_f32(const float *x, int8_t *xq, float *xscale, int16_t *xbsums,
                                   int64_t n_blocks, void *stream);

/* Embedding gather for n_tokens ids (cuda/embedding.cu:27-39 for F16 rows,
 * cuda/dense_q8.cu:60-67 for Q8_0 rows of 34-byte blocks), fused with what
 * follows it: + residual_in (nullable), n_replicas copies of the f32 row to
 * out_rows[t][rep][n_embd] (nullable; cuda/forward_token.cu:350-354 makes 4),
 * and, when norm_w is given, RMSNorm to normed_f32 / normed_bf16 (nullable).
 * ids outside [0, vocab) are the caller's error, as in the reference. */
int ds4b200_embed_gather_rows(const void *table, int table_dtype, const int32_t *ids,
                              int64_t n_tokens, int n_embd, const float *residual_in,
                              const float *norm_w, float eps, float *out_rows, int n_replicas,
                              float *normed_f32, uint16_t *normed_bf16, void *stream);

/* Tail RoPE over [n_tokens][n_heads][head_dim] with one position per token
 * (cuda/rope.cu:136-201; inverse: cuda/attn_out.cu:54-107).  unit_rms != 0
 * first applies the unit-gain per-head RMSNorm of cuda/forward_layer.cu:890.
 * In place (x_out == x_in) is allowed. */
int ds4b200_rope_rows_f32(const float *x_in, float *x_out, int64_t n_tokens, int n_heads,
                          int head_dim, int n_rot, const int32_t *pos,
                          const ds4b200_rope_params *params, int inverse, int unit_rms,
                          float eps, void *stream);

/* The (cos, sin) multipliers of the n_rot/2 tail pairs of every token, cs_table[t][n_rot/2][2] floats
 * (n_rot <= 64).  They depend on pos[t] and the parameter set only, yet the reference evaluates them
 * for every head row (cuda/rope.cu:165-200): per layer 64 query rows, 64 attention-output rows and
 * the KV row of each token share them.  Computed here once per chunk by the same device code, so a
 * RoPE entry point given the table produces the same bits as one given pos + params. */
int ds4b200_rope_table_rows(const int32_t *pos, const ds4b200_rope_params *params, int64_t n_tokens,
                            int n_rot, float *cs_table, void *stream);
/* ds4b200_rope_rows_f32 with the table in place of pos + params. */
int ds4b200_rope_rows_table_f32(const float *x_in, float *x_out, int64_t n_tokens, int n_heads,
                                int head_dim, int n_rot, const float *cs_table, int inverse,
                                int unit_rms, float eps, void *stream);

/* The same rotation with the rows leaving as Q8_0 activation blocks, the form the grouped
 * out-projection quantises its input to right behind the inverse RoPE (cuda/forward_layer.cu:1179
 * then cuda/attn_out.cu:119-145): xq int8 [n_tokens][n_heads][head_dim], xscale
 * [n_tokens][n_heads][head_dim/32] (d = amax/127 per 32 values, round to nearest even, clamp to
 * [-128, 127]).  x_out is optional: NULL drops the f32 copy, which is then never written to memory.
 * cs_table is optional (ds4b200_rope_table_rows); with it pos and params may be NULL.
 * head_dim a multiple of 32 (<= 1024), n_rot a multiple of 4, 16-byte aligned f32 rows. */
int ds4b200_rope_q8_0_rows_f32(const float *x_in, float *x_out, int8_t *xq, float *xscale,
                               int64_t n_tokens, int n_heads, int head_dim, int n_rot,
                               const int32_t *pos, const ds4b200_rope_params *params,
                               const float *cs_table, int inverse, int unit_rms, float eps,
                               void *stream);

/* FP8 E4M3FN quantise/dequantise round trip, cuda/fp8_kv.cu:144-195. */
int ds4b200_fp8_kv_round_trip_rows_f32(const float *kv_in, float *kv_out, int64_t n_rows,
                                       int head_dim, int n_rot, void *stream);

/* Fused KV row chain: optional weighted RMSNorm (norm_w nullable) -> tail RoPE
 * at pos[r] (params nullable = rows are already rotated) -> E4M3FN bytes and
 * scales into a cache.  Row r lands in slot slots[r] (slots nullable = r);
 * codes[slot][head_dim], scales[slot][n_scales] with n_scales =
 * (head_dim-n_rot)/64 (BLOCK64_POW2) or 1 (ROW_AMAX).  BLOCK64_POW2 writes the
 * rotated tail as f32 to tail_out[slot][n_rot] (nullable) and zero codes for
 * it.  rope_out[r][head_dim] (nullable) receives the f32 row before encoding. */
int ds4b200_rope_fp8_store_rows(const float *kv_in, int64_t n_rows, int head_dim, int n_rot,
                                const int32_t *pos, const ds4b200_rope_params *params,
                                const float *norm_w, float eps, int scale_mode,
                                const int32_t *slots, uint8_t *codes, float *scales,
                                float *tail_out, float *rope_out, void *stream);

/* Read side of the byte cache written by ds4b200_rope_fp8_store_rows: out[r][head_dim] =
 * the row at slot slots[r] (slots nullable = r) as f32.  With BLOCK64_POW2 the result is
 * bit for bit what the reference's f32 round trip leaves in its cache (code value x
 * power-of-two scale, f32 tail; cuda/fp8_kv.cu:161-195) — except that an input of exactly
 * -0.0 reads back as -0.0 where the reference gives +0.0.  f16_round != 0 adds the f16
 * rounding of the raw KV cache (cuda/forward_layer.cu:182-190). */
int ds4b200_fp8_cache_load_rows(const uint8_t *codes, const float *scales, const float *tail,
                                const int32_t *slots, int64_t n_rows, int head_dim, int n_rot,
                                int scale_mode, int f16_round, float *out, void *stream);

/* The whole KV row chain of the reference in one launch (cuda/forward_layer.cu:868, :910,
 * :921, :950): optional weighted RMSNorm -> tail RoPE at pos[r] -> E4M3FN round trip of the
 * non-rotated prefix with per-64 power-of-two scales -> f16 rounding -> raw_out[slot][head_dim]
 * in f32, the form rows have in the reference's raw KV cache.  slots nullable (= r). */
int ds4b200_kv_rows_to_raw_f32(const float *kv_in, int64_t n_rows, int head_dim, int n_rot,
                               const int32_t *pos, const ds4b200_rope_params *params,
                               const float *norm_w, float eps, const int32_t *slots,
                               float *raw_out, void *stream);

/* ds4b200_rope_fp8_store_rows and ds4b200_kv_rows_to_raw_f32 with the chunk's angle table
 * (ds4b200_rope_table_rows; one row of n_rot/2 (cos, sin) pairs per input row, n_rot <= 64) in place of
 * pos + params: the same bits, without 32 cos / sin evaluations per row. */
int ds4b200_rope_fp8_store_rows_table(const float *kv_in, int64_t n_rows, int head_dim, int n_rot,
                                      const float *cs_table, const float *norm_w, float eps, int scale_mode,
                                      const int32_t *slots, uint8_t *codes, float *scales, float *tail_out,
                                      float *rope_out, void *stream);
int ds4b200_kv_rows_to_raw_table_f32(const float *kv_in, int64_t n_rows, int head_dim, int n_rot,
                                     const float *cs_table, const float *norm_w, float eps, const int32_t *slots,
                                     float *raw_out, void *stream);

/* ds4b200_kv_rows_to_raw_f32 that also leaves the chunk's angle table: with one KV row per token the 32
 * (cos, sin) pairs this launch evaluates per row ARE the table's entries, so cs_out[r][n_rot/2][2] receives them
 * (the bits ds4b200_rope_table_rows writes) and the head-row RoPE launches that follow take it as cs_table. */
int ds4b200_kv_rows_to_raw_table_out_f32(const float *kv_in, int64_t n_rows, int head_dim, int n_rot,
                                         const int32_t *pos, const ds4b200_rope_params *params, const float *norm_w,
                                         float eps, const int32_t *slots, float *raw_out, float *cs_out, void *stream);

/* Sliding raw-KV window [cap][head_dim] holding n_raw rows: push n_new rows at once
 * (f16-rounded on entry).  Equivalent to n_new single-row pushes of the reference
 * (append while there is room, else shift every row down by one and write last,
 * cuda/forward_layer.cu:159-190, :941-972).  *n_raw_after (host, nullable) receives
 * min(cap, n_raw + n_new).  In place. */
int ds4b200_swa_window_push_rows_f32(float *raw_kv, int cap, int n_raw, const float *new_rows,
                                     int n_new, int head_dim, int *n_raw_after, void *stream);

/* SwiGLU whose output leaves as Q8_K blocks: mid[t][s][:] = glu(gate, up) * weights[t][s] (no
 * sum over slots: the down projection is per expert), quantised per 256 elements exactly as
 * ds4b200_quantize_q8_K_rows_f32 would quantise the f32 rows (cuda/moe_iq2_pair.cu:159-235,
 * :352-373).  gate, up [n_tokens][k][n]; weights [n_tokens][k] nullable; xq int8 [n_tokens*k*n];
 * xscale f32 and xbsums int16[16] per block; mid_f32 nullable (also writes the f32 rows).
 * n a multiple of 256; pointers 16-byte aligned. */
int ds4b200_swiglu_q8_K_rows_f32(const float *gate, const float *up, const float *weights, int8_t *xq,
                                 float *xscale, int16_t *xbsums, float *mid_f32, int64_t n_tokens, int k,
                                 int n, int mode, float clamp, int fast_exp, void *stream);

/* SwiGLU whose output leaves as Q8_0 blocks, the form the shared expert's down projection
 * quantises its activations to (launch_silu_mul_f32 at cuda/forward_layer.cu:1296, then the
 * quantiser inside the Q8_0 matvec, cuda/dense_q8.cu:122-152): per 32 elements d = amax/127,
 * q = clamp(rint(v/d)), exactly as ds4b200_quantize_q8_0_rows_f32 would quantise the f32 rows.
 * gate, up [n_tokens][k][n]; weights [n_tokens][k] nullable; xq int8 [n_tokens*k*n]; xscale
 * [n_tokens*k*n/32]; mid_f32 nullable (also writes the f32 rows).  n a multiple of 32. */
int ds4b200_swiglu_q8_0_rows_f32(const float *gate, const float *up, const float *weights, int8_t *xq,
                                 float *xscale, float *mid_f32, int64_t n_tokens, int k, int n, int mode,
                                 float clamp, int fast_exp, void *stream);

/* One streaming-compressor step after its two projections: everything
 * launch_compressor_decode_step_f32{,_prealloc} (cuda/compressor.cuh:78,102; cuda/compressor.cu:328-420)
 * does once kv_cur / sc_cur = W_kv x, W_gate x are known, in one launch.
 *   sc_cur[j] += f16(ape[pos % ratio][j]);  state row (ratio == 4 ? 4 + pos % 4 : pos % ratio) <- kv_cur, sc_cur
 * and, when (pos + 1) % ratio == 0: pool the state rows per column with softmax weights ->
 * RMSNorm (norm_w, eps 1e-6) -> tail RoPE at position pos + 1 - ratio with the parameters of
 * layer il -> E4M3FN round trip of the non-rotated prefix (is_attn != 0 only) -> emit_out[head_dim];
 * ratio 4 then copies state rows 4-7 over rows 0-3.
 * width = head_dim * (ratio == 4 ? 2 : 1).  kv_cur, sc_cur [width]; ape_f16 [ratio][width];
 * state_kv, state_score [(ratio == 4 ? 8 : ratio)][width]; n_rot 64.  *emitted_host (host,
 * nullable) receives 1 when emit_out was written.  head_dim a multiple of 64, 128..1024. */
int ds4b200_compressor_step_f32(int is_attn, const float *kv_cur, float *sc_cur, const uint16_t *ape_f16,
                                const float *norm_w, int head_dim, int compress_ratio, int pos, int il,
                                float *state_kv, float *state_score, float *emit_out,
                                int *emitted_host, void *stream);

/* The same for a chunk of n_tokens consecutive positions pos0 .. pos0 + n_tokens - 1 that starts
 * and ends on window boundaries (pos0 % ratio == 0, n_tokens % ratio == 0): equivalent to
 * n_tokens calls of ds4b200_compressor_step_f32 (bit for bit: state afterwards and the
 * n_tokens / ratio emits), in two launches.  kv_cur, sc_cur [n_tokens][width]; sc_cur is not
 * modified; emit_out [n_tokens / ratio][head_dim]. */
int ds4b200_compressor_chunk_f32(int is_attn, const float *kv_cur, const float *sc_cur, const uint16_t *ape_f16,
                                 const float *norm_w, int head_dim, int compress_ratio, int pos0,
                                 int64_t n_tokens, int il, float *state_kv, float *state_score,
                                 float *emit_out, void *stream);

/* SwiGLU over gate/up[n_tokens][k][n].  weights[n_tokens][k] nullable.
 * combine != 0: out[n_tokens][n] = sum of the k slots in slot order; else
 * out[n_tokens][k][n].  fast_exp != 0 uses the hardware exp approximation the
 * reference's expert epilogue uses (cuda/moe_iq2_pair.cu:364,367). */
int ds4b200_swiglu_rows_f32(const float *gate, const float *up, const float *weights,
                            float *out, int64_t n_tokens, int k, int n, int mode,
                            float clamp, int combine, int fast_exp, void *stream);

/* Hyper-connection pre step for n_tokens tokens (cuda/hc_sinkhorn.cu:85-305):
 * RMS over the 4*n_embd residual, 24-row f16 matvec, sigmoid / Sinkhorn split,
 * weighted sum.  post[t][4], comb[t][16], out[t][n_embd]. */
int ds4b200_hc_pre_rows_f32(const float *residual_hc, const uint16_t *hc_fn,
                            const float *hc_scale, const float *hc_base, float *post,
                            float *comb, float *out, int64_t n_tokens, int n_embd,
                            int sinkhorn_iters, float eps, void *stream);

/* The pre step and what the reference runs right behind it (cuda/forward_layer.cu:808->822 for the
 * attention half, :1235->1249 for the FFN half): normed = RMSNorm(out) * norm_w (cuda/norm.cu:52-113)
 * and its Q8_0 activation blocks (cuda/dense_q8.cu:122-152): xq int8 [t][n_embd], xscale
 * [t][n_embd/32].  normed and the xq / xscale pair are each optional (at least one is required); out,
 * post and comb are written as by ds4b200_hc_pre_rows_f32.  One call, the kernels of the two stages
 * back to back on `stream`.  The results of this call and of ds4b200_hc_pre_rows_f32 are invalid if
 * ds4b200_device_status() reports the time-out bit afterwards. */
int ds4b200_hc_pre_norm_rows_f32(const float *residual_hc, const uint16_t *hc_fn, const float *hc_scale,
                                 const float *hc_base, const float *norm_w, float *post, float *comb,
                                 float *out, float *normed, int8_t *xq, float *xscale, int64_t n_tokens,
                                 int n_embd, int sinkhorn_iters, float eps, void *stream);

/* Hyper-connection post step (cuda/hc_sinkhorn.cu:619-672) for n_tokens tokens.
 * block_out nullable (term dropped); block_out2 nullable (when given the block
 * term is block_out+block_out2, the add of cuda/forward_layer.cu:1447 fused). */
int ds4b200_hc_post_rows_f32(const float *block_out, const float *block_out2,
                             const float *residual_hc, const float *post, const float *comb,
                             float *out_hc, int64_t n_tokens, int n_embd, void *stream);

/* The post step of one sub-block followed by the pre step of the next (cuda/forward_layer.cu:1217 ->
 * :1235 inside a layer, :1456 -> :808 across layers): out_hc = post(block_out [+ block_out2],
 * residual_hc, post_in, comb_in), then (post, comb, out) = pre(out_hc, hc_fn, hc_scale, hc_base).  Same
 * bits as the two entry points called one after the other, which is what it does: two launches (post
 * and comb may be the buffers post_in and comb_in point to). */
int ds4b200_hc_post_pre_rows_f32(const float *block_out, const float *block_out2, const float *residual_hc,
                                 const float *post_in, const float *comb_in, const uint16_t *hc_fn,
                                 const float *hc_scale, const float *hc_base, float *out_hc, float *post,
                                 float *comb, float *out, int64_t n_tokens, int n_embd, int sinkhorn_iters,
                                 float eps, void *stream);

/* Output HC head for n_tokens tokens (cuda/output_head.cu:62-149): RMS over the 4*n_embd
 * block, 4-row f16 matvec, w[h] = sigmoid(pre[h]*scale[0]+base[h]) + eps, out[t] = sum_h
 * w[h]*resid[t][h].  With norm_w given, the output RMSNorm that follows it in the forward
 * pass (cuda/forward_token.cu:211) is fused: normed[t] = rmsnorm(out[t]) * norm_w.  `out`
 * may be NULL when only `normed` is wanted. */
int ds4b200_output_hc_head_rows_f32(const float *residual_hc, const uint16_t *output_hc_fn,
                                    const float *output_hc_scale, const float *output_hc_base,
                                    const float *norm_w, float *out, float *normed,
                                    int64_t n_tokens, int n_embd, float eps, void *stream);

/* The Sinkhorn step alone (cuda/hc_sinkhorn.cu:224-289): logits[t][16] (index
 * src+4*dst) -> row softmax + eps -> one column pass, then sinkhorn_iters-1
 * (row, column) passes, each dividing by (sum + eps) -> comb[t][16].  One thread
 * per token, so every token's serial chain of divisions runs side by side. */
int ds4b200_hc_sinkhorn_rows_f32(const float *logits, float *comb, int64_t n_tokens,
                                 int sinkhorn_iters, float eps, void *stream);

/* Sinkhorn mixing: comb as above, then mix the 4 residual streams,
 * out_hc[t][dst] = sum_src comb[dst+4*src]*resid[t][src].  With comb_out[t][16]
 * given this is two launches (the Sinkhorn rows, then a pure streaming mix that
 * reads comb_out); with comb_out NULL it is one kernel that runs each token's
 * sweeps on one thread of the token's CTA, which is several times slower. */
int ds4b200_hc_sinkhorn_mix_rows_f32(const float *logits, const float *residual_hc,
                                     float *out_hc, float *comb_out, int64_t n_tokens,
                                     int n_embd, int sinkhorn_iters, float eps, void *stream);

/* Sinkhorn mixing without a caller-provided buffer for the 4x4 matrices and
 * without any allocation.  This entry point has no counterpart in the reference.
 *
 * Who it is for: callers that can pass inputs and outputs but cannot come up
 * with the [n_tokens][16] intermediate that makes
 * ds4b200_hc_sinkhorn_mix_rows_f32 fast — an engine whose device memory is one
 * arena laid out at start-up, a token loop where allocator calls are banned
 * because cudaMalloc stalls the device and can fail, a binding that only ever
 * sees the pointers it is given.  The matrices live instead in a fixed array in
 * device memory inside the library: DS4B200_STATIC_MAX_TOKENS x 16 floats
 * (1 MiB), present on every GPU that loads the library until the process ends.
 *
 * Rules that follow from the shared array:
 *  - n_tokens > DS4B200_STATIC_MAX_TOKENS is refused with -EINVAL (split the
 *    batch, or use the variant above with your own comb_out);
 *  - two calls whose kernels may run at the same time on one GPU (different
 *    streams, different threads) race on the array: serialise them;
 *  - the array keeps whatever the last call wrote; every call overwrites the
 *    rows it reads before reading them, so that is harmless;
 *  - the first call on each device looks the array's address up
 *    (cudaGetSymbolAddress) and caches it; make that first call once during
 *    start-up, before any stream capture begins on that device.
 * It calls no cudaMalloc / cudaFree and no allocating library routine.
 * Results are those of ds4b200_hc_sinkhorn_mix_rows_f32 with comb_out given. */
#define DS4B200_STATIC_MAX_TOKENS 16384
int ds4b200_hc_sinkhorn_mix_rows_static_f32(const float *logits, const float *residual_hc,
                                            float *out_hc, int64_t n_tokens, int n_embd,
                                            int sinkhorn_iters, float eps, void *stream);

/* E4M3FN code of each of n f32 values (sign bit | nearest index, saturating),
 * and its inverse; used to check the encoder exhaustively. */
int ds4b200_e4m3_encode_f32(const float *x, uint8_t *codes, int64_t n, void *stream);
int ds4b200_e4m3_decode_f32(const uint8_t *codes, float *x, int64_t n, void *stream);
/* Counts the f32 bit patterns in [first_bits, first_bits+count) whose hardware
 * E4M3FN code differs from the table search of cuda/fp8_kv.cu:102-131
 * (NaN patterns skipped).  *mismatches is a device uint64 the caller zeroes. */
int ds4b200_e4m3_selfcheck(uint32_t first_bits, uint64_t count,
                           unsigned long long *mismatches, void *stream);

/* Counts, over `count` hashed (n, d) pairs with d in [1, 2], the pairs for which the
 * branch-free division the SwiGLU kernels use differs from the IEEE quotient n / d.
 * *mismatches is a device uint64 the caller zeroes. */
int ds4b200_div_selfcheck(uint64_t first, uint64_t count, unsigned long long *mismatches,
                          void *stream);

#ifdef __cplusplus
}
#endif
#endif /* DS4B200_H */
