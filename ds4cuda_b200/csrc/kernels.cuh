// kernels.cuh — internal launch functions of libds4b200.  Each one picks the
// 128-bit path when pointers and sizes allow it and a scalar-load path of the
// same kernel family otherwise, then enqueues on `stream`.  No argument checks
// here: the checked C ABI (capi.cu) and the drop-in launchers (launchers.cu)
// sit on top.
#pragma once

#include <cstdint>
#include <cuda_runtime.h>

#include "../../include/ds4b200.h"

namespace ds4b200 {

// Records the message ds4b200_last_error() returns on this thread; returns code.
int set_error(int code, const char *fmt, ...);

void add_f32(const float *a, const float *b, float *y, int64_t n, cudaStream_t s);

void rms_norm_rows(const float *x, const float *residual_in, const float *w, int64_t weight_dim,
                   float *y_f32, uint16_t *y_bf16, float *residual_out, int64_t n_rows, int n,
                   float eps, cudaStream_t s, int8_t *xq = nullptr, float *xscale = nullptr,
                   int8_t *kq = nullptr, float *kscale = nullptr, int16_t *kbsums = nullptr);

// Activation quantisers (cuda/dense_q8.cu:122-152, cuda/moe_iq2_pair.cu:159-235).
void quantize_q8_0_rows(const float *x, int8_t *xq, float *xscale, int64_t n_blocks, cudaStream_t s);
void quantize_q8_K_rows(const float *x, int8_t *xq, float *xscale, int16_t *xbsums, int64_t n_blocks,
                        cudaStream_t s);

void embed_gather_rows(const void *table, int table_dtype, const int32_t *ids, int single_id,
                       int64_t n_tokens, int n_embd, const float *residual_in,
                       const float *norm_w, float eps, float *out_rows, int n_replicas,
                       float *normed_f32, uint16_t *normed_bf16, cudaStream_t s);
int read_and_clear_device_status();   // embedding.cu owns the status word
int *device_status_word();            // its device address on the current device, or null
void selftest_bounded_wait(int max_polls, int *gave_up_dev, cudaStream_t s);

// pos == nullptr: every token uses single_pos.
// xq != nullptr: the rotated rows also leave as Q8_0 blocks (xq int8, xscale one per 32); x_out may then
// be null.  That form needs head_dim % 32 == 0, n_rot % 4 == 0 and 16-byte aligned rows.
void rope_rows(const float *x_in, float *x_out, int64_t n_tokens, int n_heads, int head_dim,
               int n_rot, const int32_t *pos, int single_pos, const ds4b200_rope_params &p,
               int inverse, int unit_rms, float eps, cudaStream_t s, int8_t *xq = nullptr,
               float *xscale = nullptr, const float *cs_table = nullptr);

// cs_table[t][n_rot/2][2]: the (cos, sin) multipliers of every tail pair at pos[t] (n_rot <= 64), the same bits the
// RoPE kernels evaluate per head row; those kernels take it in place of pos + params.
void rope_table_rows(const int32_t *pos, int64_t n_tokens, int n_rot, const ds4b200_rope_params &p, float *cs_table,
                     cudaStream_t s);

void fp8_kv_round_trip_rows(const float *kv_in, float *kv_out, int64_t n_rows, int head_dim,
                            int n_rot, cudaStream_t s);

void rope_fp8_store_rows(const float *kv_in, int64_t n_rows, int head_dim, int n_rot,
                         const int32_t *pos, const ds4b200_rope_params *p, const float *norm_w,
                         float eps, int scale_mode, const int32_t *slots, uint8_t *codes,
                         float *scales, float *tail_out, float *rope_out, cudaStream_t s,
                         float *raw_out = nullptr, const float *cs_table = nullptr, float *cs_out = nullptr);
// cs_out (n_rot <= 64, one KV row per token, no cs_table): the (cos, sin) pairs this launch evaluates for its rows are
// also written to cs_out[r][n_rot/2][2], which is then the chunk's angle table for the RoPE launches that follow.

// Read side of the FP8 byte cache: rows at slots[] -> f32 (optionally f16-rounded).
void fp8_cache_load_rows(const uint8_t *codes, const float *scales, const float *tail, const int32_t *slots,
                         int64_t n_rows, int head_dim, int n_rot, int scale_mode, int f16_out, float *out,
                         cudaStream_t s);

// raw_kv window [cap][head_dim]: push n_new rows (f16-rounded), dropping the oldest.
void swa_window_push_rows(float *raw_kv, int cap, int n_raw, const float *new_rows, int n_new, int head_dim,
                          cudaStream_t s);

void swiglu_rows(const float *gate, const float *up, const float *weights, float *out,
                 int64_t n_tokens, int k, int n, int mode, float clamp, int combine,
                 int fast_exp, cudaStream_t s);

void hc_pre_rows(const float *residual_hc, const uint16_t *hc_fn, const float *hc_scale,
                 const float *hc_base, float *post, float *comb, float *out, int64_t n_tokens,
                 int n_embd, int iters, float eps, cudaStream_t s);

// Cluster variant of the pre step without the Sinkhorn sweeps (comb receives the 16
// pre-softmax values); false = shape not covered, nothing launched.
bool hc_pre_rows_cluster(const float *residual_hc, const uint16_t *hc_fn, const float *hc_scale,
                         const float *hc_base, float *post, float *comb, float *out, int64_t n_tokens,
                         int n_embd, float eps, cudaStream_t s);
bool hc_pre_rows_mma(const float *residual_hc, const uint16_t *hc_fn, const float *hc_scale,
                         const float *hc_base, float *post, float *comb, float *out, int64_t n_tokens,
                         int n_embd, float eps, cudaStream_t s);

// tcgen05 variant (n_embd 4096, clusters of 16 CTAs)
bool hc_pre_rows_tc(const float *residual_hc, const uint16_t *hc_fn, const float *hc_scale, const float *hc_base,
                    float *post, float *comb, float *out, int64_t n_tokens, int n_embd, int iters, float eps, cudaStream_t s);

// hc_pre_rows, then RMSNorm(out) * norm_w -> normed (optional) and its Q8_0 blocks xq / xscale (optional).
void hc_pre_norm_rows(const float *residual_hc, const uint16_t *hc_fn, const float *hc_scale, const float *hc_base,
                      const float *norm_w, float *post, float *comb, float *out, float *normed, int8_t *xq,
                      float *xscale, int64_t n_tokens, int n_embd, int iters, float eps, cudaStream_t s);

// Output HC head, optionally followed by the output RMSNorm (norm_w != nullptr -> normed).
void hc_head_rows(const float *residual_hc, const uint16_t *fn, const float *scale1, const float *base4,
                  const float *norm_w, float *out, float *normed, int64_t n_tokens, int n_embd, float eps,
                  cudaStream_t s);

// comb_out[t][16] = Sinkhorn(logits[t][16]), one thread per token.
void hc_sinkhorn_rows(const float *logits, float *comb_out, int64_t n_tokens, int iters, float eps,
                      cudaStream_t s);

// logits != nullptr: comb is produced by Sinkhorn from logits (and stored to
// comb_out when given); otherwise comb/post are read.
void hc_post_rows(const float *block_out, const float *block_out2, const float *residual_hc,
                  const float *post, const float *comb, const float *logits, float *comb_out,
                  float *out_hc, int64_t n_tokens, int n_embd, int iters, float eps,
                  cudaStream_t s);

// compressor.cu: returns whether the step emitted
bool compressor_step(int is_attn, const float *kv_cur, float *sc_cur, const uint16_t *ape_f16,
                     const float *norm_w, int head_dim, int ratio, int pos, const ds4b200_rope_params &rope,
                     int n_rot, float eps, float *state_kv, float *state_score, float *emit_out,
                     cudaStream_t s);
// the same for a chunk of tokens that starts and ends on window boundaries (emit_out [n_tokens/ratio][head_dim])
void compressor_chunk(int is_attn, const float *kv_cur, const float *sc_cur, const uint16_t *ape_f16,
                      const float *norm_w, int head_dim, int ratio, int pos0, int64_t n_tokens,
                      const ds4b200_rope_params &rope, int n_rot, float eps, float *state_kv, float *state_score,
                      float *emit_out, cudaStream_t s);
void swiglu_q8_K_rows(const float *gate, const float *up, const float *weights, int8_t *xq, float *xscale,
                      int16_t *xbsums, float *mid_f32, int64_t n_rows, int n, int mode, float clamp,
                      int fast_exp, cudaStream_t s);
void swiglu_q8_0_rows(const float *gate, const float *up, const float *weights, int8_t *xq, float *xscale,
                      float *mid_f32, int64_t n_rows, int n, int mode, float clamp, int fast_exp, cudaStream_t s);
void div_selfcheck(uint64_t first, uint64_t count, unsigned long long *mismatches, cudaStream_t s);
void e4m3_encode(const float *x, uint8_t *codes, int64_t n, cudaStream_t s);
void e4m3_decode(const uint8_t *codes, float *x, int64_t n, cudaStream_t s);
void e4m3_selfcheck(uint32_t first_bits, uint64_t count, unsigned long long *mismatches,
                    cudaStream_t s);

}  // namespace ds4b200
