// ref_shim.cu — `extern "C"` names for the reference's own C++ launchers, so a
// ctypes harness can drive the reference kernels rebuilt for sm_100a.
// TEST INFRASTRUCTURE ONLY: compiled together with the reference's sources
// (where they lie in the reference tree) into oracle/_ref/libds4ref.so by
// oracle/Makefile.  Nothing here is part of the product library.
#include <cstdint>
#include <cuda_runtime.h>

#include "attn_out.cuh"
#include "compressor.cuh"
#include "dense_q8.cuh"
#include "elementwise.cuh"
#include "embedding.cuh"
#include "fp8_kv.cuh"
#include "glu.cuh"
#include "hc_sinkhorn.cuh"
#include "moe_iq2_pair.cuh"
#include "norm.cuh"
#include "output_head.cuh"
#include "rope.cuh"
#include "router.cuh"

#define S(s) static_cast<cudaStream_t>(s)
using namespace ds4cuda;

extern "C" {

void ds4ref_rms_norm_f32(const float *x, const float *w, float *y, int n, float eps, void *s) {
    launch_rms_norm_f32(x, w, y, n, eps, S(s));
}
void ds4ref_rms_norm_batch_f32(const float *x, const float *w, int weight_dim, float *y, int n_rows,
                               int n_per_row, float eps, void *s) {
    launch_rms_norm_batch_f32(x, w, weight_dim, y, n_rows, n_per_row, eps, S(s));
}
void ds4ref_add_f32(const float *a, const float *b, float *y, int n, void *s) {
    launch_add_f32(a, b, y, n, S(s));
}
void ds4ref_tail_rope_yarn_f32(const float *x_in, float *x_out, int n_heads, int head_dim, int n_rot,
                               int pos, int il, void *s) {
    launch_tail_rope_yarn_f32(x_in, x_out, n_heads, head_dim, n_rot, pos, il, S(s));
}
void ds4ref_tail_rope_yarn_inverse_f32(const float *x_in, float *x_out, int n_heads, int head_dim,
                                       int n_rot, int pos, int il, void *s) {
    launch_tail_rope_yarn_inverse_f32(x_in, x_out, n_heads, head_dim, n_rot, pos, il, S(s));
}
void ds4ref_fp8_kv_quantize_round_trip_f32(const float *kv_in, float *kv_out, int n_rows,
                                           int head_dim, int n_rot, void *s) {
    launch_fp8_kv_quantize_round_trip_f32(kv_in, kv_out, n_rows, head_dim, n_rot, S(s));
}
void ds4ref_silu_mul_f32(const float *g, const float *u, float *y, int n, void *s) {
    launch_silu_mul_f32(g, u, y, n, S(s));
}
void ds4ref_embed_token_f16_to_f32(const uint16_t *table, int token_id, int n_embd, float *out,
                                   void *s) {
    launch_embed_token_f16_to_f32(table, token_id, n_embd, out, S(s));
}
void ds4ref_dequant_q8_0_to_f32(const void *blocks, float *dst, int n_blocks, void *s) {
    launch_dequant_q8_0_to_f32(static_cast<const block_q8_0 *>(blocks), dst, n_blocks, S(s));
}
void ds4ref_hc_attn_pre_f32(const float *residual_hc, const uint16_t *fn, const float *scale,
                            const float *base, float *post, float *comb, float *out, int n_embd,
                            int n_hc, int iters, float eps, void *s) {
    launch_hc_attn_pre_f32(residual_hc, fn, scale, base, post, comb, out, n_embd, n_hc, iters, eps, S(s));
}
void ds4ref_hc_attn_pre_v2_f32(const float *residual_hc, const uint16_t *fn, const float *scale,
                               const float *base, float *post, float *comb, float *out, int n_embd,
                               int n_hc, int iters, float eps, float *rms_scratch, float *mix_scratch,
                               void *s) {
    launch_hc_attn_pre_v2_f32(residual_hc, fn, scale, base, post, comb, out, n_embd, n_hc, iters, eps,
                              rms_scratch, mix_scratch, S(s));
}
void ds4ref_hc_post_f32(const float *block_out, const float *residual_hc, const float *post,
                        const float *comb, float *out_hc, int n_hc, int n_embd, void *s) {
    launch_hc_post_f32(block_out, residual_hc, post, comb, out_hc, n_hc, n_embd, S(s));
}

void ds4ref_output_hc_head_f32(const float *residual_hc, const uint16_t *fn, const float *scale, const float *base,
                               float *out, int n_embd, int n_hc, float eps, void *s) {
    launch_output_hc_head_f32(residual_hc, fn, scale, base, out, n_embd, n_hc, eps, S(s));
}

// ---- per-token loops, issued from C++ the way the reference's forward pass issues them
// (cuda/forward_batch.cu:264-284 calls the single-token launchers once per token) ----------

void ds4ref_loop_q8_gather_add_norm(const void *blocks, const float *resid, const float *w, float *row,
                                    float *sum, float *normed, int n_tokens, int n_embd, float eps, void *s) {
    const int nb = n_embd / 32;
    for (int t = 0; t < n_tokens; ++t) {
        launch_dequant_q8_0_to_f32(static_cast<const block_q8_0 *>(blocks) + (size_t)t * nb, row + (size_t)t * n_embd, nb, S(s));
        launch_add_f32(row + (size_t)t * n_embd, resid + (size_t)t * n_embd, sum + (size_t)t * n_embd, n_embd, S(s));
        launch_rms_norm_f32(sum + (size_t)t * n_embd, w, normed + (size_t)t * n_embd, n_embd, eps, S(s));
    }
}
void ds4ref_loop_kv_rope_fp8(float *kv, int n_tokens, int head_dim, int n_rot, int il, void *s) {
    for (int t = 0; t < n_tokens; ++t)
        launch_tail_rope_yarn_f32(kv + (size_t)t * head_dim, kv + (size_t)t * head_dim, 1, head_dim, n_rot, t, il, S(s));
    launch_fp8_kv_quantize_round_trip_f32(kv, kv, n_tokens, head_dim, n_rot, S(s));
}
void ds4ref_loop_hc_post(const float *block_out, const float *residual_hc, const float *post, const float *comb,
                         float *out_hc, int n_tokens, int n_embd, void *s) {
    for (int t = 0; t < n_tokens; ++t)
        launch_hc_post_f32(block_out, residual_hc + (size_t)t * 4 * n_embd, post, comb,
                           out_hc + (size_t)t * 4 * n_embd, 4, n_embd, S(s));
}


// The two activation quantisers: Q8_K has its own launcher; Q8_0 runs inside the Q8_0 matvec and
// leaves its result in the caller's scratch.
void ds4ref_quantize_fp32_to_q8_K(const float *x, int8_t *xq, float *xscale, int16_t *xbsums, int n_blocks, void *s) {
    launch_quantize_fp32_to_q8_K(x, xq, xscale, xbsums, n_blocks, S(s));
}
void ds4ref_mul_mv_q8_0_q8_0_f32_prealloc(const void *w_blocks, const float *x, float *y, int n_rows, int n_cols,
                                          int8_t *scratch_xq, float *scratch_xscale, void *s) {
    launch_mul_mv_q8_0_q8_0_f32_prealloc(static_cast<const block_q8_0 *>(w_blocks), x, y, n_rows, n_cols, scratch_xq,
                                         scratch_xscale, S(s));
}

// The grouped out-projection quantises its input (the rows behind the inverse RoPE) into caller scratch.
void ds4ref_mul_mv_q8_0_q8_0_grouped_f32_prealloc(const void *w_blocks, const float *x, float *y, int n_groups,
                                                  int group_dim, int rank, int8_t *scratch_xq, float *scratch_xscale,
                                                  void *s) {
    launch_mul_mv_q8_0_q8_0_grouped_f32_prealloc(static_cast<const block_q8_0 *>(w_blocks), x, y, n_groups, group_dim,
                                                 rank, scratch_xq, scratch_xscale, S(s));
}

void ds4ref_mul_mv_f16_f32(const uint16_t *w, const float *x, float *y, int out_dim, int in_dim, void *s) {
    launch_mul_mv_f16_f32(w, x, y, out_dim, in_dim, S(s));
}

// The whole compressor step (projections included) with caller-owned scratch, so that the
// harness can read back the projections the step used.
int ds4ref_compressor_decode_step_prealloc(int is_attn, const float *x, const uint16_t *w_kv,
                                           const uint16_t *w_gate, const uint16_t *w_ape, const float *w_norm,
                                           int in_dim, int head_dim_out, int ratio, int pos, int il,
                                           float *state_kv, float *state_score, float *emit_out,
                                           float *scratch_kv, float *scratch_sc, void *s) {
    int emitted = 0;
    launch_compressor_decode_step_f32_prealloc(is_attn != 0, x, w_kv, w_gate, w_ape, w_norm, in_dim, head_dim_out,
                                               ratio, pos, il, state_kv, state_score, emit_out, &emitted,
                                               scratch_kv, scratch_sc, S(s));
    return emitted;
}
}  // extern "C"
