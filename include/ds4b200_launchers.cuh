// ds4b200_launchers.cuh — the reference's kernel launchers for the fused
// elementwise / row-reduction path, re-declared with identical names,
// namespace and parameter lists so that the reference's callers
// (cuda/forward_layer.cu, cuda/forward_token.cu, cuda/forward_batch.cu,
// cuda/compressor.cu) link against libds4b200 unchanged.
//
// Convention, as in the reference: device pointers owned by the caller,
// asynchronous enqueue on `stream`, no allocation, no synchronisation, `void`
// return — the caller checks cudaGetLastError() (cuda/forward_layer.cu:81-89).
// Pointers may have any natural alignment and n any value; 16-byte aligned
// pointers with n % 4 == 0 take the 128-bit path.
#pragma once

#include <cstdint>
#include <cuda_runtime.h>

namespace ds4cuda {

// cuda/norm.cuh:24
void launch_rms_norm_f32(const float *x, const float *w, float *y, int n, float eps,
                         cudaStream_t stream = 0);
// cuda/norm.cuh:42
void launch_rms_norm_batch_f32(const float *x, const float *w, int weight_dim, float *y,
                               int n_rows, int n_per_row, float eps, cudaStream_t stream = 0);
// cuda/elementwise.cuh:27
void launch_add_f32(const float *a, const float *b, float *y, int n, cudaStream_t stream = 0);
// cuda/rope.cuh:51
void launch_tail_rope_yarn_f32(const float *x_in, float *x_out, int n_heads, int head_dim,
                               int n_rot, int pos, int il, cudaStream_t stream = 0);
// cuda/attn_out.cuh:52
void launch_tail_rope_yarn_inverse_f32(const float *x_in, float *x_out, int n_heads,
                                       int head_dim, int n_rot, int pos, int il,
                                       cudaStream_t stream = 0);
// cuda/fp8_kv.cuh:62
void launch_fp8_kv_quantize_round_trip_f32(const float *kv_in, float *kv_out, int n_rows,
                                           int head_dim, int n_rot, cudaStream_t stream = 0);
// cuda/glu.cuh:30
void launch_silu_mul_f32(const float *g, const float *u, float *y, int n,
                         cudaStream_t stream = 0);
// cuda/embedding.cuh:46
void launch_embed_token_f16_to_f32(const uint16_t *token_embd_weight, int token_id,
                                   int n_embd, float *out, cudaStream_t stream = 0);
// cuda/hc_sinkhorn.cuh:55
void launch_hc_attn_pre_f32(const float *residual_hc, const uint16_t *hc_attn_fn,
                            const float *hc_attn_scale, const float *hc_attn_base,
                            float *post_weights, float *comb, float *out, int n_embd,
                            int n_hc, int sinkhorn_iters, float eps, cudaStream_t stream = 0);
// cuda/hc_sinkhorn.cuh:80 — rms_scratch / mix_scratch are accepted and left
// untouched: the fused kernel keeps both values on chip.
void launch_hc_attn_pre_v2_f32(const float *residual_hc, const uint16_t *hc_attn_fn,
                               const float *hc_attn_scale, const float *hc_attn_base,
                               float *post_weights, float *comb, float *out, int n_embd,
                               int n_hc, int sinkhorn_iters, float eps, float *rms_scratch,
                               float *mix_scratch, cudaStream_t stream = 0);
// cuda/hc_sinkhorn.cuh:99
void launch_hc_ffn_pre_v2_f32(const float *residual_hc, const uint16_t *hc_ffn_fn,
                              const float *hc_ffn_scale, const float *hc_ffn_base,
                              float *post_weights, float *comb, float *out, int n_embd,
                              int n_hc, int sinkhorn_iters, float eps, float *rms_scratch,
                              float *mix_scratch, cudaStream_t stream = 0);
// cuda/hc_sinkhorn.cuh:138
void launch_hc_post_f32(const float *block_out, const float *residual_hc, const float *post,
                        const float *comb, float *out_hc, int n_hc, int n_embd,
                        cudaStream_t stream = 0);

// cuda/output_head.cuh:68 — final collapse of the four streams (cuda/forward_token.cu:198)
void launch_output_hc_head_f32(const float *residual_hc, const uint16_t *output_hc_fn,
                               const float *output_hc_scale, const float *output_hc_base, float *out,
                               int n_embd, int n_hc, float eps, cudaStream_t stream = 0);

}  // namespace ds4cuda
