// launchers.cu — the reference's launcher functions (namespace ds4cuda, same
// parameter lists as cuda/{norm,elementwise,rope,attn_out,fp8_kv,glu,embedding,
// hc_sinkhorn}.cuh) implemented on top of the batched sm_100a kernels, plus
// `extern "C"` names for them.  Same convention as the reference: asynchronous,
// unchecked, `void`; the caller inspects cudaGetLastError().
#include <cmath>

#include "../../include/ds4b200.h"
#include "../../include/ds4b200_launchers.cuh"
#include "kernels.cuh"

// ---------------------------------------------------------------------------
// Host-side RoPE routing (cuda/rope.cu:214-250, cuda/attn_out.cu:216-245)
// ---------------------------------------------------------------------------
extern "C" void ds4b200_rope_params_explicit(float freq_base, float yarn_factor, int n_ctx_orig,
                                             int n_rot, ds4b200_rope_params *out) {
    ds4b200_rope_params p{};
    p.freq_base = freq_base;
    p.theta_scale = std::pow(freq_base, -2.0f / (float)n_rot);
    p.freq_scale = 1.0f;
    p.ext_factor = 0.0f;
    p.attn_factor = 1.0f;
    if (yarn_factor > 1.0f) {
        p.freq_scale = 1.0f / yarn_factor;
        p.ext_factor = 1.0f;
        p.attn_factor = 1.0f / (1.0f + 0.1f * std::log(1.0f / p.freq_scale));
        const float two_pi = 2.0f * 3.14159265358979323846f;
        const float denom = 2.0f * std::log(freq_base);
        const float lo = (float)n_rot * std::log((float)n_ctx_orig / (32.0f * two_pi)) / denom;
        const float hi = (float)n_rot * std::log((float)n_ctx_orig / (1.0f * two_pi)) / denom;
        p.corr_low = std::fmax(0.0f, std::floor(lo));
        p.corr_high = std::fmin((float)(n_rot - 1), std::ceil(hi));
    }
    *out = p;
}

extern "C" void ds4b200_rope_params_for_layer(int il, int n_rot, ds4b200_rope_params *out) {
    // layers 0 and 1 are dense: base 1e4, YaRN off; later layers are compressed:
    // base 1.6e5, factor 16, original context 65536 (cuda/rope.cu:114-126).
    if (il < 2) ds4b200_rope_params_explicit(10000.0f, 1.0f, 0, n_rot, out);
    else ds4b200_rope_params_explicit(160000.0f, 16.0f, 65536, n_rot, out);
    out->theta_scale = 0.0f;   // evaluated on the device, as the reference kernel does
}

namespace ds4cuda {

void launch_rms_norm_f32(const float *x, const float *w, float *y, int n, float eps,
                         cudaStream_t stream) {
    ds4b200::rms_norm_rows(x, nullptr, w, n, y, nullptr, nullptr, 1, n, eps, stream);
}

void launch_rms_norm_batch_f32(const float *x, const float *w, int weight_dim, float *y,
                               int n_rows, int n_per_row, float eps, cudaStream_t stream) {
    ds4b200::rms_norm_rows(x, nullptr, w, weight_dim, y, nullptr, nullptr, n_rows, n_per_row, eps,
                           stream);
}

void launch_add_f32(const float *a, const float *b, float *y, int n, cudaStream_t stream) {
    ds4b200::add_f32(a, b, y, n, stream);
}

void launch_tail_rope_yarn_f32(const float *x_in, float *x_out, int n_heads, int head_dim,
                               int n_rot, int pos, int il, cudaStream_t stream) {
    ds4b200_rope_params p;
    ds4b200_rope_params_for_layer(il, n_rot, &p);
    ds4b200::rope_rows(x_in, x_out, 1, n_heads, head_dim, n_rot, nullptr, pos, p, 0, 0, 0.0f, stream);
}

void launch_tail_rope_yarn_inverse_f32(const float *x_in, float *x_out, int n_heads,
                                       int head_dim, int n_rot, int pos, int il,
                                       cudaStream_t stream) {
    ds4b200_rope_params p;
    ds4b200_rope_params_for_layer(il, n_rot, &p);
    ds4b200::rope_rows(x_in, x_out, 1, n_heads, head_dim, n_rot, nullptr, pos, p, 1, 0, 0.0f, stream);
}

void launch_fp8_kv_quantize_round_trip_f32(const float *kv_in, float *kv_out, int n_rows,
                                           int head_dim, int n_rot, cudaStream_t stream) {
    ds4b200::fp8_kv_round_trip_rows(kv_in, kv_out, n_rows, head_dim, n_rot, stream);
}

void launch_silu_mul_f32(const float *g, const float *u, float *y, int n, cudaStream_t stream) {
    ds4b200::swiglu_rows(g, u, nullptr, y, 1, 1, n, DS4B200_GLU_PLAIN, 0.0f, 0, 0, stream);
}

void launch_embed_token_f16_to_f32(const uint16_t *token_embd_weight, int token_id, int n_embd,
                                   float *out, cudaStream_t stream) {
    ds4b200::embed_gather_rows(token_embd_weight, DS4B200_TABLE_F16, nullptr, token_id, 1, n_embd,
                               nullptr, nullptr, 0.0f, out, 1, nullptr, nullptr, stream);
}

void launch_hc_attn_pre_f32(const float *residual_hc, const uint16_t *hc_attn_fn,
                            const float *hc_attn_scale, const float *hc_attn_base,
                            float *post_weights, float *comb, float *out, int n_embd, int n_hc,
                            int sinkhorn_iters, float eps, cudaStream_t stream) {
    (void)n_hc;   // fixed at 4, as in the reference (cuda/hc_sinkhorn.cu:8-12)
    ds4b200::hc_pre_rows(residual_hc, hc_attn_fn, hc_attn_scale, hc_attn_base, post_weights, comb,
                         out, 1, n_embd, sinkhorn_iters, eps, stream);
}

void launch_hc_attn_pre_v2_f32(const float *residual_hc, const uint16_t *hc_attn_fn,
                               const float *hc_attn_scale, const float *hc_attn_base,
                               float *post_weights, float *comb, float *out, int n_embd,
                               int n_hc, int sinkhorn_iters, float eps, float *rms_scratch,
                               float *mix_scratch, cudaStream_t stream) {
    (void)rms_scratch;
    (void)mix_scratch;
    launch_hc_attn_pre_f32(residual_hc, hc_attn_fn, hc_attn_scale, hc_attn_base, post_weights,
                           comb, out, n_embd, n_hc, sinkhorn_iters, eps, stream);
}

void launch_hc_ffn_pre_v2_f32(const float *residual_hc, const uint16_t *hc_ffn_fn,
                              const float *hc_ffn_scale, const float *hc_ffn_base,
                              float *post_weights, float *comb, float *out, int n_embd, int n_hc,
                              int sinkhorn_iters, float eps, float *rms_scratch,
                              float *mix_scratch, cudaStream_t stream) {
    launch_hc_attn_pre_v2_f32(residual_hc, hc_ffn_fn, hc_ffn_scale, hc_ffn_base, post_weights,
                              comb, out, n_embd, n_hc, sinkhorn_iters, eps, rms_scratch,
                              mix_scratch, stream);
}

void launch_hc_post_f32(const float *block_out, const float *residual_hc, const float *post,
                        const float *comb, float *out_hc, int n_hc, int n_embd,
                        cudaStream_t stream) {
    (void)n_hc;
    ds4b200::hc_post_rows(block_out, nullptr, residual_hc, post, comb, nullptr, nullptr, out_hc, 1,
                          n_embd, 0, 0.0f, stream);
}

void launch_output_hc_head_f32(const float *residual_hc, const uint16_t *output_hc_fn,
                               const float *output_hc_scale, const float *output_hc_base, float *out,
                               int n_embd, int n_hc, float eps, cudaStream_t stream) {
    (void)n_hc;
    ds4b200::hc_head_rows(residual_hc, output_hc_fn, output_hc_scale, output_hc_base, nullptr, out, nullptr, 1,
                          n_embd, eps, stream);
}

}  // namespace ds4cuda

// ---------------------------------------------------------------------------
// C names
// ---------------------------------------------------------------------------
#define S(stream) static_cast<cudaStream_t>(stream)
extern "C" {

void ds4b200_launch_rms_norm_f32(const float *x, const float *w, float *y, int n, float eps,
                                 void *stream) {
    ds4cuda::launch_rms_norm_f32(x, w, y, n, eps, S(stream));
}
void ds4b200_launch_rms_norm_batch_f32(const float *x, const float *w, int weight_dim, float *y,
                                       int n_rows, int n_per_row, float eps, void *stream) {
    ds4cuda::launch_rms_norm_batch_f32(x, w, weight_dim, y, n_rows, n_per_row, eps, S(stream));
}
void ds4b200_launch_add_f32(const float *a, const float *b, float *y, int n, void *stream) {
    ds4cuda::launch_add_f32(a, b, y, n, S(stream));
}
void ds4b200_launch_tail_rope_yarn_f32(const float *x_in, float *x_out, int n_heads, int head_dim,
                                       int n_rot, int pos, int il, void *stream) {
    ds4cuda::launch_tail_rope_yarn_f32(x_in, x_out, n_heads, head_dim, n_rot, pos, il, S(stream));
}
void ds4b200_launch_tail_rope_yarn_inverse_f32(const float *x_in, float *x_out, int n_heads,
                                               int head_dim, int n_rot, int pos, int il,
                                               void *stream) {
    ds4cuda::launch_tail_rope_yarn_inverse_f32(x_in, x_out, n_heads, head_dim, n_rot, pos, il,
                                               S(stream));
}
void ds4b200_launch_fp8_kv_quantize_round_trip_f32(const float *kv_in, float *kv_out, int n_rows,
                                                   int head_dim, int n_rot, void *stream) {
    ds4cuda::launch_fp8_kv_quantize_round_trip_f32(kv_in, kv_out, n_rows, head_dim, n_rot, S(stream));
}
void ds4b200_launch_silu_mul_f32(const float *g, const float *u, float *y, int n, void *stream) {
    ds4cuda::launch_silu_mul_f32(g, u, y, n, S(stream));
}
void ds4b200_launch_embed_token_f16_to_f32(const uint16_t *token_embd_weight, int token_id,
                                           int n_embd, float *out, void *stream) {
    ds4cuda::launch_embed_token_f16_to_f32(token_embd_weight, token_id, n_embd, out, S(stream));
}
void ds4b200_launch_hc_attn_pre_f32(const float *residual_hc, const uint16_t *hc_fn,
                                    const float *hc_scale, const float *hc_base,
                                    float *post_weights, float *comb, float *out, int n_embd,
                                    int n_hc, int sinkhorn_iters, float eps, void *stream) {
    ds4cuda::launch_hc_attn_pre_f32(residual_hc, hc_fn, hc_scale, hc_base, post_weights, comb, out,
                                    n_embd, n_hc, sinkhorn_iters, eps, S(stream));
}
void ds4b200_launch_hc_attn_pre_v2_f32(const float *residual_hc, const uint16_t *hc_fn,
                                       const float *hc_scale, const float *hc_base,
                                       float *post_weights, float *comb, float *out, int n_embd,
                                       int n_hc, int sinkhorn_iters, float eps,
                                       float *rms_scratch, float *mix_scratch, void *stream) {
    ds4cuda::launch_hc_attn_pre_v2_f32(residual_hc, hc_fn, hc_scale, hc_base, post_weights, comb,
                                       out, n_embd, n_hc, sinkhorn_iters, eps, rms_scratch,
                                       mix_scratch, S(stream));
}
void ds4b200_launch_hc_post_f32(const float *block_out, const float *residual_hc,
                                const float *post, const float *comb, float *out_hc, int n_hc,
                                int n_embd, void *stream) {
    ds4cuda::launch_hc_post_f32(block_out, residual_hc, post, comb, out_hc, n_hc, n_embd, S(stream));
}

void ds4b200_launch_output_hc_head_f32(const float *residual_hc, const uint16_t *output_hc_fn,
                                       const float *output_hc_scale, const float *output_hc_base,
                                       float *out, int n_embd, int n_hc, float eps, void *stream) {
    ds4cuda::launch_output_hc_head_f32(residual_hc, output_hc_fn, output_hc_scale, output_hc_base, out, n_embd,
                                       n_hc, eps, S(stream));
}

}  // extern "C"
