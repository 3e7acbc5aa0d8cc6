/* ds4_oracle.h — scalar CPU restatement of the ds4cuda fused elementwise /
 * row-reduction path.  TEST INFRASTRUCTURE ONLY: this library is the checker
 * for the CUDA kernels (tests, the smoke check and the CPU-baseline leg of the
 * benchmark).  Nothing on the product path links, loads or calls it.
 *
 * Parity status: the reference ships no golden vectors for this path and the
 * upstream CPU program its comments quote (antirez/ds4, ds4.c) is not part of
 * the reference tree, so each function below restates the arithmetic of the
 * reference CUDA kernel named in its comment.  The restatement is pinned by
 * (a) the known-answer constants the reference does state (E4M3FN table
 * endpoints, Q8_0 block size, YaRN constants) and (b) outputs of the
 * reference's own kernels, rebuilt for sm_100a and run on a B200, committed
 * as fixtures under tests/golden/.
 *
 * All arithmetic is IEEE binary32 unless stated, compiled with
 * -ffp-contract=off so no fused multiply-add is introduced.
 */
#ifndef DS4_ORACLE_H
#define DS4_ORACLE_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- shared parameter blocks (mirrored by include/ds4b200.h) ---------- */

typedef struct ds4o_rope_params {
    float freq_base;
    float theta_scale;   /* powf(freq_base, -2/n_rot), host libm */
    float freq_scale;
    float ext_factor;
    float attn_factor;
    float corr_low;
    float corr_high;
} ds4o_rope_params;

enum { DS4O_TABLE_F16 = 0, DS4O_TABLE_Q8_0 = 1 };
enum { DS4O_FP8_BLOCK64_POW2 = 0, DS4O_FP8_ROW_AMAX = 1 };
enum {
    DS4O_GLU_PLAIN       = 0,  /* (g*sigmoid(g))*u, cuda/glu.cu:56-75            */
    DS4O_GLU_CLAMP_REF   = 1,  /* gate<=c, |up|<=c, cuda/moe_iq2_pair.cu:352-373 */
    DS4O_GLU_CLAMP_SYM   = 2   /* |gate|<=c, |up|<=c (benchmark-config wording)  */
};

/* ---- conversions ------------------------------------------------------ */
float    ds4o_f16_to_f32(uint16_t h);            /* cuda/common.cuh:20-24 */
uint16_t ds4o_f32_to_f16(float f);               /* RNE, test-input helper */
uint16_t ds4o_f32_to_bf16(float f);              /* RNE */
float    ds4o_bf16_to_f32(uint16_t h);

/* f32 -> f16 -> f32 per element: the rounding rows get when they enter the raw KV cache
 * (cuda/forward_layer.cu:182-190). */
void ds4o_f16_round(const float *x, float *y, int64_t n);

/* ---- E4M3FN ------------------------------------------------------------ */
float   ds4o_e4m3_value(int idx);                /* cuda/fp8_kv.cu:88-94   */
int     ds4o_e4m3_nearest_index(float ax);       /* cuda/fp8_kv.cu:102-131 */
uint8_t ds4o_e4m3_encode(float v);               /* sign bit | nearest index, saturating */
float   ds4o_e4m3_decode(uint8_t code);

/* ---- RMSNorm / add ------------------------------------------------------ */
/* cuda/norm.cu:52-105,126-197.  weight_dim: 0 unit, n shared, n*n_rows per row.
 * residual_in (nullable) is added to x first (one RN add per element); the sum
 * is written to residual_out (nullable).  y_f32 / y_bf16 nullable. */
void ds4o_rms_norm_rows(const float *x, const float *residual_in,
                        const float *w, int64_t weight_dim,
                        float *y_f32, uint16_t *y_bf16, float *residual_out,
                        int64_t n_rows, int n, float eps);
void ds4o_add(const float *a, const float *b, float *y, int64_t n); /* cuda/elementwise.cu:36-43 */

/* ---- RoPE ---------------------------------------------------------------- */
/* Reference per-layer routing, cuda/rope.cu:204-250. */
void ds4o_rope_params_for_layer(int il, int n_rot, ds4o_rope_params *p);
/* Explicit parameters: base, YaRN factor (<=1 disables YaRN), original context. */
void ds4o_rope_params_explicit(float freq_base, float yarn_factor, int n_ctx_orig,
                               int n_rot, ds4o_rope_params *p);
/* cuda/rope.cu:136-201 (+ cuda/attn_out.cu:97-106 for inverse).  Rows are
 * [n_tokens][n_heads][head_dim]; pos has one entry per token.  When
 * unit_rms != 0 every head row is first RMS-normalised with unit gain
 * (cuda/norm.cu:182-185), the q_norm -> RoPE chain of cuda/forward_layer.cu:890-901. */
void ds4o_rope_rows(const float *x_in, float *x_out, int64_t n_tokens, int n_heads,
                    int head_dim, int n_rot, const int32_t *pos,
                    const ds4o_rope_params *p, int inverse, int unit_rms, float eps);

/* ---- FP8 KV --------------------------------------------------------------- */
/* cuda/fp8_kv.cu:144-195: per-64 power-of-two scale on the first
 * head_dim-n_rot elements, round trip to f32, tail copied. */
void ds4o_fp8_kv_round_trip_rows(const float *kv_in, float *kv_out, int64_t n_rows,
                                 int head_dim, int n_rot);
/* Quantise already-rotated rows to bytes + scales.
 *   BLOCK64_POW2: codes for the first head_dim-n_rot elements (n_nope/64 scales
 *                 per row, the reference's rule); the tail is written as f32 to
 *                 tail_out (nullable -> dropped).
 *   ROW_AMAX:     codes for all head_dim elements, one scale = max(amax,1e-4)/448.
 * codes row stride = head_dim bytes; slots (nullable) scatter row r to slot[r]. */
void ds4o_fp8_encode_rows(const float *rows, int64_t n_rows, int head_dim, int n_rot,
                          int scale_mode, const int32_t *slots,
                          uint8_t *codes, float *scales, float *tail_out);
/* Fused chain: optional weighted RMSNorm (norm_w nullable) -> RoPE at pos[r]
 * -> encode as above.  rope_out (nullable) receives the f32 row after RoPE. */
void ds4o_rope_fp8_store_rows(const float *kv_in, int64_t n_rows, int head_dim, int n_rot,
                              const int32_t *pos, const ds4o_rope_params *p,
                              const float *norm_w, float eps,
                              int scale_mode, const int32_t *slots,
                              uint8_t *codes, float *scales, float *tail_out,
                              float *rope_out);

/* ---- activation quantisers that sit between these ops and the matvecs ------- */
/* Q8_0 split form (cuda/dense_q8.cu:122-152): per 32 elements d = amax/127 kept as f32,
 * q = clamp(rint(x * (d != 0 ? 1/d : 0)), -128, 127), ties to even. */
void ds4o_quantize_q8_0_rows(const float *x, int8_t *xq, float *xscale, int64_t n_blocks);
/* Q8_K (cuda/moe_iq2_pair.cu:159-235): per 256 elements, `max` = the element of largest
 * magnitude (first one on ties), iscale = -127/max, q = clamp(rint(iscale*x)), 16 sums of
 * 16 consecutive q, scale = 1/iscale; an all-zero block gives zeros and scale 0. */
void ds4o_quantize_q8_K_rows(const float *x, int8_t *xq, float *xscale, int16_t *xbsums, int64_t n_blocks);

/* ---- SwiGLU ---------------------------------------------------------------- */
/* gate/up: [n_tokens][k][n]; weights (nullable): [n_tokens][k];
 * combine != 0: out[n_tokens][n] = sum over slots in order; else out[n_tokens][k][n]. */
void ds4o_swiglu_rows(const float *gate, const float *up, const float *weights,
                      float *out, int64_t n_tokens, int k, int n,
                      int mode, float clamp, int combine);

/* ---- embedding gather --------------------------------------------------------- */
/* cuda/embedding.cu:27-39 (F16) and cuda/dense_q8.cu:60-67 (Q8_0 blocks of 34 B).
 * out_rows[t][rep][n] (n_replicas copies, cuda/forward_token.cu:350-354) gets
 * dequant(row)+residual_in[t] (residual nullable).  When norm_w != NULL the
 * RMSNorm of that sum is written to normed_f32 / normed_bf16 (nullable each). */
void ds4o_embed_gather_rows(const void *table, int table_dtype, const int32_t *ids,
                            int64_t n_tokens, int n_embd, const float *residual_in,
                            const float *norm_w, float eps,
                            float *out_rows, int n_replicas,
                            float *normed_f32, uint16_t *normed_bf16);

/* ---- hyper-connections ------------------------------------------------------------ */
/* Sinkhorn on 16 pre-softmax values v[src+4*dst] (cuda/hc_sinkhorn.cu:224-289). */
void ds4o_sinkhorn_4x4(const float *v, int iters, float eps, float *comb);
/* Full HC pre for n_tokens tokens, cuda/hc_sinkhorn.cu:85-305.
 * mix_out (nullable) receives the 24 matvec results per token. */
void ds4o_hc_pre_rows(const float *residual_hc, const uint16_t *fn_f16,
                      const float *scale3, const float *base24,
                      float *post, float *comb, float *out, float *mix_out,
                      int64_t n_tokens, int n_embd, int iters, float eps);
/* HC post, cuda/hc_sinkhorn.cu:619-672.  block_out nullable (term dropped);
 * block_out2 nullable (when given, block term = block_out+block_out2, the
 * fused cuda/forward_layer.cu:1447 add). */
void ds4o_hc_post_rows(const float *block_out, const float *block_out2,
                       const float *residual_hc, const float *post, const float *comb,
                       float *out_hc, int64_t n_tokens, int n_embd);
/* Output HC head (cuda/output_head.cu:62-149): RMS over the 4*n_embd block, 4-row f16
 * matvec, w[h] = sigmoid(pre[h]*scale[0] + base[h]) + eps, out = sum_h x[h]*w[h] in order.
 * When norm_w != NULL the output RMSNorm that follows it (cuda/forward_token.cu:211,
 * cuda/norm.cu:52-105) is applied to `out` and written to normed. */
void ds4o_output_hc_head_rows(const float *residual_hc, const uint16_t *fn_f16, const float *scale1,
                              const float *base4, const float *norm_w, float *out, float *normed,
                              int64_t n_tokens, int n_embd, float eps);
/* Benchmark config "Sinkhorn mixing": logits[t][16] -> comb -> mix 4 streams. */
void ds4o_hc_sinkhorn_mix_rows(const float *logits, const float *residual_hc,
                               float *out_hc, float *comb_out, int64_t n_tokens,
                               int n_embd, int iters, float eps);

/* One streaming-compressor step after its two projections (cuda/compressor.cu:65-90 bias and
 * state row, :107-164 pool, :173-220 RMSNorm, cuda/rope.cu tail RoPE at pos + 1 - ratio,
 * cuda/fp8_kv.cu round trip when is_attn, :232-252 state roll for ratio 4).
 * width = head_dim * (ratio == 4 ? 2 : 1); state arrays hold (ratio == 4 ? 8 : ratio) rows.
 * Returns 1 when emit_out was written. */
int ds4o_compressor_step(int is_attn, const float *kv_cur, float *sc_cur, const uint16_t *ape_f16,
                         const float *norm_w, int head_dim, int ratio, int pos,
                         const ds4o_rope_params *rope, int n_rot, float eps,
                         float *state_kv, float *state_score, float *emit_out);

#ifdef __cplusplus
}
#endif
#endif /* DS4_ORACLE_H */
