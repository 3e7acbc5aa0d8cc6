/* ds4_oracle.c — scalar CPU restatement of the ds4cuda fused elementwise /
 * row-reduction path.  TEST INFRASTRUCTURE ONLY (see ds4_oracle.h): it is the
 * checker the CUDA kernels are compared with, never a fallback for them.
 *
 * Parity status: restated from the reference CUDA kernels cited per function;
 * pinned by the reference's stated constants and by fixtures produced by the
 * reference's own kernels on a B200 (tests/golden/).
 *
 * Build: cc -O2 -ffp-contract=off -fPIC -shared (see oracle/Makefile).
 */
#include "ds4_oracle.h"

#include <math.h>
#include <stddef.h>
#include <stdlib.h>
#include <string.h>

/* ====================================================================== */
/* conversions                                                            */
/* ====================================================================== */

static inline uint32_t f32_bits(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }
static inline float bits_f32(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }

/* IEEE binary16 -> binary32, exact for every finite and subnormal input
 * (cuda/common.cuh:20-24 does the same through the hardware conversion). */
float ds4o_f16_to_f32(uint16_t h)
{
    const uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    const uint32_t exp  = (h >> 10) & 0x1fu;
    const uint32_t man  = h & 0x3ffu;
    if (exp == 0x1f) return bits_f32(sign | 0x7f800000u | (man << 13));
    if (exp != 0)    return bits_f32(sign | ((exp + 112u) << 23) | (man << 13));
    /* zero / subnormal: man * 2^-24 is exact in binary32 */
    const float mag = (float)man * 5.9604644775390625e-8f;
    return sign ? -mag : mag;
}

uint16_t ds4o_f32_to_f16(float f)
{
    const uint32_t u = f32_bits(f);
    const uint16_t sign = (uint16_t)((u >> 16) & 0x8000u);
    const uint32_t a = u & 0x7fffffffu;
    if (a >= 0x7f800000u) return (uint16_t)(sign | 0x7c00u | (a > 0x7f800000u ? 0x200u : 0));
    if (a >= 0x477ff000u) return (uint16_t)(sign | 0x7c00u);       /* rounds to inf */
    if (a < 0x33000001u)  return sign;                             /* rounds to 0   */
    int e = (int)(a >> 23) - 127;
    uint32_t m = (a & 0x7fffffu) | 0x800000u;
    int shift = (e < -14) ? (13 + (-14 - e)) : 13;
    uint32_t q = m >> shift;
    const uint32_t rem = m & ((1u << shift) - 1u);
    const uint32_t half = 1u << (shift - 1);
    if (rem > half || (rem == half && (q & 1u))) q++;
    if (e < -14) return (uint16_t)(sign | q);                      /* subnormal (q may carry to 0x400) */
    return (uint16_t)(sign | (uint16_t)(((uint32_t)(e + 15) << 10) + (q - 0x400u)));
}

uint16_t ds4o_f32_to_bf16(float f)
{
    uint32_t u = f32_bits(f);
    if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x40u); /* quiet NaN */
    u += 0x7fffu + ((u >> 16) & 1u);
    return (uint16_t)(u >> 16);
}

float ds4o_bf16_to_f32(uint16_t h) { return bits_f32((uint32_t)h << 16); }

void ds4o_f16_round(const float *x, float *y, int64_t n)
{
    for (int64_t i = 0; i < n; i++) y[i] = ds4o_f16_to_f32(ds4o_f32_to_f16(x[i]));
}

/* ====================================================================== */
/* E4M3FN  (cuda/fp8_kv.cu:11-35,88-131)                                   */
/* ====================================================================== */

float ds4o_e4m3_value(int idx)
{
    const int e = (idx >> 3) & 15, m = idx & 7;
    if (e == 0) return (float)m * 0.001953125f;               /* m * 2^-9 */
    return (1.0f + (float)m * 0.125f) * ldexpf(1.0f, e - 7);
}

/* Largest index whose value is <= ax, then step up when the next value is
 * strictly closer, or equally close while the current index is odd. */
int ds4o_e4m3_nearest_index(float ax)
{
    if (ax > 448.0f) ax = 448.0f;
    int i = 0;
    while (i < 126 && ds4o_e4m3_value(i + 1) <= ax) i++;
    if (i < 126) {
        const float d0 = fabsf(ax - ds4o_e4m3_value(i));
        const float d1 = fabsf(ax - ds4o_e4m3_value(i + 1));
        if (d1 < d0 || (d1 == d0 && (i & 1))) i++;
    }
    return i;
}

/* Byte form: bit 7 is the IEEE sign bit of the input (so -0.0 and negative
 * values that round to zero give 0x80, as the hardware conversion does); NaN
 * gives 0x7f | sign.  Callers clamp to +-448 first, as the reference does. */
uint8_t ds4o_e4m3_encode(float v)
{
    const uint8_t sign = (uint8_t)((f32_bits(v) >> 24) & 0x80u);
    if (v != v) return (uint8_t)(sign | 0x7f);
    return (uint8_t)(sign | ds4o_e4m3_nearest_index(fabsf(v)));
}

float ds4o_e4m3_decode(uint8_t code)
{
    const float mag = ds4o_e4m3_value(code & 0x7f);
    return (code & 0x80) ? -mag : mag;
}

/* ====================================================================== */
/* RMSNorm, add                                                            */
/* ====================================================================== */

static float rms_scale_of(const float *x, int64_t n, float eps)
{
    double ss = 0.0;
    for (int64_t i = 0; i < n; i++) ss += (double)x[i] * (double)x[i];
    const float mean = (float)(ss / (double)n);
    return 1.0f / sqrtf(mean + eps);
}

void ds4o_rms_norm_rows(const float *x, const float *residual_in,
                        const float *w, int64_t weight_dim,
                        float *y_f32, uint16_t *y_bf16, float *residual_out,
                        int64_t n_rows, int n, float eps)
{
    float *row = (float *)malloc((size_t)n * 4);
    for (int64_t r = 0; r < n_rows; r++) {
        const float *xr = x + r * n;
        for (int i = 0; i < n; i++)
            row[i] = residual_in ? xr[i] + residual_in[r * n + i] : xr[i];
        if (residual_out) memcpy(residual_out + r * n, row, (size_t)n * 4);
        const float scale = rms_scale_of(row, n, eps);
        const float *wr = (weight_dim == 0) ? NULL
                        : (weight_dim == n) ? w : w + r * n;
        for (int i = 0; i < n; i++) {
            float y = row[i] * scale;
            if (wr) y = y * wr[i];
            if (y_bf16) y_bf16[r * n + i] = ds4o_f32_to_bf16(y);
            if (y_f32)  y_f32[r * n + i] = y;
        }
    }
    free(row);
}

void ds4o_add(const float *a, const float *b, float *y, int64_t n)
{
    for (int64_t i = 0; i < n; i++) y[i] = a[i] + b[i];
}

/* ====================================================================== */
/* RoPE                                                                    */
/* ====================================================================== */

static void yarn_window(float freq_base, int n_ctx_orig, int n_rot, ds4o_rope_params *p)
{
    /* cuda/rope.cu:232-244: beta_fast 32 -> low edge, beta_slow 1 -> high edge */
    const float pi = 3.14159265358979323846f;
    const float c32 = (float)n_rot * logf((float)n_ctx_orig / (32.0f * 2.0f * pi)) / (2.0f * logf(freq_base));
    const float c1  = (float)n_rot * logf((float)n_ctx_orig / (1.0f  * 2.0f * pi)) / (2.0f * logf(freq_base));
    p->corr_low  = fmaxf(0.0f, floorf(c32));
    p->corr_high = fminf((float)(n_rot - 1), ceilf(c1));
}

void ds4o_rope_params_explicit(float freq_base, float yarn_factor, int n_ctx_orig,
                               int n_rot, ds4o_rope_params *p)
{
    p->freq_base = freq_base;
    p->theta_scale = powf(freq_base, -2.0f / (float)n_rot);
    p->corr_low = p->corr_high = 0.0f;
    if (yarn_factor > 1.0f) {
        p->freq_scale  = 1.0f / yarn_factor;
        p->ext_factor  = 1.0f;
        p->attn_factor = 1.0f / (1.0f + 0.1f * logf(1.0f / p->freq_scale));
        yarn_window(freq_base, n_ctx_orig, n_rot, p);
    } else {
        p->freq_scale  = 1.0f;
        p->ext_factor  = 0.0f;
        p->attn_factor = 1.0f;
    }
}

/* cuda/rope.cu:122-126,214-250: layers 0,1 are dense (base 1e4, YaRN off);
 * every later layer uses base 1.6e5, factor 16, original context 65536. */
void ds4o_rope_params_for_layer(int il, int n_rot, ds4o_rope_params *p)
{
    if (il < 2) ds4o_rope_params_explicit(10000.0f, 1.0f, 0, n_rot, p);
    else        ds4o_rope_params_explicit(160000.0f, 16.0f, 65536, n_rot, p);
}

/* Rotate the last n_rot elements of one head row in place (cuda/rope.cu:165-200). */
static void rope_tail_inplace(float *row, int head_dim, int n_rot, int pos,
                              const ds4o_rope_params *p, int inverse)
{
    float *tail = row + (head_dim - n_rot);
    float theta_extrap = (float)pos;
    for (int k = 0; k < n_rot / 2; k++) {
        const float theta_interp = p->freq_scale * theta_extrap;
        float theta = theta_interp, mscale = p->attn_factor;
        if (p->ext_factor != 0.0f) {
            const float y = ((float)k - p->corr_low) / fmaxf(0.001f, p->corr_high - p->corr_low);
            const float ramp = (1.0f - fminf(1.0f, fmaxf(0.0f, y))) * p->ext_factor;
            const float a = theta_interp * (1.0f - ramp);
            const float b = theta_extrap * ramp;
            theta = a + b;
            mscale *= 1.0f + 0.1f * logf(1.0f / p->freq_scale);
        }
        const float c = cosf(theta) * mscale;
        float s = sinf(theta) * mscale;
        if (inverse) s = -s;
        const float x0 = tail[2 * k], x1 = tail[2 * k + 1];
        const float p00 = x0 * c, p11 = x1 * s, p01 = x0 * s, p10 = x1 * c;
        tail[2 * k]     = p00 - p11;
        tail[2 * k + 1] = p01 + p10;
        theta_extrap *= p->theta_scale;
    }
}

void ds4o_rope_rows(const float *x_in, float *x_out, int64_t n_tokens, int n_heads,
                    int head_dim, int n_rot, const int32_t *pos,
                    const ds4o_rope_params *p, int inverse, int unit_rms, float eps)
{
    for (int64_t t = 0; t < n_tokens; t++) {
        for (int h = 0; h < n_heads; h++) {
            const int64_t off = (t * n_heads + h) * (int64_t)head_dim;
            if (x_out != x_in) memmove(x_out + off, x_in + off, (size_t)head_dim * 4);
            float *row = x_out + off;
            if (unit_rms) {
                const float scale = rms_scale_of(row, head_dim, eps);
                for (int i = 0; i < head_dim; i++) row[i] = row[i] * scale;
            }
            rope_tail_inplace(row, head_dim, n_rot, pos[t], p, inverse);
        }
    }
}

/* ====================================================================== */
/* FP8 KV                                                                  */
/* ====================================================================== */

#define FP8_MAX 448.0f
#define FP8_AMAX_FLOOR 1.0e-4f

static float block_amax(const float *x, int n)
{
    float m = 0.0f;
    for (int i = 0; i < n; i++) m = fmaxf(m, fabsf(x[i]));
    return fmaxf(m, FP8_AMAX_FLOOR);
}

static inline float pow2_scale(float amax) { return exp2f(ceilf(log2f(amax / FP8_MAX))); }
static inline float clamp448(float v) { return fminf(fmaxf(v, -FP8_MAX), FP8_MAX); }

void ds4o_fp8_kv_round_trip_rows(const float *kv_in, float *kv_out, int64_t n_rows,
                                 int head_dim, int n_rot)
{
    const int n_nope = head_dim - n_rot;
    for (int64_t r = 0; r < n_rows; r++) {
        const float *in = kv_in + r * head_dim;
        float *out = kv_out + r * head_dim;
        for (int off = 0; off < n_nope; off += 64) {
            const float scale = pow2_scale(block_amax(in + off, 64));
            for (int j = 0; j < 64; j++) {
                const float v = clamp448(in[off + j] / scale);
                const float sign = (v < 0.0f) ? -1.0f : 1.0f;
                out[off + j] = (sign * ds4o_e4m3_value(ds4o_e4m3_nearest_index(fabsf(v)))) * scale;
            }
        }
        for (int j = n_nope; j < head_dim; j++) out[j] = in[j];
    }
}

static void fp8_encode_row(const float *row, int head_dim, int n_rot, int scale_mode,
                           uint8_t *codes, float *scales, float *tail_out)
{
    const int n_nope = head_dim - n_rot;
    if (scale_mode == DS4O_FP8_BLOCK64_POW2) {
        for (int off = 0; off < n_nope; off += 64) {
            const float scale = pow2_scale(block_amax(row + off, 64));
            scales[off / 64] = scale;
            for (int j = 0; j < 64; j++)
                codes[off + j] = ds4o_e4m3_encode(clamp448(row[off + j] / scale));
        }
        for (int j = n_nope; j < head_dim; j++) {
            codes[j] = 0;
            if (tail_out) tail_out[j - n_nope] = row[j];
        }
    } else {
        const float scale = block_amax(row, head_dim) / FP8_MAX;
        scales[0] = scale;
        for (int j = 0; j < head_dim; j++)
            codes[j] = ds4o_e4m3_encode(clamp448(row[j] / scale));
    }
}

void ds4o_fp8_encode_rows(const float *rows, int64_t n_rows, int head_dim, int n_rot,
                          int scale_mode, const int32_t *slots,
                          uint8_t *codes, float *scales, float *tail_out)
{
    const int n_scales = (scale_mode == DS4O_FP8_BLOCK64_POW2) ? (head_dim - n_rot) / 64 : 1;
    for (int64_t r = 0; r < n_rows; r++) {
        const int64_t s = slots ? slots[r] : r;
        fp8_encode_row(rows + r * head_dim, head_dim, n_rot, scale_mode,
                       codes + s * head_dim, scales + s * n_scales,
                       tail_out ? tail_out + s * n_rot : NULL);
    }
}

void ds4o_rope_fp8_store_rows(const float *kv_in, int64_t n_rows, int head_dim, int n_rot,
                              const int32_t *pos, const ds4o_rope_params *p,
                              const float *norm_w, float eps,
                              int scale_mode, const int32_t *slots,
                              uint8_t *codes, float *scales, float *tail_out,
                              float *rope_out)
{
    float row[8192];
    const int n_scales = (scale_mode == DS4O_FP8_BLOCK64_POW2) ? (head_dim - n_rot) / 64 : 1;
    for (int64_t r = 0; r < n_rows; r++) {
        memcpy(row, kv_in + r * head_dim, (size_t)head_dim * 4);
        if (norm_w) {
            const float scale = rms_scale_of(row, head_dim, eps);
            for (int i = 0; i < head_dim; i++) row[i] = row[i] * scale * norm_w[i];
        }
        rope_tail_inplace(row, head_dim, n_rot, pos[r], p, 0);
        if (rope_out) memcpy(rope_out + r * head_dim, row, (size_t)head_dim * 4);
        const int64_t s = slots ? slots[r] : r;
        fp8_encode_row(row, head_dim, n_rot, scale_mode, codes + s * head_dim,
                       scales + s * n_scales, tail_out ? tail_out + s * n_rot : NULL);
    }
}

/* ====================================================================== */
/* activation quantisers                                                   */
/* ====================================================================== */

static inline int clamp_i8(long v) { return v > 127 ? 127 : (v < -128 ? -128 : (int)v); }

void ds4o_quantize_q8_0_rows(const float *x, int8_t *xq, float *xscale, int64_t n_blocks)
{
    for (int64_t b = 0; b < n_blocks; b++) {
        const float *xb = x + b * 32;
        float amax = 0.0f;
        for (int i = 0; i < 32; i++) amax = fmaxf(amax, fabsf(xb[i]));
        const float d = amax / 127.0f;
        const float id = (d != 0.0f) ? 1.0f / d : 0.0f;
        xscale[b] = d;
        for (int i = 0; i < 32; i++) xq[b * 32 + i] = (int8_t)clamp_i8(lrintf(xb[i] * id));
    }
}

void ds4o_quantize_q8_K_rows(const float *x, int8_t *xq, float *xscale, int16_t *xbsums, int64_t n_blocks)
{
    for (int64_t b = 0; b < n_blocks; b++) {
        const float *xb = x + b * 256;
        int8_t *qb = xq + b * 256;
        float amax = 0.0f, smax = 0.0f;
        for (int i = 0; i < 256; i++)
            if (fabsf(xb[i]) > amax) { amax = fabsf(xb[i]); smax = xb[i]; }
        if (amax == 0.0f) {
            memset(qb, 0, 256);
            for (int k = 0; k < 16; k++) xbsums[b * 16 + k] = 0;
            xscale[b] = 0.0f;
            continue;
        }
        const float iscale = -127.0f / smax;
        for (int i = 0; i < 256; i++) qb[i] = (int8_t)clamp_i8(lrintf(iscale * xb[i]));
        for (int k = 0; k < 16; k++) {
            int sum = 0;
            for (int j = 0; j < 16; j++) sum += qb[k * 16 + j];
            xbsums[b * 16 + k] = (int16_t)sum;
        }
        xscale[b] = 1.0f / iscale;
    }
}

/* ====================================================================== */
/* SwiGLU                                                                  */
/* ====================================================================== */

static inline float sigmoid_stable(float x)        /* cuda/glu.cu:56-64 */
{
    if (x >= 0.0f) { const float e = expf(-x); return 1.0f / (1.0f + e); }
    const float e = expf(x);
    return e / (1.0f + e);
}

static inline float glu_one(float g, float u, int mode, float clamp)
{
    if (mode == DS4O_GLU_PLAIN) return (g * sigmoid_stable(g)) * u;
    if (clamp > 1.0e-6f) {                          /* cuda/moe_iq2_pair.cu:355-360 */
        if (g > clamp) g = clamp;
        if (mode == DS4O_GLU_CLAMP_SYM && g < -clamp) g = -clamp;
        if (u > clamp) u = clamp;
        if (u < -clamp) u = -clamp;
    }
    float s;                                        /* cuda/moe_iq2_pair.cu:362-369 */
    if (g >= 0.0f) { const float e = expf(-g); s = g / (1.0f + e); }
    else           { const float e = expf(g);  s = g * e / (1.0f + e); }
    return s * u;
}

void ds4o_swiglu_rows(const float *gate, const float *up, const float *weights,
                      float *out, int64_t n_tokens, int k, int n,
                      int mode, float clamp, int combine)
{
    for (int64_t t = 0; t < n_tokens; t++) {
        for (int j = 0; j < n; j++) {
            float acc = 0.0f;
            for (int s = 0; s < k; s++) {
                const int64_t idx = (t * k + s) * (int64_t)n + j;
                float v = glu_one(gate[idx], up[idx], mode, clamp);
                if (weights) v = v * weights[t * k + s];
                if (combine) acc = (s == 0) ? v : acc + v;
                else out[idx] = v;
            }
            if (combine) out[t * n + j] = acc;
        }
    }
}

/* ====================================================================== */
/* embedding gather                                                        */
/* ====================================================================== */

void ds4o_embed_gather_rows(const void *table, int table_dtype, const int32_t *ids,
                            int64_t n_tokens, int n_embd, const float *residual_in,
                            const float *norm_w, float eps,
                            float *out_rows, int n_replicas,
                            float *normed_f32, uint16_t *normed_bf16)
{
    float row[16384];
    for (int64_t t = 0; t < n_tokens; t++) {
        const int64_t id = ids[t];
        if (table_dtype == DS4O_TABLE_F16) {
            const uint16_t *src = (const uint16_t *)table + id * n_embd;
            for (int i = 0; i < n_embd; i++) row[i] = ds4o_f16_to_f32(src[i]);
        } else {
            /* 34-byte records: f16 scale bits, then 32 int8 (cuda/common.cuh:29-33) */
            const uint8_t *src = (const uint8_t *)table + id * (int64_t)(n_embd / 32) * 34;
            for (int b = 0; b < n_embd / 32; b++) {
                const uint8_t *blk = src + b * 34;
                const float d = ds4o_f16_to_f32((uint16_t)(blk[0] | (blk[1] << 8)));
                for (int j = 0; j < 32; j++)
                    row[b * 32 + j] = d * (float)(int8_t)blk[2 + j];
            }
        }
        if (residual_in)
            for (int i = 0; i < n_embd; i++) row[i] = row[i] + residual_in[t * n_embd + i];
        if (out_rows)
            for (int rep = 0; rep < n_replicas; rep++)
                memcpy(out_rows + (t * n_replicas + rep) * (int64_t)n_embd, row, (size_t)n_embd * 4);
        if (norm_w) {
            const float scale = rms_scale_of(row, n_embd, eps);
            for (int i = 0; i < n_embd; i++) {
                const float y = row[i] * scale * norm_w[i];
                if (normed_f32)  normed_f32[t * n_embd + i] = y;
                if (normed_bf16) normed_bf16[t * n_embd + i] = ds4o_f32_to_bf16(y);
            }
        }
    }
}

/* ====================================================================== */
/* hyper-connections                                                       */
/* ====================================================================== */

void ds4o_sinkhorn_4x4(const float *v, int iters, float eps, float *c)
{
    /* row softmax, + eps (cuda/hc_sinkhorn.cu:224-246) */
    for (int dst = 0; dst < 4; dst++) {
        float m = -INFINITY, sum = 0.0f;
        for (int src = 0; src < 4; src++) if (v[src + 4 * dst] > m) m = v[src + 4 * dst];
        for (int src = 0; src < 4; src++) { c[src + 4 * dst] = expf(v[src + 4 * dst] - m); sum += c[src + 4 * dst]; }
        const float inv = 1.0f / sum;
        for (int src = 0; src < 4; src++) c[src + 4 * dst] = c[src + 4 * dst] * inv + eps;
    }
    /* first column pass, then (row, column) iters-1 times (cuda/hc_sinkhorn.cu:249-289) */
    for (int it = 0; it < iters; it++) {
        if (it > 0) {
            for (int dst = 0; dst < 4; dst++) {
                float sum = 0.0f;
                for (int src = 0; src < 4; src++) sum += c[src + 4 * dst];
                const float inv = 1.0f / (sum + eps);
                for (int src = 0; src < 4; src++) c[src + 4 * dst] *= inv;
            }
        }
        for (int src = 0; src < 4; src++) {
            float sum = 0.0f;
            for (int dst = 0; dst < 4; dst++) sum += c[src + 4 * dst];
            const float inv = 1.0f / (sum + eps);
            for (int dst = 0; dst < 4; dst++) c[src + 4 * dst] *= inv;
        }
    }
}

void ds4o_hc_pre_rows(const float *residual_hc, const uint16_t *fn_f16,
                      const float *scale3, const float *base24,
                      float *post, float *comb, float *out, float *mix_out,
                      int64_t n_tokens, int n_embd, int iters, float eps)
{
    const int64_t hc_dim = 4 * (int64_t)n_embd;
    for (int64_t t = 0; t < n_tokens; t++) {
        const float *x = residual_hc + t * hc_dim;
        const float rms = rms_scale_of(x, hc_dim, eps);
        float mix[24], v[16], pre[4];
        for (int o = 0; o < 24; o++) {
            const uint16_t *wrow = fn_f16 + o * hc_dim;
            double acc = 0.0;
            for (int64_t i = 0; i < hc_dim; i++) {
                const float xf = x[i] * rms;
                const float pr = ds4o_f16_to_f32(wrow[i]) * xf;
                acc += (double)pr;
            }
            mix[o] = (float)acc;
            if (mix_out) mix_out[t * 24 + o] = mix[o];
        }
        for (int h = 0; h < 4; h++) {
            const float zp = mix[h] * scale3[0] + base24[h];
            pre[h] = 1.0f / (1.0f + expf(-zp)) + eps;
            const float zq = mix[4 + h] * scale3[1] + base24[4 + h];
            post[t * 4 + h] = 2.0f / (1.0f + expf(-zq));
        }
        for (int i = 0; i < 16; i++) v[i] = mix[8 + i] * scale3[2] + base24[8 + i];
        ds4o_sinkhorn_4x4(v, iters, eps, comb + t * 16);
        for (int d = 0; d < n_embd; d++) {
            float acc = x[d] * pre[0];
            acc = acc + x[n_embd + d] * pre[1];
            acc = acc + x[2 * n_embd + d] * pre[2];
            acc = acc + x[3 * n_embd + d] * pre[3];
            out[t * n_embd + d] = acc;
        }
    }
}

void ds4o_hc_post_rows(const float *block_out, const float *block_out2,
                       const float *residual_hc, const float *post, const float *comb,
                       float *out_hc, int64_t n_tokens, int n_embd)
{
    for (int64_t t = 0; t < n_tokens; t++) {
        const float *x = residual_hc + t * 4 * (int64_t)n_embd;
        const float *c = comb + t * 16;
        for (int dst = 0; dst < 4; dst++) {
            for (int d = 0; d < n_embd; d++) {
                float acc = 0.0f;
                if (block_out) {
                    float b = block_out[t * n_embd + d];
                    if (block_out2) b = b + block_out2[t * n_embd + d];
                    acc = b * post[t * 4 + dst];
                }
                for (int src = 0; src < 4; src++) {
                    const float term = c[dst + 4 * src] * x[src * n_embd + d];
                    acc = (!block_out && src == 0) ? term : acc + term;
                }
                out_hc[(t * 4 + dst) * (int64_t)n_embd + d] = acc;
            }
        }
    }
}

void ds4o_output_hc_head_rows(const float *residual_hc, const uint16_t *fn_f16, const float *scale1,
                              const float *base4, const float *norm_w, float *out, float *normed,
                              int64_t n_tokens, int n_embd, float eps)
{
    const int64_t hc_dim = 4 * (int64_t)n_embd;
    for (int64_t t = 0; t < n_tokens; t++) {
        const float *x = residual_hc + t * hc_dim;
        const float rms = rms_scale_of(x, hc_dim, eps);
        float w[4];
        for (int h = 0; h < 4; h++) {
            double acc = 0.0;
            for (int64_t i = 0; i < hc_dim; i++) {
                const float xf = x[i] * rms;
                const float pr = ds4o_f16_to_f32(fn_f16[h * hc_dim + i]) * xf;
                acc += (double)pr;
            }
            const float z = (float)acc * scale1[0] + base4[h];
            w[h] = 1.0f / (1.0f + expf(-z)) + eps;
        }
        float *o = out + t * n_embd;
        for (int d = 0; d < n_embd; d++) {
            float acc = x[d] * w[0];
            acc = acc + x[n_embd + d] * w[1];
            acc = acc + x[2 * n_embd + d] * w[2];
            acc = acc + x[3 * n_embd + d] * w[3];
            o[d] = acc;
        }
        if (norm_w) {
            const float sc = rms_scale_of(o, n_embd, eps);
            for (int d = 0; d < n_embd; d++) normed[t * n_embd + d] = o[d] * sc * norm_w[d];
        }
    }
}

void ds4o_hc_sinkhorn_mix_rows(const float *logits, const float *residual_hc,
                               float *out_hc, float *comb_out, int64_t n_tokens,
                               int n_embd, int iters, float eps)
{
    for (int64_t t = 0; t < n_tokens; t++) {
        float c[16];
        ds4o_sinkhorn_4x4(logits + t * 16, iters, eps, c);
        if (comb_out) memcpy(comb_out + t * 16, c, sizeof c);
        ds4o_hc_post_rows(NULL, NULL, residual_hc + t * 4 * (int64_t)n_embd, NULL, c,
                          out_hc + t * 4 * (int64_t)n_embd, 1, n_embd);
    }
}

/* ====================================================================== */
/* Streaming compressor step (after the projections)                      */
/* ====================================================================== */

int ds4o_compressor_step(int is_attn, const float *kv_cur, float *sc_cur, const uint16_t *ape_f16,
                         const float *norm_w, int head_dim, int ratio, int pos,
                         const ds4o_rope_params *rope, int n_rot, float eps,
                         float *state_kv, float *state_score, float *emit_out)
{
    const int coff = ratio == 4 ? 2 : 1, width = coff * head_dim;
    const int pos_mod = pos % ratio;
    const int row = ratio == 4 ? ratio + pos_mod : pos_mod;          /* cuda/compressor.cu:84-86 */
    for (int j = 0; j < width; j++) {
        const float sc = sc_cur[j] + ds4o_f16_to_f32(ape_f16[(size_t)pos_mod * width + j]);
        state_kv[(size_t)row * width + j] = kv_cur[j];
        state_score[(size_t)row * width + j] = sc;
        sc_cur[j] = sc;
    }
    if ((pos + 1) % ratio != 0) return 0;

    const float neg_inf = -1.0e30f;                                  /* cuda/compressor.cu:52 */
    for (int j = 0; j < head_dim; j++) {                             /* cuda/compressor.cu:107-164 */
        float mx = neg_inf;
        if (ratio == 4) {
            for (int r = 0; r < 4; r++) {
                const float sp = state_score[(size_t)r * width + j];
                const float sc = state_score[(size_t)(4 + r) * width + head_dim + j];
                if (sp > mx) mx = sp;
                if (sc > mx) mx = sc;
            }
        } else {
            for (int r = 0; r < ratio; r++) {
                const float s = state_score[(size_t)r * width + j];
                if (s > mx) mx = s;
            }
        }
        if (mx <= neg_inf * 0.5f) { emit_out[j] = 0.0f; continue; }
        float denom = 0.0f, sum = 0.0f;
        if (ratio == 4) {
            for (int r = 0; r < 4; r++) {
                const float wp = expf(state_score[(size_t)r * width + j] - mx);
                const float wc = expf(state_score[(size_t)(4 + r) * width + head_dim + j] - mx);
                denom += wp + wc;
                sum += wp * state_kv[(size_t)r * width + j];
                sum += wc * state_kv[(size_t)(4 + r) * width + head_dim + j];
            }
        } else {
            for (int r = 0; r < ratio; r++) {
                const float w = expf(state_score[(size_t)r * width + j] - mx);
                denom += w;
                sum += w * state_kv[(size_t)r * width + j];
            }
        }
        emit_out[j] = denom > 0.0f ? sum / denom : 0.0f;
    }
    {                                                                /* cuda/compressor.cu:173-220 */
        const float scale = rms_scale_of(emit_out, head_dim, eps);
        for (int i = 0; i < head_dim; i++) emit_out[i] = emit_out[i] * scale * norm_w[i];
    }
    rope_tail_inplace(emit_out, head_dim, n_rot, pos + 1 - ratio, rope, 0);
    if (is_attn) ds4o_fp8_kv_round_trip_rows(emit_out, emit_out, 1, head_dim, n_rot);
    if (ratio == 4) {                                                /* cuda/compressor.cu:232-252 */
        for (int i = 0; i < 4 * width; i++) {
            state_kv[i] = state_kv[4 * width + i];
            state_score[i] = state_score[4 * width + i];
        }
    }
    return 1;
}
