// capi.cu — the checked `extern "C"` entry points of libds4b200 for the batched
// kernels: argument validation, launch, launch-error check.  Nothing here
// allocates or synchronises (ds4b200_device_status() excepted).
#include <cerrno>
#include <cstdarg>
#include <cstdio>

#include "../../include/ds4b200.h"
#include "device_utils.cuh"
#include "kernels.cuh"

namespace ds4b200 {
thread_local char t_error[256] = "";

int set_error(int code, const char *fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(t_error, sizeof t_error, fmt, ap);
    va_end(ap);
    return code;
}
}  // namespace ds4b200

namespace {

using ds4b200::t_error;
#define fail ds4b200::set_error

int launched(const char *what) {
    const cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return fail(-EIO, "%s: %s", what, cudaGetErrorString(e));
    return 0;
}

bool a16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
bool a4(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 3u) == 0; }

#define REQUIRE(cond, ...) do { if (!(cond)) return fail(-EINVAL, __VA_ARGS__); } while (0)
#define STREAM(s) static_cast<cudaStream_t>(s)

}  // namespace

extern "C" {

const char *ds4b200_version(void) { return "ds4b200 0.1 (sm_100a)"; }
const char *ds4b200_last_error(void) { return t_error; }

int ds4b200_device_status(void) {
    const int v = ds4b200::read_and_clear_device_status();
    if (v < 0) return fail(-EIO, "device_status: CUDA error");
    return v;
}

int ds4b200_selftest_bounded_wait(int max_polls, int *gave_up, void *stream) {
    REQUIRE(gave_up, "selftest_bounded_wait: null pointer");
    REQUIRE(max_polls >= 1 && max_polls <= (1 << 16), "selftest_bounded_wait: max_polls must be in [1, 65536]");
    ds4b200::selftest_bounded_wait(max_polls, gave_up, STREAM(stream));
    return launched("selftest_bounded_wait");
}

int ds4b200_add_f32(const float *a, const float *b, float *y, int64_t n, void *stream) {
    REQUIRE(n >= 0, "add: n < 0");
    if (n == 0) return 0;
    REQUIRE(a && b && y, "add: null pointer");
    ds4b200::add_f32(a, b, y, n, STREAM(stream));
    return launched("add");
}

int ds4b200_rms_norm_rows_f32(const float *x, const float *residual_in, const float *w,
                              int64_t weight_dim, float *y_f32, uint16_t *y_bf16,
                              float *residual_out, int64_t n_rows, int n, float eps,
                              void *stream) {
    REQUIRE(n_rows >= 0 && n >= 0, "rms_norm_rows: negative size");
    if (n_rows == 0 || n == 0) return 0;
    REQUIRE(n_rows < ((int64_t)1 << 31), "rms_norm_rows: n_rows >= 2^31");
    REQUIRE(x, "rms_norm_rows: x is null");
    REQUIRE(y_f32 || y_bf16, "rms_norm_rows: no output");
    REQUIRE(weight_dim == 0 || weight_dim == n || weight_dim == (int64_t)n * n_rows,
            "rms_norm_rows: weight_dim must be 0, n or n*n_rows");
    REQUIRE(weight_dim == 0 || w, "rms_norm_rows: w is null");
    REQUIRE(!residual_out || residual_in, "rms_norm_rows: residual_out without residual_in");
    ds4b200::rms_norm_rows(x, residual_in, w, weight_dim, y_f32, y_bf16, residual_out, n_rows, n,
                           eps, STREAM(stream));
    return launched("rms_norm_rows");
}

int ds4b200_rms_norm_q8_0_rows_f32(const float *x, const float *residual_in, const float *w,
                                   int64_t weight_dim, float *y_f32, float *residual_out, int8_t *xq,
                                   float *xscale, int64_t n_rows, int n, float eps, void *stream) {
    REQUIRE(n_rows >= 0 && n >= 0, "rms_norm_q8_0_rows: negative size");
    if (n_rows == 0 || n == 0) return 0;
    REQUIRE(n_rows < ((int64_t)1 << 31), "rms_norm_q8_0_rows: n_rows >= 2^31");
    REQUIRE(x && xq && xscale, "rms_norm_q8_0_rows: null pointer");
    REQUIRE(n % 32 == 0 && n <= 8192, "rms_norm_q8_0_rows: n must be a multiple of 32, at most 8192");
    REQUIRE(weight_dim == 0 || weight_dim == n || weight_dim == (int64_t)n * n_rows,
            "rms_norm_q8_0_rows: weight_dim must be 0, n or n*n_rows");
    REQUIRE(weight_dim == 0 || w, "rms_norm_q8_0_rows: w is null");
    REQUIRE(!residual_out || residual_in, "rms_norm_q8_0_rows: residual_out without residual_in");
    REQUIRE(a16(x) && a16(residual_in) && a16(w) && a16(y_f32) && a16(residual_out) && a4(xq),
            "rms_norm_q8_0_rows: f32 buffers need 16-byte and xq 4-byte alignment");
    ds4b200::rms_norm_rows(x, residual_in, w, weight_dim, y_f32, nullptr, residual_out, n_rows, n, eps,
                           STREAM(stream), xq, xscale);
    return launched("rms_norm_q8_0_rows");
}

int ds4b200_rms_norm_q8_K_rows_f32(const float *x, const float *residual_in, const float *w,
                                   int64_t weight_dim, float *y_f32, float *residual_out, int8_t *xq,
                                   float *xscale, int8_t *kq, float *kscale, int16_t *kbsums, int64_t n_rows,
                                   int n, float eps, void *stream) {
    REQUIRE(n_rows >= 0 && n >= 0, "rms_norm_q8_K_rows: negative size");
    if (n_rows == 0 || n == 0) return 0;
    REQUIRE(n_rows < ((int64_t)1 << 31), "rms_norm_q8_K_rows: n_rows >= 2^31");
    REQUIRE(x && kq && kscale && kbsums, "rms_norm_q8_K_rows: null pointer");
    REQUIRE(!xq == !xscale, "rms_norm_q8_K_rows: xq and xscale go together");
    REQUIRE(n % 256 == 0 && n <= 8192, "rms_norm_q8_K_rows: n must be a multiple of 256, at most 8192");
    REQUIRE(weight_dim == 0 || weight_dim == n || weight_dim == (int64_t)n * n_rows,
            "rms_norm_q8_K_rows: weight_dim must be 0, n or n*n_rows");
    REQUIRE(weight_dim == 0 || w, "rms_norm_q8_K_rows: w is null");
    REQUIRE(!residual_out || residual_in, "rms_norm_q8_K_rows: residual_out without residual_in");
    REQUIRE(a16(x) && a16(residual_in) && a16(w) && a16(y_f32) && a16(residual_out) && a4(xq) && a4(kq) &&
                (reinterpret_cast<uintptr_t>(kbsums) & 1u) == 0,
            "rms_norm_q8_K_rows: f32 buffers need 16-byte, xq / kq 4-byte and kbsums 2-byte alignment");
    ds4b200::rms_norm_rows(x, residual_in, w, weight_dim, y_f32, nullptr, residual_out, n_rows, n, eps,
                           STREAM(stream), xq, xscale, kq, kscale, kbsums);
    return launched("rms_norm_q8_K_rows");
}

int ds4b200_quantize_q8_0_rows_f32(const float *x, int8_t *xq, float *xscale, int64_t n_blocks, void *stream) {
    REQUIRE(n_blocks >= 0, "quantize_q8_0_rows: n_blocks < 0");
    if (n_blocks == 0) return 0;
    REQUIRE(x && xq && xscale, "quantize_q8_0_rows: null pointer");
    ds4b200::quantize_q8_0_rows(x, xq, xscale, n_blocks, STREAM(stream));
    return launched("quantize_q8_0_rows");
}

int ds4b200_quantize_q8_K_rows_f32(const float *x, int8_t *xq, float *xscale, int16_t *xbsums,
                                   int64_t n_blocks, void *stream) {
    REQUIRE(n_blocks >= 0, "quantize_q8_K_rows: n_blocks < 0");
    if (n_blocks == 0) return 0;
    REQUIRE(x && xq && xscale && xbsums, "quantize_q8_K_rows: null pointer");
    REQUIRE(a16(x) && a4(xq), "quantize_q8_K_rows: x needs 16-byte and xq 4-byte alignment");
    ds4b200::quantize_q8_K_rows(x, xq, xscale, xbsums, n_blocks, STREAM(stream));
    return launched("quantize_q8_K_rows");
}

int ds4b200_embed_gather_rows(const void *table, int table_dtype, const int32_t *ids,
                              int64_t n_tokens, int n_embd, const float *residual_in,
                              const float *norm_w, float eps, float *out_rows, int n_replicas,
                              float *normed_f32, uint16_t *normed_bf16, void *stream) {
    REQUIRE(n_tokens >= 0 && n_embd >= 0, "embed_gather_rows: negative size");
    if (n_tokens == 0 || n_embd == 0) return 0;
    REQUIRE(n_tokens < ((int64_t)1 << 31), "embed_gather_rows: n_tokens >= 2^31");
    REQUIRE(table && ids, "embed_gather_rows: null table or ids");
    REQUIRE(table_dtype == DS4B200_TABLE_F16 || table_dtype == DS4B200_TABLE_Q8_0,
            "embed_gather_rows: unknown table dtype");
    REQUIRE(table_dtype != DS4B200_TABLE_Q8_0 || n_embd % 32 == 0,
            "embed_gather_rows: Q8_0 rows need n_embd %% 32 == 0");
    REQUIRE(!out_rows || n_replicas >= 1, "embed_gather_rows: n_replicas < 1");
    REQUIRE(out_rows || norm_w, "embed_gather_rows: no output");
    REQUIRE(!norm_w || normed_f32 || normed_bf16, "embed_gather_rows: norm_w without normed output");
    ds4b200::embed_gather_rows(table, table_dtype, ids, 0, n_tokens, n_embd, residual_in, norm_w,
                               eps, out_rows, n_replicas, normed_f32, normed_bf16, STREAM(stream));
    return launched("embed_gather_rows");
}

int ds4b200_rope_rows_f32(const float *x_in, float *x_out, int64_t n_tokens, int n_heads,
                          int head_dim, int n_rot, const int32_t *pos,
                          const ds4b200_rope_params *params, int inverse, int unit_rms,
                          float eps, void *stream) {
    REQUIRE(n_tokens >= 0 && n_heads >= 0 && head_dim >= 0, "rope_rows: negative size");
    if (n_tokens == 0 || n_heads == 0 || head_dim == 0) return 0;
    REQUIRE(n_tokens * n_heads < ((int64_t)1 << 31), "rope_rows: too many rows");
    REQUIRE(x_in && x_out && pos && params, "rope_rows: null pointer");
    REQUIRE(n_rot >= 0 && n_rot <= head_dim && (n_rot & 1) == 0, "rope_rows: n_rot must be even and <= head_dim");
    REQUIRE(params->theta_scale > 0.0f || params->freq_base > 0.0f, "rope_rows: no theta_scale and no freq_base");
    ds4b200::rope_rows(x_in, x_out, n_tokens, n_heads, head_dim, n_rot, pos, 0, *params, inverse,
                       unit_rms, eps, STREAM(stream));
    return launched("rope_rows");
}

int ds4b200_rope_table_rows(const int32_t *pos, const ds4b200_rope_params *params, int64_t n_tokens, int n_rot,
                            float *cs_table, void *stream) {
    REQUIRE(n_tokens >= 0, "rope_table_rows: n_tokens < 0");
    if (n_tokens == 0) return 0;
    REQUIRE(pos && params && cs_table, "rope_table_rows: null pointer");
    REQUIRE(n_rot > 0 && n_rot <= 64 && (n_rot & 1) == 0, "rope_table_rows: n_rot must be even, at most 64");
    REQUIRE(params->theta_scale > 0.0f || params->freq_base > 0.0f, "rope_table_rows: no theta_scale and no freq_base");
    REQUIRE((reinterpret_cast<uintptr_t>(cs_table) & 7u) == 0, "rope_table_rows: cs_table must be 8-byte aligned");
    ds4b200::rope_table_rows(pos, n_tokens, n_rot, *params, cs_table, STREAM(stream));
    return launched("rope_table_rows");
}

int ds4b200_rope_rows_table_f32(const float *x_in, float *x_out, int64_t n_tokens, int n_heads, int head_dim,
                                int n_rot, const float *cs_table, int inverse, int unit_rms, float eps,
                                void *stream) {
    REQUIRE(n_tokens >= 0 && n_heads >= 0 && head_dim >= 0, "rope_rows_table: negative size");
    if (n_tokens == 0 || n_heads == 0 || head_dim == 0) return 0;
    REQUIRE(n_tokens * n_heads < ((int64_t)1 << 31), "rope_rows_table: too many rows");
    REQUIRE(x_in && x_out && cs_table, "rope_rows_table: null pointer");
    REQUIRE(head_dim % 4 == 0 && head_dim <= 1024, "rope_rows_table: head_dim must be a multiple of 4, at most 1024");
    REQUIRE(n_rot > 0 && n_rot <= 64 && n_rot <= head_dim && (n_rot & 3) == 0,
            "rope_rows_table: n_rot must be a multiple of 4, at most 64 and head_dim");
    REQUIRE(ds4b200::aligned16(x_in) && ds4b200::aligned16(x_out) && (reinterpret_cast<uintptr_t>(cs_table) & 7u) == 0,
            "rope_rows_table: alignment (16 bytes for the rows, 8 for cs_table)");
    ds4b200_rope_params unused{};
    unused.theta_scale = 1.0f;
    ds4b200::rope_rows(x_in, x_out, n_tokens, n_heads, head_dim, n_rot, nullptr, 0, unused, inverse, unit_rms, eps,
                       STREAM(stream), nullptr, nullptr, cs_table);
    return launched("rope_rows_table");
}

int ds4b200_rope_q8_0_rows_f32(const float *x_in, float *x_out, int8_t *xq, float *xscale, int64_t n_tokens,
                               int n_heads, int head_dim, int n_rot, const int32_t *pos,
                               const ds4b200_rope_params *params, const float *cs_table, int inverse,
                               int unit_rms, float eps, void *stream) {
    REQUIRE(n_tokens >= 0 && n_heads >= 0 && head_dim >= 0, "rope_q8_0_rows: negative size");
    if (n_tokens == 0 || n_heads == 0 || head_dim == 0) return 0;
    REQUIRE(n_tokens * n_heads < ((int64_t)1 << 31), "rope_q8_0_rows: too many rows");
    REQUIRE(x_in && xq && xscale && ((pos && params) || cs_table), "rope_q8_0_rows: null pointer");
    REQUIRE(!cs_table || (n_rot <= 64 && (reinterpret_cast<uintptr_t>(cs_table) & 7u) == 0),
            "rope_q8_0_rows: a table needs n_rot <= 64 and 8-byte alignment");
    REQUIRE(head_dim % 32 == 0 && head_dim <= 1024, "rope_q8_0_rows: head_dim must be a multiple of 32, at most 1024");
    REQUIRE(n_rot >= 0 && n_rot <= head_dim && (n_rot & 3) == 0, "rope_q8_0_rows: n_rot must be a multiple of 4 and <= head_dim");
    REQUIRE(cs_table || params->theta_scale > 0.0f || params->freq_base > 0.0f, "rope_q8_0_rows: no theta_scale and no freq_base");
    REQUIRE(ds4b200::aligned16(x_in) && (!x_out || ds4b200::aligned16(x_out)) &&
                (reinterpret_cast<uintptr_t>(xq) & 3u) == 0,
            "rope_q8_0_rows: alignment (16 bytes for the f32 rows, 4 for xq)");
    ds4b200_rope_params none{};
    none.theta_scale = 1.0f;
    ds4b200::rope_rows(x_in, x_out, n_tokens, n_heads, head_dim, n_rot, pos, 0, params ? *params : none, inverse,
                       unit_rms, eps, STREAM(stream), xq, xscale, cs_table);
    return launched("rope_q8_0_rows");
}

int ds4b200_fp8_kv_round_trip_rows_f32(const float *kv_in, float *kv_out, int64_t n_rows,
                                       int head_dim, int n_rot, void *stream) {
    REQUIRE(n_rows >= 0 && head_dim >= 0, "fp8_kv_round_trip_rows: negative size");
    if (n_rows == 0 || head_dim == 0) return 0;
    REQUIRE(kv_in && kv_out, "fp8_kv_round_trip_rows: null pointer");
    REQUIRE(n_rot >= 0 && n_rot <= head_dim && (head_dim - n_rot) % 64 == 0,
            "fp8_kv_round_trip_rows: head_dim - n_rot must be a multiple of 64");
    ds4b200::fp8_kv_round_trip_rows(kv_in, kv_out, n_rows, head_dim, n_rot, STREAM(stream));
    return launched("fp8_kv_round_trip_rows");
}

int ds4b200_rope_fp8_store_rows(const float *kv_in, int64_t n_rows, int head_dim, int n_rot,
                                const int32_t *pos, const ds4b200_rope_params *params,
                                const float *norm_w, float eps, int scale_mode,
                                const int32_t *slots, uint8_t *codes, float *scales,
                                float *tail_out, float *rope_out, void *stream) {
    REQUIRE(n_rows >= 0, "rope_fp8_store_rows: n_rows < 0");
    if (n_rows == 0) return 0;
    REQUIRE(kv_in && codes && scales, "rope_fp8_store_rows: null pointer");
    REQUIRE(head_dim > 0 && head_dim <= 1024 && head_dim % 4 == 0,
            "rope_fp8_store_rows: head_dim must be a multiple of 4, at most 1024");
    REQUIRE(n_rot >= 0 && n_rot <= head_dim && n_rot % 4 == 0, "rope_fp8_store_rows: n_rot must be a multiple of 4");
    REQUIRE(scale_mode == DS4B200_FP8_BLOCK64_POW2 || scale_mode == DS4B200_FP8_ROW_AMAX,
            "rope_fp8_store_rows: unknown scale mode");
    REQUIRE(scale_mode != DS4B200_FP8_BLOCK64_POW2 || ((head_dim - n_rot) % 64 == 0 && n_rot % 64 == 0),
            "rope_fp8_store_rows: BLOCK64_POW2 needs head_dim - n_rot and n_rot multiples of 64");
    REQUIRE(!params || pos, "rope_fp8_store_rows: params without pos");
    REQUIRE(!params || params->theta_scale > 0.0f || params->freq_base > 0.0f,
            "rope_fp8_store_rows: no theta_scale and no freq_base");
    REQUIRE(a16(kv_in) && a16(norm_w) && a16(tail_out) && a16(rope_out) && a4(codes),
            "rope_fp8_store_rows: kv_in, norm_w, tail_out, rope_out need 16-byte and codes 4-byte alignment");
    ds4b200::rope_fp8_store_rows(kv_in, n_rows, head_dim, n_rot, pos, params, norm_w, eps,
                                 scale_mode, slots, codes, scales, tail_out, rope_out,
                                 STREAM(stream));
    return launched("rope_fp8_store_rows");
}

int ds4b200_fp8_cache_load_rows(const uint8_t *codes, const float *scales, const float *tail,
                                const int32_t *slots, int64_t n_rows, int head_dim, int n_rot,
                                int scale_mode, int f16_round, float *out, void *stream) {
    REQUIRE(n_rows >= 0, "fp8_cache_load_rows: n_rows < 0");
    if (n_rows == 0) return 0;
    REQUIRE(codes && scales && out, "fp8_cache_load_rows: null pointer");
    REQUIRE(head_dim > 0 && head_dim <= 1024 && head_dim % 4 == 0 && n_rot >= 0 && n_rot <= head_dim && n_rot % 4 == 0,
            "fp8_cache_load_rows: head_dim and n_rot must be multiples of 4, head_dim at most 1024");
    REQUIRE(scale_mode == DS4B200_FP8_BLOCK64_POW2 || scale_mode == DS4B200_FP8_ROW_AMAX,
            "fp8_cache_load_rows: unknown scale mode");
    REQUIRE(scale_mode != DS4B200_FP8_BLOCK64_POW2 || ((head_dim - n_rot) % 64 == 0 && (tail || n_rot == 0)),
            "fp8_cache_load_rows: BLOCK64_POW2 needs a prefix that is a multiple of 64 and the f32 tail");
    REQUIRE(a4(codes) && a16(tail) && a16(out), "fp8_cache_load_rows: codes need 4-byte, tail and out 16-byte alignment");
    ds4b200::fp8_cache_load_rows(codes, scales, tail, slots, n_rows, head_dim, n_rot, scale_mode, f16_round, out,
                                 STREAM(stream));
    return launched("fp8_cache_load_rows");
}

int ds4b200_kv_rows_to_raw_f32(const float *kv_in, int64_t n_rows, int head_dim, int n_rot, const int32_t *pos,
                               const ds4b200_rope_params *params, const float *norm_w, float eps,
                               const int32_t *slots, float *raw_out, void *stream) {
    REQUIRE(n_rows >= 0, "kv_rows_to_raw: n_rows < 0");
    if (n_rows == 0) return 0;
    REQUIRE(kv_in && raw_out, "kv_rows_to_raw: null pointer");
    REQUIRE(head_dim > 0 && head_dim <= 1024 && head_dim % 64 == 0 && n_rot >= 0 && n_rot <= head_dim && n_rot % 64 == 0,
            "kv_rows_to_raw: head_dim and n_rot must be multiples of 64, head_dim at most 1024");
    REQUIRE(!params || pos, "kv_rows_to_raw: params without pos");
    REQUIRE(!params || params->theta_scale > 0.0f || params->freq_base > 0.0f,
            "kv_rows_to_raw: no theta_scale and no freq_base");
    REQUIRE(a16(kv_in) && a16(norm_w) && a16(raw_out), "kv_rows_to_raw: buffers need 16-byte alignment");
    ds4b200::rope_fp8_store_rows(kv_in, n_rows, head_dim, n_rot, pos, params, norm_w, eps, DS4B200_FP8_BLOCK64_POW2,
                                 slots, nullptr, nullptr, nullptr, nullptr, STREAM(stream), raw_out);
    return launched("kv_rows_to_raw");
}

// The two KV-row entry points with the chunk's angle table in place of pos + params: cs_table holds one
// row of n_rot/2 (cos, sin) pairs per input row.
static ds4b200_rope_params table_only_params() {
    ds4b200_rope_params p{};
    p.freq_base = 1.0f;            // marks "rotate"; the angles come from the table
    return p;
}

int ds4b200_rope_fp8_store_rows_table(const float *kv_in, int64_t n_rows, int head_dim, int n_rot,
                                      const float *cs_table, const float *norm_w, float eps, int scale_mode,
                                      const int32_t *slots, uint8_t *codes, float *scales, float *tail_out,
                                      float *rope_out, void *stream) {
    REQUIRE(n_rows >= 0, "rope_fp8_store_rows_table: n_rows < 0");
    if (n_rows == 0) return 0;
    REQUIRE(kv_in && codes && scales && cs_table, "rope_fp8_store_rows_table: null pointer");
    REQUIRE(head_dim > 0 && head_dim <= 1024 && head_dim % 4 == 0,
            "rope_fp8_store_rows_table: head_dim must be a multiple of 4, at most 1024");
    REQUIRE(n_rot > 0 && n_rot <= 64 && n_rot <= head_dim && n_rot % 4 == 0,
            "rope_fp8_store_rows_table: n_rot must be a multiple of 4, at most 64");
    REQUIRE(scale_mode == DS4B200_FP8_BLOCK64_POW2 || scale_mode == DS4B200_FP8_ROW_AMAX,
            "rope_fp8_store_rows_table: unknown scale mode");
    REQUIRE(scale_mode != DS4B200_FP8_BLOCK64_POW2 || ((head_dim - n_rot) % 64 == 0 && n_rot % 64 == 0),
            "rope_fp8_store_rows_table: BLOCK64_POW2 needs head_dim - n_rot and n_rot multiples of 64");
    REQUIRE(a16(kv_in) && a16(norm_w) && a16(tail_out) && a16(rope_out) && a4(codes) &&
                (reinterpret_cast<uintptr_t>(cs_table) & 7u) == 0,
            "rope_fp8_store_rows_table: kv_in, norm_w, tail_out, rope_out need 16-byte, cs_table 8-byte, codes 4-byte alignment");
    const ds4b200_rope_params p = table_only_params();
    ds4b200::rope_fp8_store_rows(kv_in, n_rows, head_dim, n_rot, nullptr, &p, norm_w, eps, scale_mode, slots, codes,
                                 scales, tail_out, rope_out, STREAM(stream), nullptr, cs_table);
    return launched("rope_fp8_store_rows_table");
}

int ds4b200_kv_rows_to_raw_table_f32(const float *kv_in, int64_t n_rows, int head_dim, int n_rot,
                                     const float *cs_table, const float *norm_w, float eps, const int32_t *slots,
                                     float *raw_out, void *stream) {
    REQUIRE(n_rows >= 0, "kv_rows_to_raw_table: n_rows < 0");
    if (n_rows == 0) return 0;
    REQUIRE(kv_in && raw_out && cs_table, "kv_rows_to_raw_table: null pointer");
    REQUIRE(head_dim > 0 && head_dim <= 1024 && head_dim % 64 == 0 && n_rot == 64 && n_rot <= head_dim,
            "kv_rows_to_raw_table: head_dim must be a multiple of 64, at most 1024, and n_rot 64");
    REQUIRE(a16(kv_in) && a16(norm_w) && a16(raw_out) && (reinterpret_cast<uintptr_t>(cs_table) & 7u) == 0,
            "kv_rows_to_raw_table: buffers need 16-byte alignment (cs_table 8)");
    const ds4b200_rope_params p = table_only_params();
    ds4b200::rope_fp8_store_rows(kv_in, n_rows, head_dim, n_rot, nullptr, &p, norm_w, eps, DS4B200_FP8_BLOCK64_POW2,
                                 slots, nullptr, nullptr, nullptr, nullptr, STREAM(stream), raw_out, cs_table);
    return launched("kv_rows_to_raw_table");
}

int ds4b200_kv_rows_to_raw_table_out_f32(const float *kv_in, int64_t n_rows, int head_dim, int n_rot,
                                         const int32_t *pos, const ds4b200_rope_params *params, const float *norm_w,
                                         float eps, const int32_t *slots, float *raw_out, float *cs_out, void *stream) {
    REQUIRE(n_rows >= 0, "kv_rows_to_raw_table_out: n_rows < 0");
    if (n_rows == 0) return 0;
    REQUIRE(kv_in && raw_out && pos && params && cs_out, "kv_rows_to_raw_table_out: null pointer");
    REQUIRE(head_dim > 0 && head_dim <= 1024 && head_dim % 64 == 0 && n_rot == 64 && n_rot <= head_dim,
            "kv_rows_to_raw_table_out: head_dim must be a multiple of 64, at most 1024, and n_rot 64");
    REQUIRE(params->theta_scale > 0.0f || params->freq_base > 0.0f, "kv_rows_to_raw_table_out: no theta_scale and no freq_base");
    REQUIRE(a16(kv_in) && a16(norm_w) && a16(raw_out) && (reinterpret_cast<uintptr_t>(cs_out) & 7u) == 0,
            "kv_rows_to_raw_table_out: buffers need 16-byte alignment (cs_out 8)");
    ds4b200::rope_fp8_store_rows(kv_in, n_rows, head_dim, n_rot, pos, params, norm_w, eps, DS4B200_FP8_BLOCK64_POW2,
                                 slots, nullptr, nullptr, nullptr, nullptr, STREAM(stream), raw_out, nullptr, cs_out);
    return launched("kv_rows_to_raw_table_out");
}

int ds4b200_swa_window_push_rows_f32(float *raw_kv, int cap, int n_raw, const float *new_rows, int n_new,
                                     int head_dim, int *n_raw_after, void *stream) {
    REQUIRE(cap > 0 && n_raw >= 0 && n_raw <= cap && n_new >= 0, "swa_window_push_rows: bad window state");
    REQUIRE(head_dim > 0 && head_dim % 4 == 0, "swa_window_push_rows: head_dim must be a multiple of 4");
    const int total = n_raw + n_new;
    if (n_raw_after) *n_raw_after = total < cap ? total : cap;
    if (n_new == 0) return 0;
    REQUIRE(raw_kv && new_rows, "swa_window_push_rows: null pointer");
    REQUIRE(a16(raw_kv) && a16(new_rows), "swa_window_push_rows: buffers need 16-byte alignment");
    ds4b200::swa_window_push_rows(raw_kv, cap, n_raw, new_rows, n_new, head_dim, STREAM(stream));
    return launched("swa_window_push_rows");
}

int ds4b200_swiglu_rows_f32(const float *gate, const float *up, const float *weights, float *out,
                            int64_t n_tokens, int k, int n, int mode, float clamp, int combine,
                            int fast_exp, void *stream) {
    REQUIRE(n_tokens >= 0 && k >= 0 && n >= 0, "swiglu_rows: negative size");
    if (n_tokens == 0 || k == 0 || n == 0) return 0;
    REQUIRE(gate && up && out, "swiglu_rows: null pointer");
    REQUIRE(mode >= DS4B200_GLU_PLAIN && mode <= DS4B200_GLU_CLAMP_SYM, "swiglu_rows: unknown mode");
    ds4b200::swiglu_rows(gate, up, weights, out, n_tokens, k, n, mode, clamp, combine, fast_exp,
                         STREAM(stream));
    return launched("swiglu_rows");
}

int ds4b200_hc_pre_rows_f32(const float *residual_hc, const uint16_t *hc_fn,
                            const float *hc_scale, const float *hc_base, float *post, float *comb,
                            float *out, int64_t n_tokens, int n_embd, int sinkhorn_iters,
                            float eps, void *stream) {
    REQUIRE(n_tokens >= 0, "hc_pre_rows: n_tokens < 0");
    if (n_tokens == 0) return 0;
    REQUIRE(n_tokens < ((int64_t)1 << 31), "hc_pre_rows: n_tokens >= 2^31");
    REQUIRE(residual_hc && hc_fn && hc_scale && hc_base && post && comb && out,
            "hc_pre_rows: null pointer");
    REQUIRE(n_embd > 0 && n_embd % 4 == 0 && n_embd <= 8192,
            "hc_pre_rows: n_embd must be a multiple of 4, at most 8192");
    REQUIRE(sinkhorn_iters >= 1, "hc_pre_rows: sinkhorn_iters < 1");
    ds4b200::hc_pre_rows(residual_hc, hc_fn, hc_scale, hc_base, post, comb, out, n_tokens, n_embd,
                         sinkhorn_iters, eps, STREAM(stream));
    return launched("hc_pre_rows");
}

int ds4b200_hc_pre_norm_rows_f32(const float *residual_hc, const uint16_t *hc_fn, const float *hc_scale,
                                 const float *hc_base, const float *norm_w, float *post, float *comb, float *out,
                                 float *normed, int8_t *xq, float *xscale, int64_t n_tokens, int n_embd,
                                 int sinkhorn_iters, float eps, void *stream) {
    REQUIRE(n_tokens >= 0, "hc_pre_norm_rows: n_tokens < 0");
    if (n_tokens == 0) return 0;
    REQUIRE(n_tokens < ((int64_t)1 << 31), "hc_pre_norm_rows: n_tokens >= 2^31");
    REQUIRE(residual_hc && hc_fn && hc_scale && hc_base && norm_w && post && comb && out,
            "hc_pre_norm_rows: null pointer");
    REQUIRE(normed || xq, "hc_pre_norm_rows: neither normed nor xq given");
    REQUIRE(!xq == !xscale, "hc_pre_norm_rows: xq and xscale go together");
    REQUIRE(n_embd > 0 && n_embd % 32 == 0 && n_embd <= 8192,
            "hc_pre_norm_rows: n_embd must be a multiple of 32, at most 8192");
    REQUIRE(sinkhorn_iters >= 1, "hc_pre_norm_rows: sinkhorn_iters < 1");
    ds4b200::hc_pre_norm_rows(residual_hc, hc_fn, hc_scale, hc_base, norm_w, post, comb, out, normed, xq, xscale,
                              n_tokens, n_embd, sinkhorn_iters, eps, STREAM(stream));
    return launched("hc_pre_norm_rows");
}

int ds4b200_output_hc_head_rows_f32(const float *residual_hc, const uint16_t *output_hc_fn,
                                    const float *output_hc_scale, const float *output_hc_base,
                                    const float *norm_w, float *out, float *normed, int64_t n_tokens,
                                    int n_embd, float eps, void *stream) {
    REQUIRE(n_tokens >= 0, "output_hc_head_rows: n_tokens < 0");
    if (n_tokens == 0) return 0;
    REQUIRE(n_tokens < ((int64_t)1 << 31), "output_hc_head_rows: n_tokens >= 2^31");
    REQUIRE(residual_hc && output_hc_fn && output_hc_scale && output_hc_base, "output_hc_head_rows: null pointer");
    REQUIRE(out || normed, "output_hc_head_rows: no output");
    REQUIRE(!normed == !norm_w, "output_hc_head_rows: normed and norm_w go together");
    REQUIRE(n_embd > 0 && n_embd % 4 == 0 && n_embd <= 8192,
            "output_hc_head_rows: n_embd must be a multiple of 4, at most 8192");
    ds4b200::hc_head_rows(residual_hc, output_hc_fn, output_hc_scale, output_hc_base, norm_w, out, normed,
                          n_tokens, n_embd, eps, STREAM(stream));
    return launched("output_hc_head_rows");
}

int ds4b200_hc_post_rows_f32(const float *block_out, const float *block_out2,
                             const float *residual_hc, const float *post, const float *comb,
                             float *out_hc, int64_t n_tokens, int n_embd, void *stream) {
    REQUIRE(n_tokens >= 0, "hc_post_rows: n_tokens < 0");
    if (n_tokens == 0) return 0;
    REQUIRE(n_tokens < ((int64_t)1 << 31), "hc_post_rows: n_tokens >= 2^31");
    REQUIRE(residual_hc && comb && out_hc, "hc_post_rows: null pointer");
    REQUIRE(!block_out || post, "hc_post_rows: block_out without post");
    REQUIRE(!block_out2 || block_out, "hc_post_rows: block_out2 without block_out");
    REQUIRE(n_embd > 0 && n_embd % 4 == 0 && n_embd <= 8192,
            "hc_post_rows: n_embd must be a multiple of 4, at most 8192");
    ds4b200::hc_post_rows(block_out, block_out2, residual_hc, post, comb, nullptr, nullptr, out_hc,
                          n_tokens, n_embd, 0, 0.0f, STREAM(stream));
    return launched("hc_post_rows");
}

int ds4b200_hc_post_pre_rows_f32(const float *block_out, const float *block_out2, const float *residual_hc,
                                 const float *post_in, const float *comb_in, const uint16_t *hc_fn,
                                 const float *hc_scale, const float *hc_base, float *out_hc, float *post, float *comb,
                                 float *out, int64_t n_tokens, int n_embd, int sinkhorn_iters, float eps,
                                 void *stream) {
    REQUIRE(n_tokens >= 0, "hc_post_pre_rows: n_tokens < 0");
    if (n_tokens == 0) return 0;
    REQUIRE(n_tokens < ((int64_t)1 << 31), "hc_post_pre_rows: n_tokens >= 2^31");
    REQUIRE(residual_hc && comb_in && out_hc && hc_fn && hc_scale && hc_base && post && comb && out,
            "hc_post_pre_rows: null pointer");
    REQUIRE(!block_out || post_in, "hc_post_pre_rows: block_out without post_in");
    REQUIRE(!block_out2 || block_out, "hc_post_pre_rows: block_out2 without block_out");
    REQUIRE(n_embd > 0 && n_embd % 4 == 0 && n_embd <= 8192,
            "hc_post_pre_rows: n_embd must be a multiple of 4, at most 8192");
    REQUIRE(sinkhorn_iters >= 1, "hc_post_pre_rows: sinkhorn_iters < 1");
    REQUIRE(out_hc != residual_hc && out != block_out, "hc_post_pre_rows: outputs alias inputs of the first step");
    // two launches: the post step's rows go through HBM once more.  A one-kernel form would put the post
    // arithmetic (80 multiply-adds per 16 bytes) into the operand-writing warps of the pre kernel, which are
    // its longest stage already, and that kernel does not wait for memory.
    ds4b200::hc_post_rows(block_out, block_out2, residual_hc, post_in, comb_in, nullptr, nullptr, out_hc, n_tokens,
                          n_embd, 0, 0.0f, STREAM(stream));
    ds4b200::hc_pre_rows(out_hc, hc_fn, hc_scale, hc_base, post, comb, out, n_tokens, n_embd, sinkhorn_iters, eps,
                         STREAM(stream));
    return launched("hc_post_pre_rows");
}

int ds4b200_hc_sinkhorn_mix_rows_f32(const float *logits, const float *residual_hc, float *out_hc,
                                     float *comb_out, int64_t n_tokens, int n_embd,
                                     int sinkhorn_iters, float eps, void *stream) {
    REQUIRE(n_tokens >= 0, "hc_sinkhorn_mix_rows: n_tokens < 0");
    if (n_tokens == 0) return 0;
    REQUIRE(n_tokens < ((int64_t)1 << 31), "hc_sinkhorn_mix_rows: n_tokens >= 2^31");
    REQUIRE(logits && residual_hc && out_hc, "hc_sinkhorn_mix_rows: null pointer");
    REQUIRE(n_embd > 0 && n_embd % 4 == 0 && n_embd <= 8192,
            "hc_sinkhorn_mix_rows: n_embd must be a multiple of 4, at most 8192");
    REQUIRE(sinkhorn_iters >= 1, "hc_sinkhorn_mix_rows: sinkhorn_iters < 1");
    if (comb_out) {
        // two launches: all tokens' 4x4 matrices side by side, then pure streaming
        ds4b200::hc_sinkhorn_rows(logits, comb_out, n_tokens, sinkhorn_iters, eps, STREAM(stream));
        ds4b200::hc_post_rows(nullptr, nullptr, residual_hc, nullptr, comb_out, nullptr, nullptr,
                              out_hc, n_tokens, n_embd, 0, 0.0f, STREAM(stream));
    } else {
        ds4b200::hc_post_rows(nullptr, nullptr, residual_hc, nullptr, nullptr, logits, nullptr, out_hc,
                              n_tokens, n_embd, sinkhorn_iters, eps, STREAM(stream));
    }
    return launched("hc_sinkhorn_mix_rows");
}

int ds4b200_hc_sinkhorn_rows_f32(const float *logits, float *comb, int64_t n_tokens,
                                 int sinkhorn_iters, float eps, void *stream) {
    REQUIRE(n_tokens >= 0, "hc_sinkhorn_rows: n_tokens < 0");
    if (n_tokens == 0) return 0;
    REQUIRE(logits && comb, "hc_sinkhorn_rows: null pointer");
    REQUIRE(sinkhorn_iters >= 1, "hc_sinkhorn_rows: sinkhorn_iters < 1");
    ds4b200::hc_sinkhorn_rows(logits, comb, n_tokens, sinkhorn_iters, eps, STREAM(stream));
    return launched("hc_sinkhorn_rows");
}

int ds4b200_e4m3_encode_f32(const float *x, uint8_t *codes, int64_t n, void *stream) {
    REQUIRE(n >= 0, "e4m3_encode: n < 0");
    if (n == 0) return 0;
    REQUIRE(x && codes, "e4m3_encode: null pointer");
    ds4b200::e4m3_encode(x, codes, n, STREAM(stream));
    return launched("e4m3_encode");
}

int ds4b200_e4m3_decode_f32(const uint8_t *codes, float *x, int64_t n, void *stream) {
    REQUIRE(n >= 0, "e4m3_decode: n < 0");
    if (n == 0) return 0;
    REQUIRE(x && codes, "e4m3_decode: null pointer");
    ds4b200::e4m3_decode(codes, x, n, STREAM(stream));
    return launched("e4m3_decode");
}

int ds4b200_swiglu_q8_0_rows_f32(const float *gate, const float *up, const float *weights, int8_t *xq,
                                 float *xscale, float *mid_f32, int64_t n_tokens, int k, int n, int mode,
                                 float clamp, int fast_exp, void *stream) {
    REQUIRE(n_tokens >= 0 && k >= 1 && n >= 32 && n % 32 == 0, "swiglu_q8_0_rows: n must be a multiple of 32, got %d", n);
    if (n_tokens == 0) return 0;
    REQUIRE(gate && up && xq && xscale, "swiglu_q8_0_rows: null pointer");
    REQUIRE(mode >= DS4B200_GLU_PLAIN && mode <= DS4B200_GLU_CLAMP_SYM, "swiglu_q8_0_rows: unknown mode %d", mode);
    REQUIRE(a16(gate) && a16(up) && a16(mid_f32) && a4(xq), "swiglu_q8_0_rows: pointers must be 16-byte aligned (xq: 4)");
    ds4b200::swiglu_q8_0_rows(gate, up, weights, xq, xscale, mid_f32, n_tokens * k, n, mode, clamp, fast_exp,
                              STREAM(stream));
    return launched("swiglu_q8_0_rows");
}

int ds4b200_swiglu_q8_K_rows_f32(const float *gate, const float *up, const float *weights, int8_t *xq,
                                 float *xscale, int16_t *xbsums, float *mid_f32, int64_t n_tokens, int k,
                                 int n, int mode, float clamp, int fast_exp, void *stream) {
    REQUIRE(gate && up && xq && xscale && xbsums, "swiglu_q8_K_rows: null pointer");
    REQUIRE(n_tokens >= 0 && k >= 1 && n >= 256 && n % 256 == 0, "swiglu_q8_K_rows: n must be a multiple of 256, got %d", n);
    REQUIRE(mode >= DS4B200_GLU_PLAIN && mode <= DS4B200_GLU_CLAMP_SYM, "swiglu_q8_K_rows: unknown mode %d", mode);
    REQUIRE(a16(gate) && a16(up) && a16(mid_f32) && a4(xq), "swiglu_q8_K_rows: pointers must be 16-byte aligned (xq: 4)");
    ds4b200::swiglu_q8_K_rows(gate, up, weights, xq, xscale, xbsums, mid_f32, n_tokens * k, n, mode, clamp, fast_exp,
                              STREAM(stream));
    return launched("swiglu_q8_K_rows");
}

int ds4b200_compressor_step_f32(int is_attn, const float *kv_cur, float *sc_cur, const uint16_t *ape_f16,
                                const float *norm_w, int head_dim, int compress_ratio, int pos, int il,
                                float *state_kv, float *state_score, float *emit_out,
                                int *emitted_host, void *stream) {
    REQUIRE(kv_cur && sc_cur && ape_f16 && norm_w && state_kv && state_score && emit_out,
            "compressor_step: null pointer");
    REQUIRE(head_dim >= 128 && head_dim <= 1024 && head_dim % 64 == 0,
            "compressor_step: head_dim must be a multiple of 64 in [128, 1024], got %d", head_dim);
    REQUIRE(compress_ratio == 4 || (compress_ratio >= 1 && compress_ratio <= 4096),
            "compressor_step: compress_ratio out of range");
    REQUIRE(pos >= 0, "compressor_step: negative position");
    ds4b200_rope_params rope;
    ds4b200_rope_params_for_layer(il, 64, &rope);
    const bool emitted = ds4b200::compressor_step(is_attn, kv_cur, sc_cur, ape_f16, norm_w, head_dim, compress_ratio,
                                                  pos, rope, 64, 1.0e-6f, state_kv, state_score, emit_out,
                                                  STREAM(stream));
    if (emitted_host) *emitted_host = emitted ? 1 : 0;
    return launched("compressor_step");
}

int ds4b200_compressor_chunk_f32(int is_attn, const float *kv_cur, const float *sc_cur, const uint16_t *ape_f16,
                                 const float *norm_w, int head_dim, int compress_ratio, int pos0,
                                 int64_t n_tokens, int il, float *state_kv, float *state_score,
                                 float *emit_out, void *stream) {
    REQUIRE(kv_cur && sc_cur && ape_f16 && norm_w && state_kv && state_score && emit_out,
            "compressor_chunk: null pointer");
    REQUIRE(head_dim >= 128 && head_dim <= 1024 && head_dim % 64 == 0,
            "compressor_chunk: head_dim must be a multiple of 64 in [128, 1024], got %d", head_dim);
    REQUIRE(compress_ratio >= 1 && compress_ratio <= 4096, "compressor_chunk: compress_ratio out of range");
    REQUIRE(pos0 >= 0 && n_tokens >= 0, "compressor_chunk: negative position or count");
    REQUIRE(pos0 % compress_ratio == 0 && n_tokens % compress_ratio == 0,
            "compressor_chunk: the chunk must start and end on window boundaries (use compressor_step for the rest)");
    if (n_tokens == 0) return 0;
    ds4b200_rope_params rope;
    ds4b200_rope_params_for_layer(il, 64, &rope);
    ds4b200::compressor_chunk(is_attn, kv_cur, sc_cur, ape_f16, norm_w, head_dim, compress_ratio, pos0, n_tokens, rope,
                              64, 1.0e-6f, state_kv, state_score, emit_out, STREAM(stream));
    return launched("compressor_chunk");
}

int ds4b200_div_selfcheck(uint64_t first, uint64_t count, unsigned long long *mismatches, void *stream) {
    REQUIRE(mismatches, "div_selfcheck: null pointer");
    ds4b200::div_selfcheck(first, count, mismatches, STREAM(stream));
    return launched("div_selfcheck");
}

int ds4b200_e4m3_selfcheck(uint32_t first_bits, uint64_t count, unsigned long long *mismatches,
                           void *stream) {
    REQUIRE(mismatches, "e4m3_selfcheck: null pointer");
    REQUIRE(count <= ((uint64_t)1 << 32), "e4m3_selfcheck: count > 2^32");
    ds4b200::e4m3_selfcheck(first_bits, count, mismatches, STREAM(stream));
    return launched("e4m3_selfcheck");
}

}  // extern "C"
