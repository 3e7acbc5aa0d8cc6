// rope_fp8.cu — partial (tail) YaRN RoPE over head rows, the E4M3FN KV
// quantiser, and the two fused: RMSNorm -> RoPE -> FP8 bytes + scales written
// straight into the KV cache.
//
// Arithmetic follows the reference:
//   RoPE      cuda/rope.cu:136-201 (inverse: cuda/attn_out.cu:54-107): pair k of
//             the tail uses theta_extrap = (float)pos * theta_scale^k built by k
//             successive f32 multiplies, the YaRN ramp mix, accurate cosf/sinf.
//   FP8       cuda/fp8_kv.cu:144-195: per 64 elements of the non-rotated prefix,
//             scale = exp2f(ceilf(log2f(max(amax,1e-4)/448))), nearest E4M3FN
//             value with ties to the even index, saturating at 448.
//
// Data movement: one warp owns one row of up to 1024 floats in registers
// (lane l holds float4 number l, l+32, ...), so loads and stores are 128-bit and
// coalesced, reductions are shuffles only, and the fused kernel reads 4 bytes
// and writes ~1 byte per element instead of four f32 round trips.
#include "device_utils.cuh"
#include "kernels.cuh"
#include "rope_device.cuh"

namespace ds4b200 {
namespace {

constexpr int kRowsPerCta = 8;      // warps per CTA in the warp-per-row kernels

// Rotate the float4 that starts at tail element `e_tail` (a multiple of 4).
__device__ __forceinline__ void rope_float4(float4 &v, int e_tail, float posf, float ts,
                                            const RopeDev &p, bool inverse) {
    const int k0 = e_tail >> 1;
    float te = posf;
    for (int k = 0; k < k0; ++k) te *= ts;
    float c, s;
    rope_cs(p, k0, te, inverse, c, s);
    rotate(v.x, v.y, c, s);
    te *= ts;
    rope_cs(p, k0 + 1, te, inverse, c, s);
    rotate(v.z, v.w, c, s);
}

// Rotate the tail of a row held by one warp (lane l holds float4 number l + 32 j).  With at
// most 32 pairs, lane k evaluates the angle of pair k (the same k multiplies and the same
// cosf / sinf as rope_float4) and the lanes that hold the tail fetch the two (cos, sin) they
// need by shuffle, instead of 16 lanes doing two pairs each; more pairs fall back to
// rope_float4 per lane.  Every lane of the warp must call this.
// cs_row (optional, only with n_rot <= 64): the token's (cos, sin) multipliers as rope_table_kernel
// wrote them, pair k at cs_row[k]; the same bits as evaluating them here, at the cost of one load.
// n_rot <= 64: lane k holds (c, sn) of pair k; the lanes that hold the tail fetch the two pairs they need by shuffle.
template <int VPT>
__device__ __forceinline__ void rope_tail_apply(float4 (&v)[VPT], int lane, int n4, int n_nope, float c, float sn) {
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
        if ((32 * j + 31) * 4 < n_nope) continue;          // no lane of this j is in the tail
        const int i = lane + 32 * j;
        const bool tail = i < n4 && 4 * i >= n_nope;
        const int k0 = tail ? (4 * i - n_nope) >> 1 : 0;
        const float c0 = __shfl_sync(0xffffffffu, c, k0), s0 = __shfl_sync(0xffffffffu, sn, k0);
        const float c1 = __shfl_sync(0xffffffffu, c, k0 + 1), s1 = __shfl_sync(0xffffffffu, sn, k0 + 1);
        if (tail) {
            rotate(v[j].x, v[j].y, c0, s0);
            rotate(v[j].z, v[j].w, c1, s1);
        }
    }
}

// cs_save (optional, forward rotation only): the lane's (cos, sin) is also written there, which makes this
// row's evaluation the chunk's angle table entry (the bits rope_table_kernel would write).
template <int VPT>
__device__ __forceinline__ void rope_tail_warp(float4 (&v)[VPT], int lane, int n4, int n_nope, int n_rot,
                                               float posf, const RopeDev &p, bool inverse,
                                               const float2 *cs_row = nullptr, float2 *cs_save = nullptr) {
    if (n_rot <= 64) {
        float c = 1.0f, sn = 0.0f;
        if (2 * lane < n_rot) {
            if (cs_row) {
                const float2 cs = __ldg(cs_row + lane);
                c = cs.x;
                sn = inverse ? -cs.y : cs.y;
            } else {
                const float ts = rope_theta_scale(p, n_rot);
                float te = posf;
                for (int k = 0; k < lane; ++k) te *= ts;
                rope_cs(p, lane, te, inverse, c, sn);
                if (cs_save) cs_save[lane] = make_float2(c, sn);
            }
        }
        rope_tail_apply<VPT>(v, lane, n4, n_nope, c, sn);
    } else {
        const float ts = rope_theta_scale(p, n_rot);
#pragma unroll
        for (int j = 0; j < VPT; ++j) {
            const int i = lane + 32 * j;
            if (i < n4 && 4 * i >= n_nope) rope_float4(v[j], 4 * i - n_nope, posf, ts, p, inverse);
        }
    }
}

// The (cos, sin) multipliers of every tail pair of every token, computed once per chunk: they depend on the
// position and the layer's parameter set only, yet each of a layer's 64 + 64 + 1 head rows per token needs
// them (cuda/rope.cu:165-200 evaluates them per head row).  One thread per (token, pair); the same
// multiply chain and the same cosf / sinf as rope_tail_warp, so the rotated rows keep their bits.
__global__ void rope_table_kernel(const int32_t *pos, int64_t n_tokens, int n_pairs, int n_rot, RopeDev p, float2 *cs) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n_tokens * n_pairs) return;
    const int64_t t = i / n_pairs;
    const int k = (int)(i - t * n_pairs);
    const float ts = rope_theta_scale(p, n_rot);
    float te = (float)pos[t];
    for (int q = 0; q < k; ++q) te *= ts;
    float c, s;
    rope_cs(p, k, te, false, c, s);
    cs[i] = make_float2(c, s);
}

// ------------------------------- RoPE rows ---------------------------------
// Q8: the rotated row also (or only, x_out == nullptr) leaves as Q8_0 blocks, the activation form of
// the matvec that consumes it (cuda/attn_out.cu:119-145 for the rows behind the inverse RoPE): 32
// elements = 8 consecutive lanes of one float4 slot, amax by shuffles, d = amax / 127, RNE, clamp.
template <int VPT, bool Q8>
__global__ void __launch_bounds__(kRowsPerCta * 32)
rope_rows_kernel(const float *x_in, float *x_out, int64_t n_rows, int n_heads, int head_dim,
                 int n_rot, const int32_t *pos, int single_pos, RopeDev p, int inverse,
                 int unit_rms, float eps, int8_t *xq, float *xscale, const float2 *cs_table) {
    const int lane = threadIdx.x & 31;
    const int64_t row = (int64_t)blockIdx.x * kRowsPerCta + (threadIdx.x >> 5);
    if (row >= n_rows) return;
    const int n4 = head_dim >> 2, n_nope = head_dim - n_rot;
    const float *xr = x_in + row * head_dim;
    float *yr = x_out + row * head_dim;
    float4 v[VPT];
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
        const int i = lane + 32 * j;
        v[j] = (i < n4) ? ld_stream4(xr + 4 * i) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    if (unit_rms) {
        float ss = 0.0f;
#pragma unroll
        for (int j = 0; j < VPT; ++j) ss += dot4(v[j]);
        const float scale = rms_scale(warp_sum(ss), (float)head_dim, eps);
#pragma unroll
        for (int j = 0; j < VPT; ++j) { v[j].x *= scale; v[j].y *= scale; v[j].z *= scale; v[j].w *= scale; }
    }
    // (fetching the table entry ahead of the row loads measured slower here: 127 against 117 us for the Q8_0 form)
    const float posf = cs_table ? 0.0f : (float)(pos ? pos[row / n_heads] : single_pos);
    rope_tail_warp<VPT>(v, lane, n4, n_nope, n_rot, posf, p, inverse != 0,
                        cs_table ? cs_table + (row / n_heads) * (n_rot >> 1) : nullptr);
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
        const int i = lane + 32 * j;
        const bool live = i < n4;
        if (live && (!Q8 || x_out)) st_stream4(yr + 4 * i, v[j]);
        if (Q8) {
            // head_dim % 32 == 0, so a group of 8 lanes is live or dead as a whole
            float amax = live ? amax4(v[j]) : 0.0f;
#pragma unroll
            for (int off = 4; off > 0; off >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
            float d, id;
            q8_0_block_scale(amax, d, id);
            if (live) {
                reinterpret_cast<uint32_t *>(xq + row * head_dim)[i] = q8_pack4_sat(v[j].x * id, v[j].y * id, v[j].z * id, v[j].w * id);
                if ((i & 7) == 0) xscale[row * (head_dim >> 5) + (i >> 3)] = d;
            }
        }
    }
}

// Any head_dim / n_rot (even) / alignment: one CTA per row, scalar accesses.
__global__ void rope_rows_scalar_kernel(const float *x_in, float *x_out, int n_heads,
                                        int head_dim, int n_rot, const int32_t *pos,
                                        int single_pos, RopeDev p, int inverse, int unit_rms,
                                        float eps) {
    __shared__ float red[33];
    const int64_t row = blockIdx.x;
    const int n_nope = head_dim - n_rot;
    const float *xr = x_in + row * head_dim;
    float *yr = x_out + row * head_dim;
    float scale = 1.0f;
    if (unit_rms) {
        float ss = 0.0f;
        for (int i = threadIdx.x; i < head_dim; i += blockDim.x) ss += xr[i] * xr[i];
        scale = rms_scale(block_sum(ss, red), (float)head_dim, eps);   // barrier: all reads done
    }
    for (int i = threadIdx.x; i < n_nope; i += blockDim.x) {
        const float v = xr[i];
        yr[i] = unit_rms ? v * scale : v;
    }
    const float posf = (float)(pos ? pos[row / n_heads] : single_pos);
    const float ts = rope_theta_scale(p, n_rot);
    for (int k = threadIdx.x; k < n_rot / 2; k += blockDim.x) {
        float te = posf;
        for (int q = 0; q < k; ++q) te *= ts;
        float c, s;
        rope_cs(p, k, te, inverse != 0, c, s);
        float x0 = xr[n_nope + 2 * k], x1 = xr[n_nope + 2 * k + 1];
        if (unit_rms) { x0 *= scale; x1 *= scale; }
        rotate(x0, x1, c, s);
        yr[n_nope + 2 * k] = x0;
        yr[n_nope + 2 * k + 1] = x1;
    }
}

// --------------------------- FP8 round trip ---------------------------------
// head_dim % 64 == 0 and n_rot % 64 == 0: float4 number i belongs to 64-block
// i/16, i.e. one half-warp, so the block amax is a 4-step shuffle.
template <int VPT>
__global__ void __launch_bounds__(kRowsPerCta * 32)
fp8_round_trip_kernel(const float *kv_in, float *kv_out, int64_t n_rows, int head_dim, int n_rot) {
    const int lane = threadIdx.x & 31;
    const int64_t row = (int64_t)blockIdx.x * kRowsPerCta + (threadIdx.x >> 5);
    if (row >= n_rows) return;
    const int n4 = head_dim >> 2, n_nope = head_dim - n_rot;
    const float *xr = kv_in + row * head_dim;
    float *yr = kv_out + row * head_dim;
    float4 v[VPT];
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
        const int i = lane + 32 * j;
        v[j] = (i < n4) ? ld_stream4(xr + 4 * i) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
        const int i = lane + 32 * j;
        const float amax = fmaxf(halfwarp_max(amax4(v[j])), kFp8AmaxFloor);
        if (i >= n4) continue;
        if (4 * i < n_nope) {
            const float scale = pow2_scale(amax), inv = pow2_recip(scale);
            v[j] = e4m3_round_trip4(v[j], scale, inv);
        }
        st_stream4(yr + 4 * i, v[j]);
    }
}

// Scalar path: one warp per row, two elements of a 64-block per lane.
__global__ void fp8_round_trip_scalar_kernel(const float *kv_in, float *kv_out, int64_t n_rows,
                                             int head_dim, int n_rot) {
    const int lane = threadIdx.x & 31;
    const int64_t row = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= n_rows) return;
    const int n_nope = head_dim - n_rot;
    const float *xr = kv_in + row * head_dim;
    float *yr = kv_out + row * head_dim;
    for (int off = 0; off < n_nope; off += 64) {
        const float a = xr[off + lane], b = xr[off + 32 + lane];
        const float amax = fmaxf(warp_max(fmaxf(fabsf(a), fabsf(b))), kFp8AmaxFloor);
        const float scale = pow2_scale(amax), inv = 1.0f / scale;
        yr[off + lane] = e4m3_round_trip(a, scale, inv);
        yr[off + 32 + lane] = e4m3_round_trip(b, scale, inv);
    }
    for (int i = n_nope + lane; i < head_dim; i += 32) yr[i] = xr[i];
}

// ------------------ fused norm -> RoPE -> FP8 cache store -------------------
struct StoreArgs {
    const float *kv_in;
    int64_t n_rows;
    int head_dim, n_rot;
    const int32_t *pos;
    RopeDev rope;
    int do_rope;
    const float *norm_w;
    float eps;
    int scale_mode;
    const int32_t *slots;
    uint8_t *codes;
    float *scales;
    float *tail_out;
    float *rope_out;
    float *raw_out;     // BLOCK64_POW2 only: f16-rounded round-trip row, the raw-KV cache form
    const float2 *cs_table;   // optional [n_rows][n_rot / 2] from rope_table_kernel (replaces pos + rope)
    float2 *cs_out;           // optional [n_rows][n_rot / 2]: the angles evaluated here become that table
};

// f32 -> f16 -> f32, the rounding the reference applies when a row enters its raw KV cache
// (cuda/forward_layer.cu:182-190).
__device__ __forceinline__ float f16_round(float v) { return __half2float(__float2half_rn(v)); }
__device__ __forceinline__ float4 f16_round4(float4 v) {
    return make_float4(f16_round(v.x), f16_round(v.y), f16_round(v.z), f16_round(v.w));
}

template <int VPT>
__global__ void __launch_bounds__(kRowsPerCta * 32) rope_fp8_store_kernel(StoreArgs a) {
    const int lane = threadIdx.x & 31;
    const int64_t row = (int64_t)blockIdx.x * kRowsPerCta + (threadIdx.x >> 5);
    if (row >= a.n_rows) return;
    const int head_dim = a.head_dim, n4 = head_dim >> 2, n_nope = head_dim - a.n_rot;
    const float *xr = a.kv_in + row * head_dim;
    // the lane's table entry travels with the row loads instead of behind the norm's reduction
    float2 cs = make_float2(1.0f, 0.0f);
    if (a.cs_table && 2 * lane < a.n_rot) cs = __ldg(a.cs_table + row * (a.n_rot >> 1) + lane);
    float4 v[VPT];
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
        const int i = lane + 32 * j;
        v[j] = (i < n4) ? ld_stream4(xr + 4 * i) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    if (a.norm_w) {                                   // cuda/forward_layer.cu:868 kv_norm
        float ss = 0.0f;
#pragma unroll
        for (int j = 0; j < VPT; ++j) ss += dot4(v[j]);
        const float scale = rms_scale(warp_sum(ss), (float)head_dim, a.eps);
#pragma unroll
        for (int j = 0; j < VPT; ++j) {
            const int i = lane + 32 * j;
            if (i >= n4) continue;
            const float4 w4 = ld_ro4(a.norm_w + 4 * i);
            v[j] = make_float4(v[j].x * scale * w4.x, v[j].y * scale * w4.y,
                               v[j].z * scale * w4.z, v[j].w * scale * w4.w);
        }
    }
    if (a.do_rope) {                                  // cuda/forward_layer.cu:910 KV RoPE
        if (a.cs_table) rope_tail_apply<VPT>(v, lane, n4, n_nope, cs.x, cs.y);
        else rope_tail_warp<VPT>(v, lane, n4, n_nope, a.n_rot, (float)a.pos[row], a.rope, false, nullptr,
                                 a.cs_out ? a.cs_out + row * (a.n_rot >> 1) : nullptr);
    }
    if (a.rope_out) {
#pragma unroll
        for (int j = 0; j < VPT; ++j) {
            const int i = lane + 32 * j;
            if (i < n4) st_stream4(a.rope_out + row * head_dim + 4 * i, v[j]);
        }
    }
    const int64_t slot = a.slots ? a.slots[row] : row;
    uint32_t *code_row = reinterpret_cast<uint32_t *>(a.codes + slot * head_dim);
    if (a.scale_mode == DS4B200_FP8_ROW_AMAX) {
        float amax = 0.0f;
#pragma unroll
        for (int j = 0; j < VPT; ++j) amax = fmaxf(amax, amax4(v[j]));
        amax = fmaxf(warp_max(amax), kFp8AmaxFloor);
        const float scale = amax / kFp8Max;
        const float inv = 1.0f / scale;               // one IEEE reciprocal per row, see div_with_rcp
        if (lane == 0) a.scales[slot] = scale;
#pragma unroll
        for (int j = 0; j < VPT; ++j) {
            const int i = lane + 32 * j;
            if (i >= n4) continue;
            // the conversion saturates at +-448 itself
            const float4 q = make_float4(div_with_rcp(v[j].x, scale, inv), div_with_rcp(v[j].y, scale, inv),
                                         div_with_rcp(v[j].z, scale, inv), div_with_rcp(v[j].w, scale, inv));
            __stcs(code_row + i, e4m3_encode4(q));
        }
    } else {                                          // cuda/fp8_kv.cu:161-180 scale rule
        const int n_scales = n_nope >> 6;
#pragma unroll
        for (int j = 0; j < VPT; ++j) {
            const int i = lane + 32 * j;
            const float amax = fmaxf(halfwarp_max(amax4(v[j])), kFp8AmaxFloor);
            if (i >= n4) continue;
            if (4 * i < n_nope) {
                const float scale = pow2_scale(amax), inv = pow2_recip(scale);     // power of two: x*inv == x/scale
                if (a.scales && (lane & 15) == 0) a.scales[slot * n_scales + (i >> 4)] = scale;
                if (a.codes) {
                    // the conversion saturates at +-448 itself
                    __stcs(code_row + i, e4m3_encode4(make_float4(v[j].x * inv, v[j].y * inv, v[j].z * inv, v[j].w * inv)));
                }
                if (a.raw_out)
                    st_stream4(a.raw_out + slot * head_dim + 4 * i,
                               f16_round4(e4m3_round_trip4(v[j], scale, inv)));
            } else {
                if (a.codes) __stcs(code_row + i, 0u);
                if (a.tail_out) st_stream4(a.tail_out + slot * a.n_rot + (4 * i - n_nope), v[j]);
                if (a.raw_out) st_stream4(a.raw_out + slot * head_dim + 4 * i, f16_round4(v[j]));
            }
        }
    }
}

// ------------------------------ FP8 cache read -------------------------------
// The read side of the byte cache: row r = slot slots[r] -> f32.  BLOCK64_POW2: prefix =
// code value x block scale (exactly what the reference's round trip leaves in its f32 cache,
// cuda/fp8_kv.cu:176-180), tail = the stored f32 tail.  ROW_AMAX: every element = code value
// x row scale.  One warp per row, 32-bit code loads, 128-bit stores.
template <int VPT>
__global__ void __launch_bounds__(kRowsPerCta * 32)
fp8_cache_load_kernel(const uint8_t *__restrict__ codes, const float *__restrict__ scales,
                      const float *__restrict__ tail, const int32_t *__restrict__ slots, int64_t n_rows,
                      int head_dim, int n_rot, int scale_mode, int f16_out, float *__restrict__ out) {
    const int lane = threadIdx.x & 31;
    const int64_t row = (int64_t)blockIdx.x * kRowsPerCta + (threadIdx.x >> 5);
    if (row >= n_rows) return;
    const int n4 = head_dim >> 2, n_nope = head_dim - n_rot;
    const int64_t slot = slots ? slots[row] : row;
    const uint32_t *code_row = reinterpret_cast<const uint32_t *>(codes + slot * head_dim);
    const int n_scales = scale_mode == DS4B200_FP8_BLOCK64_POW2 ? n_nope >> 6 : 1;
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
        const int i = lane + 32 * j;
        if (i >= n4) continue;
        float4 v;
        if (scale_mode == DS4B200_FP8_BLOCK64_POW2 && 4 * i >= n_nope) {
            v = ld_stream4(tail + slot * n_rot + (4 * i - n_nope));
        } else {
            const uint32_t c = __ldcs(code_row + i);
            const float sc = __ldg(scales + slot * n_scales + (scale_mode == DS4B200_FP8_BLOCK64_POW2 ? (i >> 4) : 0));
            float e[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const uint32_t b = (c >> (8 * k)) & 0xffu;
                const float m = e4m3_magnitude(b & 0x7fu);
                e[k] = ((b & 0x80u) ? -m : m) * sc;
            }
            v = make_float4(e[0], e[1], e[2], e[3]);
        }
        if (f16_out) v = f16_round4(v);
        st_stream4(out + row * head_dim + 4 * i, v);
    }
}

// --------------------------- sliding raw-KV window ---------------------------
// The reference keeps the last `cap` rows in a linear window: append while there is room,
// otherwise move every row down by one and write the new row last, one token per call
// (cuda/forward_layer.cu:159-190, :941-972).  Here n_new rows enter at once: the window
// afterwards holds the last min(cap, n_raw + n_new) rows of old ++ new.  New rows get the
// f16 rounding; old rows already have it.
__global__ void __launch_bounds__(1024)
swa_window_push_kernel(float *raw_kv, int cap, int n_raw, const float *new_rows, int n_new, int head_dim) {
    const int n4 = head_dim >> 2;
    const int total = n_raw + n_new;
    const int kept = total < cap ? total : cap;              // rows in the window afterwards
    const int first = total - kept;                          // index in old ++ new of window row 0
    // One CTA.  A pass moves up to blockDim.x * kBatch float4s: every thread loads its share,
    // the CTA synchronises, every thread stores.  Passes go upwards through the window and a
    // pass only reads rows at or above the ones it writes, so the move is safe in place.
    constexpr int kBatch = 8;
    const int64_t begin = (int64_t)(first == 0 ? n_raw : 0) * n4;          // pure append: old rows stay
    const int64_t end = (int64_t)kept * n4;
    for (int64_t base = begin; base < end; base += (int64_t)blockDim.x * kBatch) {
        float4 v[kBatch];
#pragma unroll
        for (int b = 0; b < kBatch; ++b) {
            const int64_t e = base + (int64_t)b * blockDim.x + threadIdx.x;
            if (e < end) {
                const int r = (int)(e / n4), c = (int)(e - (int64_t)r * n4), src = first + r;
                v[b] = src < n_raw ? *reinterpret_cast<const float4 *>(raw_kv + (int64_t)src * head_dim + 4 * c)
                                   : f16_round4(__ldg(reinterpret_cast<const float4 *>(
                                         new_rows + (int64_t)(src - n_raw) * head_dim + 4 * c)));
            }
        }
        __syncthreads();
#pragma unroll
        for (int b = 0; b < kBatch; ++b) {
            const int64_t e = base + (int64_t)b * blockDim.x + threadIdx.x;
            if (e < end) *reinterpret_cast<float4 *>(raw_kv + 4 * e) = v[b];
        }
        __syncthreads();
    }
}

// ------------------------------ E4M3 utilities --------------------------------
__global__ void e4m3_encode_kernel(const float *x, uint8_t *codes, int64_t n) {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n;
         i += (int64_t)gridDim.x * blockDim.x)
        codes[i] = e4m3_encode1(x[i]);
}
__global__ void e4m3_decode_kernel(const uint8_t *codes, float *x, int64_t n) {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n;
         i += (int64_t)gridDim.x * blockDim.x) {
        const float m = e4m3_magnitude(codes[i] & 0x7fu);
        x[i] = (codes[i] & 0x80u) ? -m : m;
    }
}

// The reference's selection rule stated arithmetically: the largest index whose
// value is <= ax comes from the exponent and the top three mantissa bits, then
// the tie rule of cuda/fp8_kv.cu:118-127 decides between it and the next one.
__device__ __forceinline__ uint32_t e4m3_index_by_rule(float ax) {
    ax = fminf(ax, kFp8Max);
    uint32_t i;
    if (ax < 0.015625f) {
        i = (uint32_t)(ax * 512.0f);                   // floor; values are m * 2^-9
    } else {
        const uint32_t b = __float_as_uint(ax);
        i = (((b >> 23) - 120u) << 3) | ((b >> 20) & 7u);
    }
    if (i < 126u) {
        const float d0 = fabsf(ax - e4m3_magnitude(i));
        const float d1 = fabsf(ax - e4m3_magnitude(i + 1u));
        if (d1 < d0 || (d1 == d0 && (i & 1u))) ++i;
    }
    return i;
}

__global__ void e4m3_selfcheck_kernel(uint32_t first_bits, uint64_t count,
                                      unsigned long long *mismatches) {
    unsigned long long bad = 0;
    for (uint64_t k = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; k < count;
         k += (uint64_t)gridDim.x * blockDim.x) {
        const uint32_t bits = first_bits + (uint32_t)k;
        const float v = __uint_as_float(bits);
        if (v != v) continue;
        const uint32_t want = ((bits >> 24) & 0x80u) | e4m3_index_by_rule(fabsf(v));
        const uint32_t got = e4m3_encode1(v);
        bad += (want != got);
    }
    bad = __reduce_add_sync(0xffffffffu, (unsigned)bad);
    if ((threadIdx.x & 31) == 0 && bad) atomicAdd(mismatches, bad);
}

unsigned warp_row_grid(int64_t n_rows) { return (unsigned)((n_rows + kRowsPerCta - 1) / kRowsPerCta); }

}  // namespace

void rope_rows(const float *x_in, float *x_out, int64_t n_tokens, int n_heads, int head_dim,
               int n_rot, const int32_t *pos, int single_pos, const ds4b200_rope_params &p,
               int inverse, int unit_rms, float eps, cudaStream_t s, int8_t *xq, float *xscale,
               const float *cs_table) {
    const int64_t n_rows = n_tokens * n_heads;
    if (n_rows <= 0 || head_dim <= 0) return;
    const RopeDev d = to_dev(p);
    const float2 *cs = (n_rot <= 64) ? reinterpret_cast<const float2 *>(cs_table) : nullptr;
    if (xq) {
        // checked by the caller: head_dim % 32 == 0, head_dim <= 1024, n_rot % 4 == 0, 16-byte rows
        const int vpt = ((head_dim >> 2) + 31) / 32;
        const unsigned grid = warp_row_grid(n_rows);
#define DS4B200_ROPEQ(V) rope_rows_kernel<V, true><<<grid, kRowsPerCta * 32, 0, s>>>( \
        x_in, x_out, n_rows, n_heads, head_dim, n_rot, pos, single_pos, d, inverse, unit_rms, eps, xq, xscale, cs)
        if (vpt <= 1) DS4B200_ROPEQ(1);
        else if (vpt <= 2) DS4B200_ROPEQ(2);
        else if (vpt <= 4) DS4B200_ROPEQ(4);
        else DS4B200_ROPEQ(8);
#undef DS4B200_ROPEQ
        return;
    }
    const bool vec = (head_dim & 3) == 0 && (n_rot & 3) == 0 && head_dim <= 1024 &&
                     aligned16(x_in) && aligned16(x_out);
    if (!vec) {
        rope_rows_scalar_kernel<<<(unsigned)n_rows, 64, 0, s>>>(x_in, x_out, n_heads, head_dim, n_rot,
                                                              pos, single_pos, d, inverse, unit_rms, eps);
        return;
    }
    const int vpt = ((head_dim >> 2) + 31) / 32;
    const unsigned grid = warp_row_grid(n_rows);
#define DS4B200_ROPE(V) rope_rows_kernel<V, false><<<grid, kRowsPerCta * 32, 0, s>>>( \
        x_in, x_out, n_rows, n_heads, head_dim, n_rot, pos, single_pos, d, inverse, unit_rms, eps, nullptr, nullptr, cs)
    if (vpt <= 1) DS4B200_ROPE(1);
    else if (vpt <= 2) DS4B200_ROPE(2);
    else if (vpt <= 4) DS4B200_ROPE(4);
    else DS4B200_ROPE(8);
#undef DS4B200_ROPE
}

void rope_table_rows(const int32_t *pos, int64_t n_tokens, int n_rot, const ds4b200_rope_params &p, float *cs_table,
                     cudaStream_t s) {
    const int n_pairs = n_rot >> 1;
    const int64_t n = n_tokens * n_pairs;
    if (n <= 0) return;
    rope_table_kernel<<<(unsigned)((n + 255) / 256), 256, 0, s>>>(pos, n_tokens, n_pairs, n_rot, to_dev(p),
                                                                  reinterpret_cast<float2 *>(cs_table));
}

void fp8_kv_round_trip_rows(const float *kv_in, float *kv_out, int64_t n_rows, int head_dim,
                            int n_rot, cudaStream_t s) {
    if (n_rows <= 0 || head_dim <= 0) return;
    const bool vec = (head_dim & 63) == 0 && (n_rot & 63) == 0 && head_dim <= 1024 &&
                     aligned16(kv_in) && aligned16(kv_out);
    const unsigned grid = warp_row_grid(n_rows);
    if (!vec) {
        fp8_round_trip_scalar_kernel<<<grid, kRowsPerCta * 32, 0, s>>>(kv_in, kv_out, n_rows, head_dim, n_rot);
        return;
    }
    const int vpt = ((head_dim >> 2) + 31) / 32;
#define DS4B200_FP8RT(V) fp8_round_trip_kernel<V><<<grid, kRowsPerCta * 32, 0, s>>>(kv_in, kv_out, n_rows, head_dim, n_rot)
    if (vpt <= 1) DS4B200_FP8RT(1);
    else if (vpt <= 2) DS4B200_FP8RT(2);
    else if (vpt <= 4) DS4B200_FP8RT(4);
    else DS4B200_FP8RT(8);
#undef DS4B200_FP8RT
}

void rope_fp8_store_rows(const float *kv_in, int64_t n_rows, int head_dim, int n_rot,
                         const int32_t *pos, const ds4b200_rope_params *p, const float *norm_w,
                         float eps, int scale_mode, const int32_t *slots, uint8_t *codes,
                         float *scales, float *tail_out, float *rope_out, cudaStream_t s, float *raw_out,
                         const float *cs_table, float *cs_out) {
    if (n_rows <= 0) return;
    StoreArgs a{};
    a.raw_out = raw_out;
    a.cs_table = (p && n_rot <= 64) ? reinterpret_cast<const float2 *>(cs_table) : nullptr;
    a.cs_out = (p && n_rot <= 64 && !cs_table) ? reinterpret_cast<float2 *>(cs_out) : nullptr;
    a.kv_in = kv_in; a.n_rows = n_rows; a.head_dim = head_dim; a.n_rot = n_rot; a.pos = pos;
    a.do_rope = p != nullptr;
    if (p) a.rope = to_dev(*p);
    a.norm_w = norm_w; a.eps = eps; a.scale_mode = scale_mode; a.slots = slots; a.codes = codes;
    a.scales = scales; a.tail_out = tail_out; a.rope_out = rope_out;
    const int vpt = ((head_dim >> 2) + 31) / 32;
    const unsigned grid = warp_row_grid(n_rows);
    if (vpt <= 1) rope_fp8_store_kernel<1><<<grid, kRowsPerCta * 32, 0, s>>>(a);
    else if (vpt <= 2) rope_fp8_store_kernel<2><<<grid, kRowsPerCta * 32, 0, s>>>(a);
    else if (vpt <= 4) rope_fp8_store_kernel<4><<<grid, kRowsPerCta * 32, 0, s>>>(a);
    else rope_fp8_store_kernel<8><<<grid, kRowsPerCta * 32, 0, s>>>(a);
}

void fp8_cache_load_rows(const uint8_t *codes, const float *scales, const float *tail, const int32_t *slots,
                         int64_t n_rows, int head_dim, int n_rot, int scale_mode, int f16_out, float *out,
                         cudaStream_t s) {
    if (n_rows <= 0) return;
    const int vpt = ((head_dim >> 2) + 31) / 32;
    const unsigned grid = warp_row_grid(n_rows);
#define DS4B200_LOAD(V) fp8_cache_load_kernel<V><<<grid, kRowsPerCta * 32, 0, s>>>( \
        codes, scales, tail, slots, n_rows, head_dim, n_rot, scale_mode, f16_out, out)
    if (vpt <= 1) DS4B200_LOAD(1);
    else if (vpt <= 2) DS4B200_LOAD(2);
    else if (vpt <= 4) DS4B200_LOAD(4);
    else DS4B200_LOAD(8);
#undef DS4B200_LOAD
}

void swa_window_push_rows(float *raw_kv, int cap, int n_raw, const float *new_rows, int n_new, int head_dim,
                          cudaStream_t s) {
    if (n_new <= 0 || cap <= 0) return;
    swa_window_push_kernel<<<1, 1024, 0, s>>>(raw_kv, cap, n_raw, new_rows, n_new, head_dim);
}

void e4m3_encode(const float *x, uint8_t *codes, int64_t n, cudaStream_t s) {
    if (n > 0) e4m3_encode_kernel<<<148 * 8, 256, 0, s>>>(x, codes, n);
}
void e4m3_decode(const uint8_t *codes, float *x, int64_t n, cudaStream_t s) {
    if (n > 0) e4m3_decode_kernel<<<148 * 8, 256, 0, s>>>(codes, x, n);
}
void e4m3_selfcheck(uint32_t first_bits, uint64_t count, unsigned long long *mismatches,
                    cudaStream_t s) {
    if (count > 0) e4m3_selfcheck_kernel<<<148 * 16, 256, 0, s>>>(first_bits, count, mismatches);
}

}  // namespace ds4b200
