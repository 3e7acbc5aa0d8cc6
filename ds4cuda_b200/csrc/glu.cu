// glu.cu — SwiGLU over token rows: plain silu(g)*u (cuda/glu.cu:56-75), the
// clamped, router-weighted form of the routed-expert epilogue
// (cuda/moe_iq2_pair.cu:352-373), and the sum over the k selected experts fused
// in, so the k gate rows and k up rows of a token are read once and one
// combined row is written.
//
// Data movement: pure streaming.  One thread owns one float4 column of one
// token across all k slots: 2k independent 128-bit loads are in flight per
// thread before the first use, stores are 128-bit, all coalesced.
#include "device_utils.cuh"
#include "kernels.cuh"
#include "q8k_device.cuh"

namespace ds4b200 {
namespace {

template <bool FAST>
__device__ __forceinline__ float exp_sel(float x) { return FAST ? __expf(x) : expf(x); }

// One exponential and one division per element: both branches of the
// reference's sign test use e = exp(-|g|) and divide by (1 + e); only the
// numerator differs (g or g*e, 1 or e), so selecting the numerator first gives
// the same bits as evaluating the taken branch.
template <int MODE, bool FAST>
__device__ __forceinline__ float glu_one(float g, float u, float clamp) {
    if (MODE != DS4B200_GLU_PLAIN && clamp > 1.0e-6f) {
        g = fminf(g, clamp);
        if (MODE == DS4B200_GLU_CLAMP_SYM) g = fmaxf(g, -clamp);
        u = fminf(fmaxf(u, -clamp), clamp);
    }
    const float e = exp_sel<FAST>(-fabsf(g));
    const float den = 1.0f + e;
    if (MODE == DS4B200_GLU_PLAIN) {
        // (g * sigmoid_stable(g)) * u, cuda/glu.cu:56-75
        const float sg = div_by_1to2(g >= 0.0f ? 1.0f : e, den);
        return (g * sg) * u;
    }
    // s = g/(1+e) or (g*e)/(1+e), then s*u, cuda/moe_iq2_pair.cu:362-372
    const float s = div_by_1to2(g >= 0.0f ? g : g * e, den);
    return s * u;
}

// The reference rounds s*u*w to f32 (it is stored to memory) before the slot sum
// (cuda/moe_iq2_pair.cu:372, cuda/moe_q2k_sum6.cu:159-181): keep the multiply and the add
// as two roundings in every code path, never one fused multiply-add.
__device__ __forceinline__ float4 mul4_rn(float4 v, float w) {
    return make_float4(__fmul_rn(v.x, w), __fmul_rn(v.y, w), __fmul_rn(v.z, w), __fmul_rn(v.w, w));
}
__device__ __forceinline__ float4 add4_rn(float4 a, float4 b) {
    return make_float4(__fadd_rn(a.x, b.x), __fadd_rn(a.y, b.y), __fadd_rn(a.z, b.z), __fadd_rn(a.w, b.w));
}

template <int MODE, bool FAST>
__device__ __forceinline__ float4 glu4(float4 g, float4 u, float clamp) {
    return make_float4(glu_one<MODE, FAST>(g.x, u.x, clamp), glu_one<MODE, FAST>(g.y, u.y, clamp),
                       glu_one<MODE, FAST>(g.z, u.z, clamp), glu_one<MODE, FAST>(g.w, u.w, clamp));
}

// K > 0: compile-time slot count (loads fully unrolled); K == 0: runtime k.
template <int K, int MODE, bool FAST>
__global__ void __launch_bounds__(256, 4)
swiglu_vec_kernel(const float *__restrict__ gate, const float *__restrict__ up,
                  const float *__restrict__ weights, float *__restrict__ out, int64_t n_tokens,
                  int k_rt, int n4, float clamp, int combine) {
    const int k = K > 0 ? K : k_rt;
    const int64_t total = n_tokens * n4;
    for (int64_t gid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; gid < total;
         gid += (int64_t)gridDim.x * blockDim.x) {
        const int64_t t = gid / n4;
        const int c = (int)(gid - t * n4);
        const int64_t base = (t * k) * (int64_t)n4 + c;       // float4 index of slot 0
        if (K > 0) {
            float4 g[K > 0 ? K : 1], u[K > 0 ? K : 1];
#pragma unroll
            for (int s = 0; s < K; ++s) {
                g[s] = ld_stream4(gate + 4 * (base + (int64_t)s * n4));
                u[s] = ld_stream4(up + 4 * (base + (int64_t)s * n4));
            }
            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
            for (int s = 0; s < K; ++s) {
                float4 v = glu4<MODE, FAST>(g[s], u[s], clamp);
                if (weights) {
                    const float w = __ldg(weights + t * k + s);
                    v = mul4_rn(v, w);
                }
                if (combine) acc = (s == 0) ? v : add4_rn(acc, v);
                else st_stream4(out + 4 * (base + (int64_t)s * n4), v);
            }
            if (combine) st_stream4(out + 4 * gid, acc);
        } else {
            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
            for (int s = 0; s < k; ++s) {
                float4 v = glu4<MODE, FAST>(ld_stream4(gate + 4 * (base + (int64_t)s * n4)),
                                            ld_stream4(up + 4 * (base + (int64_t)s * n4)), clamp);
                if (weights) {
                    const float w = __ldg(weights + t * k + s);
                    v = mul4_rn(v, w);
                }
                if (combine) acc = (s == 0) ? v : add4_rn(acc, v);
                else st_stream4(out + 4 * (base + (int64_t)s * n4), v);
            }
            if (combine) st_stream4(out + 4 * gid, acc);
        }
    }
}

// SwiGLU whose output leaves as Q8_K blocks, the form the routed experts' down projection
// takes its activations in (cuda/moe_iq2_pair.cu:159-235 quantises the f32 `mid` rows in a
// second kernel).  One warp per 256-element block of one (token, slot) row: the eight values
// of a lane go from the epilogue straight into the block quantiser, so the f32 rows are
// neither written nor read back (mid_f32 is optional, for callers that want them too).
template <int MODE, bool FAST, int NB>
__global__ void __launch_bounds__(256)
swiglu_q8k_kernel(const float *__restrict__ gate, const float *__restrict__ up,
                  const float *__restrict__ weights, int8_t *__restrict__ xq, float *__restrict__ xscale,
                  int16_t *__restrict__ xbsums, float *__restrict__ mid_f32, int64_t n_blocks,
                  int blocks_per_row, float clamp) {
    const int lane = threadIdx.x & 31;
    const int64_t b0 = ((int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5)) * NB;
    if (b0 >= n_blocks) return;
    // a warp takes NB consecutive blocks and issues all 4*NB loads of a lane before the first
    // epilogue, so every thread keeps 64*NB bytes in flight
    float4 g[NB][2], u[NB][2];
#pragma unroll
    for (int i = 0; i < NB; ++i) {
        if (b0 + i < n_blocks) {
            const int64_t base = (b0 + i) * 256;
            g[i][0] = ld_stream4(gate + base + 4 * lane); g[i][1] = ld_stream4(gate + base + 128 + 4 * lane);
            u[i][0] = ld_stream4(up + base + 4 * lane);   u[i][1] = ld_stream4(up + base + 128 + 4 * lane);
        }
    }
#pragma unroll
    for (int i = 0; i < NB; ++i) {
        const int64_t b = b0 + i;
        if (b >= n_blocks) break;
        const int64_t base = b * 256;
        float4 v0 = glu4<MODE, FAST>(g[i][0], u[i][0], clamp);
        float4 v1 = glu4<MODE, FAST>(g[i][1], u[i][1], clamp);
        if (weights) {
            const float w = __ldg(weights + b / blocks_per_row);        // one weight per (token, slot) row
            v0 = mul4_rn(v0, w);
            v1 = mul4_rn(v1, w);
        }
        if (mid_f32) {
            st_stream4(mid_f32 + base + 4 * lane, v0);
            st_stream4(mid_f32 + base + 128 + 4 * lane, v1);
        }
        const float e[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
        q8k_block_store(e, lane, xq + base, xscale + b, xbsums + b * 16);
    }
}

// SwiGLU whose output leaves as Q8_0 blocks, the form the shared expert's down projection quantises its
// activations to (launch_silu_mul_f32 at cuda/forward_layer.cu:1296, then the quantiser inside the Q8_0
// matvec, cuda/dense_q8.cu:122-152).  A thread holds four values, a block of 32 is eight consecutive lanes;
// n % 32 == 0, so the groups of eight lanes never straddle a row.  mid_f32 is optional.
template <int MODE, bool FAST>
__global__ void __launch_bounds__(256)
swiglu_q8_0_kernel(const float *__restrict__ gate, const float *__restrict__ up, const float *__restrict__ weights,
                   int8_t *__restrict__ xq, float *__restrict__ xscale, float *__restrict__ mid_f32, int64_t total4,
                   int n4, float clamp) {
    const int lane = threadIdx.x & 31;
    // the loop bound is the warp's, not the thread's: the shuffles below want all 32 lanes
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i - lane < total4;
         i += (int64_t)gridDim.x * blockDim.x) {
        const bool live = i < total4;
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (live) {
            v = glu4<MODE, FAST>(ld_stream4(gate + 4 * i), ld_stream4(up + 4 * i), clamp);
            if (weights) v = mul4_rn(v, __ldg(weights + i / n4));
            if (mid_f32) st_stream4(mid_f32 + 4 * i, v);
        }
        float amax = amax4(v);
#pragma unroll
        for (int off = 4; off > 0; off >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
        float d, id;
        q8_0_block_scale(amax, d, id);
        if (live) {
            reinterpret_cast<uint32_t *>(xq)[i] = q8_pack4_sat(v.x * id, v.y * id, v.z * id, v.w * id);
            if ((i & 7) == 0) xscale[i >> 3] = d;
        }
    }
}

template <int MODE, bool FAST>
__global__ void swiglu_scalar_kernel(const float *gate, const float *up, const float *weights,
                                     float *out, int64_t n_tokens, int k, int n, float clamp,
                                     int combine) {
    const int64_t total = n_tokens * n;
    for (int64_t gid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; gid < total;
         gid += (int64_t)gridDim.x * blockDim.x) {
        const int64_t t = gid / n;
        const int j = (int)(gid - t * n);
        float acc = 0.0f;
        for (int s = 0; s < k; ++s) {
            const int64_t idx = (t * k + s) * (int64_t)n + j;
            float v = glu_one<MODE, FAST>(gate[idx], up[idx], clamp);
            if (weights) v = __fmul_rn(v, weights[t * k + s]);
            if (combine) acc = (s == 0) ? v : __fadd_rn(acc, v);
            else out[idx] = v;
        }
        if (combine) out[gid] = acc;
    }
}

// One decode row without slots, weights or a sum: no loop, 32-bit index.
template <int MODE, bool FAST>
__global__ void swiglu_row_kernel(const float *__restrict__ gate, const float *__restrict__ up, float *__restrict__ out,
                                  int n, float clamp) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = glu_one<MODE, FAST>(gate[i], up[i], clamp);
}

// Counts (n, d) pairs, d in [1, 2], n spread over +-2^-40..2^40 and signs, for which
// div_by_1to2 differs from the IEEE division, plus (a, b) pairs for which div_with_rcp does, plus block
// maxima for which q8_0_block_scale differs from amax / 127 and its IEEE reciprocal, or q8k_block_scale from
// -127 / max and its IEEE reciprocal.
// Pairs come from a counter-based hash.
__global__ void div_selfcheck_kernel(uint64_t first, uint64_t count, unsigned long long *mismatches) {
    unsigned bad = 0;
    for (uint64_t k = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; k < count;
         k += (uint64_t)gridDim.x * blockDim.x) {
        uint64_t z = (first + k) * 0x9E3779B97F4A7C15ull;
        z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
        z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
        z ^= z >> 31;
        const float d = __uint_as_float(0x3f800000u | (uint32_t)(z & 0x7fffffu));          // [1, 2)
        const uint32_t ne = 87u + (uint32_t)((z >> 23) % 81u);                               // exponent 2^-40..2^40
        const float n = __uint_as_float(((uint32_t)(z >> 63) << 31) | (ne << 23) | (uint32_t)((z >> 32) & 0x7fffffu));
        const float dd = (k & 1023u) == 0 ? 2.0f : d;                                         // include the end point
        bad += (__float_as_uint(div_by_1to2(n, dd)) != __float_as_uint(n / dd));
        // the shared-reciprocal division of the FP8 row quantiser: divisor 2^-23..2^23, quotient
        // 2^-20..2^9, both signs
        const float b = __uint_as_float(((104u + (uint32_t)((z >> 40) % 47u)) << 23) | (uint32_t)(z & 0x7fffffu));
        const float qt = __uint_as_float(((uint32_t)(z >> 63) << 31) | ((107u + (uint32_t)((z >> 48) % 30u)) << 23) |
                                         (uint32_t)((z >> 9) & 0x7fffffu));
        const float a = qt * b;
        bad += (__float_as_uint(div_with_rcp(a, b, 1.0f / b)) != __float_as_uint(a / b));
        // the Q8_0 block scale and its reciprocal against the plain IEEE expressions (cuda/dense_q8.cu:140-143):
        // every mantissa at the exponents 2^-99 .. 2^126, taken in turn (2^31 counters cover them all)
        const uint64_t kk = first + k;
        const float amax = __uint_as_float(((28u + (uint32_t)((kk >> 23) % 226u)) << 23) | (uint32_t)(kk & 0x7fffffu));
        float sd, sid;
        q8_0_block_scale(amax, sd, sid);
        const float want_d = amax / 127.0f;
        bad += (__float_as_uint(sd) != __float_as_uint(want_d)) + (__float_as_uint(sid) != __float_as_uint(1.0f / want_d));
        // the Q8_K block scale, both signs of the same maxima
#pragma unroll
        for (int sgn = 0; sgn < 2; ++sgn) {
            const float smax = sgn ? -amax : amax;
            float is, dq;
            q8k_block_scale(smax, is, dq);
            const float want_is = -127.0f / smax;
            bad += (__float_as_uint(is) != __float_as_uint(want_is)) + (__float_as_uint(dq) != __float_as_uint(1.0f / want_is));
        }
    }
    bad = __reduce_add_sync(0xffffffffu, bad);
    if ((threadIdx.x & 31) == 0 && bad) atomicAdd(mismatches, (unsigned long long)bad);
}

template <int MODE, bool FAST>
void launch_mode(const float *gate, const float *up, const float *weights, float *out,
                 int64_t n_tokens, int k, int n, float clamp, int combine, cudaStream_t s) {
    constexpr int kThreads = 256;
    const bool vec = (n & 3) == 0 && aligned16(gate) && aligned16(up) && aligned16(out);
    // A single decode row (a few thousand elements) is latency-bound: one element per
    // thread over many small CTAs finishes sooner than four per thread over two CTAs.
    const bool tiny = n_tokens * (int64_t)n <= 8192;
    if (tiny && k == 1 && !weights) {
        const int total = (int)(n_tokens * n);
        swiglu_row_kernel<MODE, FAST><<<(unsigned)((total + 127) / 128), 128, 0, s>>>(gate, up, out, total, clamp);
        return;
    }
    if (!vec || tiny) {
        const int threads = tiny ? 128 : kThreads;
        int64_t blocks = (n_tokens * n + threads - 1) / threads;
        if (blocks > 148 * 32) blocks = 148 * 32;
        swiglu_scalar_kernel<MODE, FAST><<<(unsigned)blocks, threads, 0, s>>>(
            gate, up, weights, out, n_tokens, k, n, clamp, combine);
        return;
    }
    const int n4 = n >> 2;
    int64_t blocks = (n_tokens * n4 + kThreads - 1) / kThreads;
    if (blocks > (int64_t)1 << 30) blocks = (int64_t)1 << 30;
#define DS4B200_GLU(K) swiglu_vec_kernel<K, MODE, FAST><<<(unsigned)blocks, kThreads, 0, s>>>( \
        gate, up, weights, out, n_tokens, k, n4, clamp, combine)
    if (k == 1) DS4B200_GLU(1);
    else if (k == 6) DS4B200_GLU(6);
    else if (k == 8) DS4B200_GLU(8);
    else DS4B200_GLU(0);
#undef DS4B200_GLU
}

}  // namespace

void div_selfcheck(uint64_t first, uint64_t count, unsigned long long *mismatches, cudaStream_t s) {
    if (count > 0) div_selfcheck_kernel<<<148 * 16, 256, 0, s>>>(first, count, mismatches);
}

void swiglu_q8_K_rows(const float *gate, const float *up, const float *weights, int8_t *xq, float *xscale,
                      int16_t *xbsums, float *mid_f32, int64_t n_rows, int n, int mode, float clamp,
                      int fast_exp, cudaStream_t s) {
    const int blocks_per_row = n / 256;
    const int64_t n_blocks = n_rows * blocks_per_row;
    if (n_blocks <= 0) return;
    // few blocks: one per warp (more warps); many: two per warp (more bytes in flight per thread)
    const bool many = n_blocks >= 148 * 64;
    const unsigned grid = (unsigned)(many ? (n_blocks + 15) / 16 : (n_blocks + 7) / 8);
#define DS4B200_Q8K(M, F)                                                                                              \
    do {                                                                                                               \
        if (many) swiglu_q8k_kernel<M, F, 2><<<grid, 256, 0, s>>>(gate, up, weights, xq, xscale, xbsums, mid_f32,      \
                                                                  n_blocks, blocks_per_row, clamp);                    \
        else swiglu_q8k_kernel<M, F, 1><<<grid, 256, 0, s>>>(gate, up, weights, xq, xscale, xbsums, mid_f32, n_blocks, \
                                                             blocks_per_row, clamp);                                   \
    } while (0)
    if (mode == DS4B200_GLU_PLAIN) { if (fast_exp) DS4B200_Q8K(DS4B200_GLU_PLAIN, true); else DS4B200_Q8K(DS4B200_GLU_PLAIN, false); }
    else if (mode == DS4B200_GLU_CLAMP_REF) { if (fast_exp) DS4B200_Q8K(DS4B200_GLU_CLAMP_REF, true); else DS4B200_Q8K(DS4B200_GLU_CLAMP_REF, false); }
    else { if (fast_exp) DS4B200_Q8K(DS4B200_GLU_CLAMP_SYM, true); else DS4B200_Q8K(DS4B200_GLU_CLAMP_SYM, false); }
#undef DS4B200_Q8K
}

void swiglu_q8_0_rows(const float *gate, const float *up, const float *weights, int8_t *xq, float *xscale,
                      float *mid_f32, int64_t n_rows, int n, int mode, float clamp, int fast_exp, cudaStream_t s) {
    const int n4 = n >> 2;
    const int64_t total4 = n_rows * n4;
    if (total4 <= 0) return;
    int64_t blocks = (total4 + 255) / 256;
    if (blocks > (int64_t)1 << 30) blocks = (int64_t)1 << 30;
#define DS4B200_Q80(M, F) swiglu_q8_0_kernel<M, F><<<(unsigned)blocks, 256, 0, s>>>(gate, up, weights, xq, xscale, \
                                                                                   mid_f32, total4, n4, clamp)
    if (mode == DS4B200_GLU_PLAIN) { if (fast_exp) DS4B200_Q80(DS4B200_GLU_PLAIN, true); else DS4B200_Q80(DS4B200_GLU_PLAIN, false); }
    else if (mode == DS4B200_GLU_CLAMP_REF) { if (fast_exp) DS4B200_Q80(DS4B200_GLU_CLAMP_REF, true); else DS4B200_Q80(DS4B200_GLU_CLAMP_REF, false); }
    else { if (fast_exp) DS4B200_Q80(DS4B200_GLU_CLAMP_SYM, true); else DS4B200_Q80(DS4B200_GLU_CLAMP_SYM, false); }
#undef DS4B200_Q80
}

void swiglu_rows(const float *gate, const float *up, const float *weights, float *out,
                 int64_t n_tokens, int k, int n, int mode, float clamp, int combine,
                 int fast_exp, cudaStream_t s) {
    if (n_tokens <= 0 || k <= 0 || n <= 0) return;
#define DS4B200_MODE(M)                                                                          \
    do {                                                                                          \
        if (fast_exp) launch_mode<M, true>(gate, up, weights, out, n_tokens, k, n, clamp, combine, s); \
        else launch_mode<M, false>(gate, up, weights, out, n_tokens, k, n, clamp, combine, s);       \
    } while (0)
    if (mode == DS4B200_GLU_PLAIN) DS4B200_MODE(DS4B200_GLU_PLAIN);
    else if (mode == DS4B200_GLU_CLAMP_REF) DS4B200_MODE(DS4B200_GLU_CLAMP_REF);
    else DS4B200_MODE(DS4B200_GLU_CLAMP_SYM);
#undef DS4B200_MODE
}

}  // namespace ds4b200
