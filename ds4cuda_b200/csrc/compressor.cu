// compressor.cu — the row work of one streaming-compressor step, everything after its two
// projections, in ONE launch: add the position bias to the scores and store the token's row
// in the state; when the window closes, pool the state rows per column with softmax
// weights, RMSNorm the pooled row, rotate its tail (YaRN RoPE at the window's position),
// round the prefix through E4M3FN (attention path only) and roll the state.
//
// Arithmetic follows cuda/compressor.cu of the reference: state row and bias :65-90, pool
// :107-164 (maximum first, then exp(s - max) weights summed in row order; ratio 4 pairs
// column j of rows 0-3 with column head_dim + j of rows 4-7), RMSNorm :173-220 (256 strided
// partial sums, xor butterfly inside the warps, then over the eight warp sums — the same
// order here, so the scale comes out bit for bit), tail RoPE cuda/rope.cu:136-201 at
// comp_pos = pos + 1 - ratio, FP8 round trip cuda/fp8_kv.cu:144-195, state roll :232-252.
//
// The reference runs these as five to six launches, the pool with one thread per CTA; here
// one CTA of 512 threads keeps the pooled row in shared memory between the stages.  A step
// is latency-bound (a few KiB of traffic); the point of the fusion is launch count.
#include "device_utils.cuh"
#include "kernels.cuh"
#include "rope_device.cuh"

namespace ds4b200 {
namespace {

constexpr int kThreads = 512;
constexpr int kMaxHeadDim = 1024;
constexpr float kNegInf = -1.0e30f;

struct StepArgs {
    const float *kv_cur;          // [width]
    float *sc_cur;                // [width] in/out: += bias
    const uint16_t *ape;          // [ratio][width] f16
    const float *norm_w;          // [head_dim]
    float *state_kv, *state_score;   // [rows][width]
    float *emit_out;              // [head_dim], written on emit only
    int head_dim, ratio, pos, n_rot, is_attn, emit;
    float eps;
    RopeDev rope;
};

// Pooled row in `row` (shared) -> RMSNorm -> tail RoPE at comp_pos -> FP8 round trip of the prefix
// (attention path) -> emit_out.  Every thread of the CTA calls this.
struct EmitScratch {
    float warp_sums[8];
    float block_amax[kMaxHeadDim / 64];
    float scale;
    float wmax[kThreads / 32];
};

__device__ __forceinline__ void emit_tail(float *row, EmitScratch &sc, int hd, int n_rot, int comp_pos, int is_attn,
                                          float eps, const float *norm_w, const RopeDev &rope, float *emit_out) {
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    // RMSNorm in the reference's summation order: thread t < 256 takes elements t, t+256, ...
    if (tid < 256) {
        float ss = 0.0f;
        for (int i = tid; i < hd; i += 256) ss = fmaf(row[i], row[i], ss);
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, off);
        if (lane == 0) sc.warp_sums[warp] = ss;
    }
    __syncthreads();
    if (warp == 0) {
        float total = lane < 8 ? sc.warp_sums[lane] : 0.0f;
#pragma unroll
        for (int off = 4; off > 0; off >>= 1) total += __shfl_xor_sync(0xffffffffu, total, off);
        if (lane == 0) sc.scale = 1.0f / sqrtf(total / (float)hd + eps);
    }
    __syncthreads();
    const float scale = sc.scale;
    for (int i = tid; i < hd; i += kThreads) row[i] = row[i] * scale * norm_w[i];
    __syncthreads();

    // tail RoPE at the window's position: thread k rotates pair k
    const int n_nope = hd - n_rot;
    if (tid < n_rot / 2) {
        const float ts = rope_theta_scale(rope, n_rot);
        float te = (float)comp_pos;
        for (int k = 0; k < tid; ++k) te *= ts;
        float c, s;
        rope_cs(rope, tid, te, false, c, s);
        rotate(row[n_nope + 2 * tid], row[n_nope + 2 * tid + 1], c, s);
    }

    // FP8 round trip of the prefix, 64 columns per scale (attention path)
    if (is_attn) {
        for (int base = 0; base < n_nope; base += kThreads) {
            const int i = base + tid;
            float m = i < n_nope ? fabsf(row[i]) : 0.0f;
            m = warp_max(m);
            // a 64-block is two consecutive warps
            if (lane == 0) sc.wmax[warp] = m;
            __syncthreads();
            if (i < n_nope && (i & 63) == 0)
                sc.block_amax[i >> 6] = fmaxf(fmaxf(sc.wmax[warp], sc.wmax[warp + 1]), kFp8AmaxFloor);
            __syncthreads();
            if (i < n_nope) {
                const float s8 = pow2_scale(sc.block_amax[i >> 6]);
                row[i] = e4m3_round_trip(row[i], s8, 1.0f / s8);
            }
        }
    }
    __syncthreads();
    for (int i = tid; i < hd; i += kThreads) emit_out[i] = row[i];
}

__global__ void __launch_bounds__(kThreads) compressor_step_kernel(StepArgs a) {
    __shared__ float row[kMaxHeadDim];
    __shared__ EmitScratch scratch;
    const int tid = threadIdx.x;
    const int hd = a.head_dim, ratio = a.ratio;
    const int coff = ratio == 4 ? 2 : 1, width = coff * hd;
    const int pos_mod = a.pos % ratio;

    // ---- score bias and state row (cuda/compressor.cu:65-90)
    const int state_row = ratio == 4 ? ratio + pos_mod : pos_mod;
    for (int j = tid; j < width; j += kThreads) {
        const float sc = a.sc_cur[j] + f16_bits_to_f32(a.ape[(size_t)pos_mod * width + j]);
        a.state_kv[(size_t)state_row * width + j] = a.kv_cur[j];
        a.state_score[(size_t)state_row * width + j] = sc;
        a.sc_cur[j] = sc;
    }
    if (!a.emit) return;
    __syncthreads();                                   // the new row is read back below

    // ---- pool: one thread per output column, rows in the reference's order
    for (int j = tid; j < hd; j += kThreads) {
        float mx = kNegInf;
        if (ratio == 4) {
            for (int r = 0; r < 4; ++r) {
                mx = fmaxf(mx, a.state_score[(size_t)r * width + j]);
                mx = fmaxf(mx, a.state_score[(size_t)(4 + r) * width + hd + j]);
            }
        } else {
#pragma unroll 8
            for (int r = 0; r < ratio; ++r) mx = fmaxf(mx, a.state_score[(size_t)r * width + j]);
        }
        float pooled = 0.0f;
        if (mx > kNegInf * 0.5f) {
            float denom = 0.0f, sum = 0.0f;
            if (ratio == 4) {
                for (int r = 0; r < 4; ++r) {
                    const float wp = expf(a.state_score[(size_t)r * width + j] - mx);
                    const float wc = expf(a.state_score[(size_t)(4 + r) * width + hd + j] - mx);
                    denom += wp + wc;
                    sum += wp * a.state_kv[(size_t)r * width + j];
                    sum += wc * a.state_kv[(size_t)(4 + r) * width + hd + j];
                }
            } else {
#pragma unroll 8
                for (int r = 0; r < ratio; ++r) {
                    const float w = expf(a.state_score[(size_t)r * width + j] - mx);
                    denom += w;
                    sum += w * a.state_kv[(size_t)r * width + j];
                }
            }
            pooled = denom > 0.0f ? sum / denom : 0.0f;
        }
        row[j] = pooled;
    }
    __syncthreads();

    // ---- state roll for ratio 4 (rows 4-7 become rows 0-3 too); the pool has read the state
    if (ratio == 4) {
        for (int idx = tid; idx < 4 * width; idx += kThreads) {
            a.state_kv[idx] = a.state_kv[4 * width + idx];
            a.state_score[idx] = a.state_score[4 * width + idx];
        }
    }

    emit_tail(row, scratch, hd, a.n_rot, a.pos + 1 - ratio, a.is_attn, a.eps, a.norm_w, a.rope, a.emit_out);
}

// ---- a whole chunk of tokens at once -------------------------------------------------------
// The steps of a chunk depend on each other only through the state, and an emit reads nothing
// but the rows of its own window (ratio 4: plus the window before it).  So for a chunk that
// starts and ends on window boundaries every window gets its own CTA, which reads its rows
// straight from the chunk's projections (score + bias recomputed on the fly: the same single
// f32 add the step performs) instead of going through the state; the first window takes its
// "previous window" from the incoming state.  A second small kernel then leaves the state as
// the last step would have.  Same arithmetic, in the same order, as compressor_step_kernel.
struct ChunkArgs {
    const float *kv_cur, *sc_cur;   // [T][width]
    const uint16_t *ape;            // [ratio][width] f16
    const float *norm_w;
    float *state_kv, *state_score;
    float *emit_out;                // [T / ratio][head_dim]
    int head_dim, ratio, pos0, n_rot, is_attn;
    int64_t n_tokens;
    float eps;
    RopeDev rope;
};

__global__ void __launch_bounds__(kThreads) compressor_chunk_kernel(ChunkArgs a) {
    __shared__ float row[kMaxHeadDim];
    __shared__ EmitScratch scratch;
    const int tid = threadIdx.x;
    const int hd = a.head_dim, ratio = a.ratio;
    const int coff = ratio == 4 ? 2 : 1, width = coff * hd;
    const int64_t e = blockIdx.x, t0 = e * ratio;
    auto score = [&](int64_t t, int r, int col) {     // biased score of token t (r = its place in the window)
        return a.sc_cur[t * width + col] + f16_bits_to_f32(a.ape[(size_t)r * width + col]);
    };
    for (int j = tid; j < hd; j += kThreads) {
        float mx = kNegInf, pooled = 0.0f;
        if (ratio == 4) {
            float sp[4], sc[4], kp[4], kc[4];
#pragma unroll
            for (int r = 0; r < 4; ++r) {
                if (e == 0) {
                    sp[r] = a.state_score[(size_t)r * width + j];
                    kp[r] = a.state_kv[(size_t)r * width + j];
                } else {
                    sp[r] = score(t0 - 4 + r, r, j);
                    kp[r] = a.kv_cur[(t0 - 4 + r) * width + j];
                }
                sc[r] = score(t0 + r, r, hd + j);
                kc[r] = a.kv_cur[(t0 + r) * width + hd + j];
                mx = fmaxf(mx, sp[r]);
                mx = fmaxf(mx, sc[r]);
            }
            if (mx > kNegInf * 0.5f) {
                float denom = 0.0f, sum = 0.0f;
#pragma unroll
                for (int r = 0; r < 4; ++r) {
                    const float wp = expf(sp[r] - mx);
                    const float wc = expf(sc[r] - mx);
                    denom += wp + wc;
                    sum += wp * kp[r];
                    sum += wc * kc[r];
                }
                pooled = denom > 0.0f ? sum / denom : 0.0f;
            }
        } else {
#pragma unroll 8
            for (int r = 0; r < ratio; ++r) mx = fmaxf(mx, score(t0 + r, r, j));
            if (mx > kNegInf * 0.5f) {
                float denom = 0.0f, sum = 0.0f;
#pragma unroll 8
                for (int r = 0; r < ratio; ++r) {
                    const float w = expf(score(t0 + r, r, j) - mx);
                    denom += w;
                    sum += w * a.kv_cur[(t0 + r) * width + j];
                }
                pooled = denom > 0.0f ? sum / denom : 0.0f;
            }
        }
        row[j] = pooled;
    }
    __syncthreads();
    emit_tail(row, scratch, hd, a.n_rot, a.pos0 + (int)t0, a.is_attn, a.eps, a.norm_w, a.rope, a.emit_out + e * hd);
}

// State after the chunk's last step: the last window's rows (ratio 4: in rows 4-7 and, rolled,
// in rows 0-3).
__global__ void compressor_chunk_state_kernel(ChunkArgs a) {
    const int hd = a.head_dim, ratio = a.ratio;
    const int coff = ratio == 4 ? 2 : 1, width = coff * hd;
    const int64_t t0 = a.n_tokens - ratio;
    for (int idx = blockIdx.x * blockDim.x + threadIdx.x; idx < ratio * width; idx += gridDim.x * blockDim.x) {
        const int r = idx / width, col = idx - r * width;
        const float kv = a.kv_cur[(t0 + r) * width + col];
        const float sc = a.sc_cur[(t0 + r) * width + col] + f16_bits_to_f32(a.ape[(size_t)r * width + col]);
        if (ratio == 4) {
            a.state_kv[(size_t)r * width + col] = kv;
            a.state_score[(size_t)r * width + col] = sc;
            a.state_kv[(size_t)(4 + r) * width + col] = kv;
            a.state_score[(size_t)(4 + r) * width + col] = sc;
        } else {
            a.state_kv[(size_t)r * width + col] = kv;
            a.state_score[(size_t)r * width + col] = sc;
        }
    }
}

}  // namespace

bool compressor_step(int is_attn, const float *kv_cur, float *sc_cur, const uint16_t *ape_f16,
                     const float *norm_w, int head_dim, int ratio, int pos, const ds4b200_rope_params &rope,
                     int n_rot, float eps, float *state_kv, float *state_score, float *emit_out,
                     cudaStream_t s) {
    StepArgs a{};
    a.kv_cur = kv_cur; a.sc_cur = sc_cur; a.ape = ape_f16; a.norm_w = norm_w;
    a.state_kv = state_kv; a.state_score = state_score; a.emit_out = emit_out;
    a.head_dim = head_dim; a.ratio = ratio; a.pos = pos; a.n_rot = n_rot; a.is_attn = is_attn;
    a.emit = ((pos + 1) % ratio) == 0;
    a.eps = eps;
    a.rope = to_dev(rope);
    compressor_step_kernel<<<1, kThreads, 0, s>>>(a);
    return a.emit;
}

void compressor_chunk(int is_attn, const float *kv_cur, const float *sc_cur, const uint16_t *ape_f16,
                      const float *norm_w, int head_dim, int ratio, int pos0, int64_t n_tokens,
                      const ds4b200_rope_params &rope, int n_rot, float eps, float *state_kv, float *state_score,
                      float *emit_out, cudaStream_t s) {
    if (n_tokens <= 0) return;
    ChunkArgs a{};
    a.kv_cur = kv_cur; a.sc_cur = sc_cur; a.ape = ape_f16; a.norm_w = norm_w;
    a.state_kv = state_kv; a.state_score = state_score; a.emit_out = emit_out;
    a.head_dim = head_dim; a.ratio = ratio; a.pos0 = pos0; a.n_rot = n_rot; a.is_attn = is_attn;
    a.n_tokens = n_tokens; a.eps = eps;
    a.rope = to_dev(rope);
    compressor_chunk_kernel<<<(unsigned)(n_tokens / ratio), kThreads, 0, s>>>(a);
    const int width = (ratio == 4 ? 2 : 1) * head_dim;
    compressor_chunk_state_kernel<<<(ratio * width + 255) / 256, 256, 0, s>>>(a);
}

}  // namespace ds4b200
