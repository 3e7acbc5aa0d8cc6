// norm.cu — RMSNorm over rows (with the residual add before it and the bf16
// cast after it fused in) and the plain f32 add.
//
// Arithmetic follows cuda/norm.cu:52-105 and :126-197 of the reference:
//   ss = sum x^2 (f32), scale = 1/sqrtf(ss/n + eps), y = x*scale*w
// and cuda/elementwise.cu:36-43 (y = a + b).
//
// Data movement: each row is read from HBM once.  A row of up to 8192 floats is
// held in registers between the reduction and the scaling pass — by one warp
// (rows up to 1024 floats: no block barrier at all) or by one CTA.  All global
// traffic is 128-bit, coalesced, with the streaming cache policy.  Rows that are
// not 16-byte aligned, not a multiple of 4 long, or longer than 8192 take a
// scalar two-pass kernel (second pass served by L2).
//
// A row's bits do not depend on how many rows a call has: whichever shape of CTA
// the row count selects, the squares are added in the order of the many-row
// kernel for that row length (rms_norm_cta_kernel).
#include "device_utils.cuh"
#include "kernels.cuh"
#include "q8k_device.cuh"

namespace ds4b200 {
namespace {

struct NormArgs {
    const float *x;
    const float *residual_in;
    const float *w;
    int64_t weight_dim;
    float *y_f32;
    uint16_t *y_bf16;
    float *residual_out;
    int64_t n_rows;
    int n;
    float eps;
    int8_t *xq;        // optional Q8_0 split form of the normalised row (n % 32 == 0)
    float *xscale;     // [n_rows][n / 32]
    int8_t *kq;        // optional Q8_K form of the normalised row (n % 256 == 0, CTA kernel only)
    float *kscale;     // [n_rows][n / 256]
    int16_t *kbsums;   // [n_rows][n / 256][16]
};

__device__ __forceinline__ const float *row_gain(const NormArgs &a, int64_t row) {
    if (a.weight_dim == 0) return nullptr;
    return a.weight_dim == a.n ? a.w : a.w + row * a.n;
}

// Load this thread's float4s of one row (index first + j*stride), add the
// residual, store the sum, return the partial sum of squares.
template <int VPT>
__device__ __forceinline__ float load_row(const NormArgs &a, int64_t row, int first, int stride,
                                          float4 (&v)[VPT]) {
    const int n4 = a.n >> 2;
    const float *xr = a.x + row * a.n;
    const float *rr = a.residual_in ? a.residual_in + row * a.n : nullptr;
    float ss = 0.0f;
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
        const int i = first + j * stride;
        v[j] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (i < n4) v[j] = ld_stream4(xr + 4 * i);
    }
    if (rr) {
#pragma unroll
        for (int j = 0; j < VPT; ++j) {
            const int i = first + j * stride;
            if (i < n4) v[j] = add4(v[j], ld_stream4(rr + 4 * i));
        }
        if (a.residual_out) {
            float *ro = a.residual_out + row * a.n;
#pragma unroll
            for (int j = 0; j < VPT; ++j) {
                const int i = first + j * stride;
                if (i < n4) st_stream4(ro + 4 * i, v[j]);
            }
        }
    }
#pragma unroll
    for (int j = 0; j < VPT; ++j) ss += dot4(v[j]);
    return ss;
}

__device__ __forceinline__ int q8_round(float v) {
    const int q = __float2int_rn(v);
    return q > 127 ? 127 : (q < -128 ? -128 : q);
}

// y = x * scale * w for one float4 of the row
__device__ __forceinline__ float4 normalised4(const float4 &v, float scale, const float *g, int i, bool live) {
    float4 y = make_float4(v.x * scale, v.y * scale, v.z * scale, v.w * scale);
    if (g && live) {
        const float4 w4 = ld_ro4(g + 4 * i);
        y.x *= w4.x; y.y *= w4.y; y.z *= w4.z; y.w *= w4.w;
    }
    return y;
}

template <int VPT>
__device__ __forceinline__ void store_row(const NormArgs &a, int64_t row, int first, int stride,
                                          const float4 (&v)[VPT], float scale) {
    const int n4 = a.n >> 2;
    const float *g = row_gain(a, row);
    float *yf = a.y_f32 ? a.y_f32 + row * a.n : nullptr;
    uint16_t *yb = a.y_bf16 ? a.y_bf16 + row * a.n : nullptr;
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
        const int i = first + j * stride;
        const bool live = i < n4;
        const float4 y = normalised4(v[j], scale, g, i, live);
        if (live && yf) st_stream4(yf + 4 * i, y);
        if (live && yb) st_bf16x4(yb + 4 * i, y);
        if (a.xq) {
            // Q8_0 activation quantiser of the matvec that consumes this row
            // (cuda/dense_q8.cu:122-152): 32 elements = 8 consecutive lanes.  n % 32 == 0, so
            // a group of 8 lanes is live or dead as a whole; dead lanes only feed the shuffles.
            float amax = live ? amax4(y) : 0.0f;
#pragma unroll
            for (int off = 4; off > 0; off >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
            float d, id;
            q8_0_block_scale(amax, d, id);
            if (live) {
                reinterpret_cast<uint32_t *>(a.xq + row * a.n)[i] = q8_pack4_sat(y.x * id, y.y * id, y.z * id, y.w * id);
                if ((i & 7) == 0) a.xscale[row * (a.n >> 5) + (i >> 3)] = d;
            }
        }
    }
}

// The normalised row as the Q8_K blocks the routed experts' gate / up dots read (the reference quantises the
// row inside that launcher, cuda/moe_iq2_pair.cu:159-235).  A block of 256 values is held by 64 consecutive
// threads, two warps (blockDim is a multiple of 64 and so is n / 4): each warp finds the element of largest
// magnitude of its half, the first one on ties, the halves meet in shared memory, and the lower half wins a
// tie between them, as index order has it.
template <int VPT>
__device__ __forceinline__ void q8_K_half_maxima(const NormArgs &a, int64_t row, const float4 (&v)[VPT], float scale,
                                                 float4 (&y)[VPT], float2 (*half_max)[32]) {
    const int n4 = a.n >> 2;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const float *g = row_gain(a, row);
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
        const int i = threadIdx.x + j * blockDim.x;
        const bool live = i < n4;                       // a warp is live or dead as a whole
        y[j] = normalised4(v[j], scale, g, i, live);
        const float mine_a = live ? amax4(y[j]) : 0.0f;
        float amax = mine_a;
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
        const unsigned hits = __ballot_sync(0xffffffffu, mine_a == amax);
        float mine = y[j].w;
        mine = fabsf(y[j].z) == amax ? y[j].z : mine;
        mine = fabsf(y[j].y) == amax ? y[j].y : mine;
        mine = fabsf(y[j].x) == amax ? y[j].x : mine;
        const float smax = __shfl_sync(0xffffffffu, mine, __ffs(hits) - 1);
        if (lane == 0) half_max[j][warp] = make_float2(amax, smax);
    }
}

template <int VPT>
__device__ __forceinline__ void store_row_q8_K(const NormArgs &a, int64_t row, const float4 (&y)[VPT],
                                               float2 (*half_max)[32]) {
    const int n4 = a.n >> 2;
    const int warp = threadIdx.x >> 5;
    __syncthreads();
    const int blocks_per_row = a.n >> 8;
    // lane j works out the scale of the warp pair's block j (an all-zero block keeps 0, 0); the others
    // read it by shuffle
    const int lane = threadIdx.x & 31;
    float lane_iscale = 0.0f, lane_dq = 0.0f;
    if (lane < VPT) {
        const float2 lo = half_max[lane][warp & ~1], hi = half_max[lane][warp | 1];
        const float amax = fmaxf(lo.x, hi.x);
        if (amax != 0.0f) q8k_block_scale(lo.x == amax ? lo.y : hi.y, lane_iscale, lane_dq);
    }
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
        const int i = threadIdx.x + j * blockDim.x;
        const float iscale = __shfl_sync(0xffffffffu, lane_iscale, j);
        const float dq = __shfl_sync(0xffffffffu, lane_dq, j);
        if (i >= n4) continue;
        const int64_t blk = row * blocks_per_row + (i >> 6);
        const uint32_t packed = q8_pack4_sat(iscale * y[j].x, iscale * y[j].y, iscale * y[j].z, iscale * y[j].w);
        reinterpret_cast<uint32_t *>(a.kq + row * a.n)[i] = packed;
        int sum = __dp4a((int)packed, 0x01010101, 0);   // 16 consecutive values = 4 consecutive lanes
        sum += __shfl_xor_sync(0xffffffffu, sum, 1);
        sum += __shfl_xor_sync(0xffffffffu, sum, 2);
        if ((i & 3) == 0) a.kbsums[blk * 16 + ((i & 63) >> 2)] = (int16_t)sum;
        if ((i & 63) == 0) a.kscale[blk] = dq;
    }
}

// One CTA per row; the row lives in VPT float4 registers per thread.
template <int VPT, bool Q8K>
__global__ void rms_norm_cta_kernel(NormArgs a) {
    __shared__ float red[33];
    __shared__ float sq[2048];                 // squares per float4 of the row (rows of up to 8192 floats)
    __shared__ float2 half_max[Q8K ? VPT : 1][32];
    const int64_t row = blockIdx.x;
    float4 v[VPT];
    float ss = load_row<VPT>(a, row, threadIdx.x, blockDim.x, v);
    const int n4 = a.n >> 2;
    if (blockDim.x == 256 && n4 > 256) {
        // one barrier instead of three: every thread adds the eight warp sums itself, in the order the
        // butterfly of block_sum adds them (same bits)
        ss = warp_sum(ss);
        if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
        __syncthreads();
    } else {
        // Any other shape of CTA adds the row up in the order of the kernel that many rows of this length
        // get, so that a row's bits do not depend on how many rows the call has: rows of up to 1024 floats
        // as one warp does (lane l takes float4 l, l + 32, ... in turn, then the butterfly), longer ones as
        // 256 threads do (thread t takes float4 t, t + 256, ..., butterflies, the eight warp sums below).
#pragma unroll
        for (int j = 0; j < VPT; ++j) {
            const int i = threadIdx.x + j * blockDim.x;
            if (i < n4) sq[i] = dot4(v[j]);
        }
        __syncthreads();
        const int takers = n4 <= 256 ? 32 : 256;
        if (threadIdx.x < takers) {
            float part = 0.0f;
            for (int i = threadIdx.x; i < n4; i += takers) part += sq[i];
            part = warp_sum(part);
            if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = part;
        }
        __syncthreads();
    }
    ss = n4 <= 256 ? red[0]
                   : __fadd_rn(__fadd_rn(__fadd_rn(red[0], red[4]), __fadd_rn(red[2], red[6])),
                               __fadd_rn(__fadd_rn(red[1], red[5]), __fadd_rn(red[3], red[7])));
    const float scale = rms_scale(ss, (float)a.n, a.eps);
    if (Q8K) {
        float4 y[VPT];
        store_row<VPT>(a, row, threadIdx.x, blockDim.x, v, scale);
        q8_K_half_maxima<VPT>(a, row, v, scale, y, half_max);
        store_row_q8_K<VPT>(a, row, y, half_max);
    } else {
        store_row<VPT>(a, row, threadIdx.x, blockDim.x, v, scale);
    }
}

// One warp per row (rows up to 1024 floats): shuffle reduction only.
template <int VPT>
__global__ void rms_norm_warp_kernel(NormArgs a) {
    const int lane = threadIdx.x & 31;
    const int64_t row = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= a.n_rows) return;
    float4 v[VPT];
    float ss = load_row<VPT>(a, row, lane, 32, v);
    ss = warp_sum(ss);
    const float scale = rms_scale(ss, (float)a.n, a.eps);
    store_row<VPT>(a, row, lane, 32, v, scale);
}

// Any n, any natural alignment: scalar loads, two passes over the row.  When a
// residual is added without residual_out the second pass repeats the add.
__global__ void rms_norm_scalar_kernel(NormArgs a) {
    __shared__ float red[33];
    const int64_t row = blockIdx.x;
    const float *xr = a.x + row * a.n;
    const float *rr = a.residual_in ? a.residual_in + row * a.n : nullptr;
    float *ro = (rr && a.residual_out) ? a.residual_out + row * a.n : nullptr;
    float ss = 0.0f;
    for (int i = threadIdx.x; i < a.n; i += blockDim.x) {
        float v = xr[i];
        if (rr) v += rr[i];
        if (ro) ro[i] = v;
        ss += v * v;
    }
    ss = block_sum(ss, red);
    const float scale = rms_scale(ss, (float)a.n, a.eps);
    const float *g = row_gain(a, row);
    for (int i = threadIdx.x; i < a.n; i += blockDim.x) {
        float v = xr[i];
        if (rr) v += rr[i];
        float y = v * scale;
        if (g) y *= g[i];
        if (a.y_f32) a.y_f32[row * a.n + i] = y;
        if (a.y_bf16) a.y_bf16[row * a.n + i] = bf16_bits(y);
    }
}

__global__ void add_vec_kernel(const float *__restrict__ a, const float *__restrict__ b,
                               float *__restrict__ y, int64_t n4) {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4;
         i += (int64_t)gridDim.x * blockDim.x)
        st_stream4(y + 4 * i, add4(ld_stream4(a + 4 * i), ld_stream4(b + 4 * i)));
}
__global__ void add_scalar_kernel(const float *__restrict__ a, const float *__restrict__ b,
                                  float *__restrict__ y, int64_t n) {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n;
         i += (int64_t)gridDim.x * blockDim.x)
        y[i] = a[i] + b[i];
}

// one decode row: no loop, 32-bit index
__global__ void add_row_kernel(const float *__restrict__ a, const float *__restrict__ b, float *__restrict__ y, int n) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) y[i] = a[i] + b[i];
}

template <int VPT>
void launch_cta(const NormArgs &a, int threads, cudaStream_t s) {
    if (a.kq) rms_norm_cta_kernel<VPT, true><<<(unsigned)a.n_rows, threads, 0, s>>>(a);
    else rms_norm_cta_kernel<VPT, false><<<(unsigned)a.n_rows, threads, 0, s>>>(a);
}
template <int VPT>
void launch_warp(const NormArgs &a, cudaStream_t s) {
    constexpr int kRowsPerCta = 8;
    const unsigned grid = (unsigned)((a.n_rows + kRowsPerCta - 1) / kRowsPerCta);
    rms_norm_warp_kernel<VPT><<<grid, kRowsPerCta * 32, 0, s>>>(a);
}

}  // namespace

void add_f32(const float *a, const float *b, float *y, int64_t n, cudaStream_t s) {
    if (n <= 0) return;
    constexpr int kThreads = 256;
    if (n <= 8192) {
        // one decode row is latency-bound: one element per thread over many small CTAs finishes sooner than
        // four per thread over a few
        add_row_kernel<<<(unsigned)((n + 255) / 256), 256, 0, s>>>(a, b, y, (int)n);
        return;
    }
    if (aligned16(a) && aligned16(b) && aligned16(y) && (n & 3) == 0) {
        const int64_t n4 = n >> 2;
        const int64_t blocks = (n4 + kThreads - 1) / kThreads;
        add_vec_kernel<<<(unsigned)(blocks < 148 * 16 ? blocks : 148 * 16), kThreads, 0, s>>>(a, b, y, n4);
    } else {
        const int64_t blocks = (n + kThreads - 1) / kThreads;
        add_scalar_kernel<<<(unsigned)(blocks < 148 * 16 ? blocks : 148 * 16), kThreads, 0, s>>>(a, b, y, n);
    }
}

void rms_norm_rows(const float *x, const float *residual_in, const float *w, int64_t weight_dim,
                   float *y_f32, uint16_t *y_bf16, float *residual_out, int64_t n_rows, int n,
                   float eps, cudaStream_t s, int8_t *xq, float *xscale, int8_t *kq, float *kscale,
                   int16_t *kbsums) {
    if (n_rows <= 0 || n <= 0) return;
    const NormArgs a{x, residual_in, w, weight_dim, y_f32, y_bf16, residual_out, n_rows, n, eps, xq, xscale,
                     kq, kscale, kbsums};
    const bool vec = (n & 3) == 0 && n <= 8192 && aligned16(x) && aligned16(residual_in) &&
                     aligned16(w) && aligned16(y_f32) && aligned8(y_bf16) &&
                     aligned16(residual_out);
    if (!vec) {
        rms_norm_scalar_kernel<<<(unsigned)n_rows, 256, 0, s>>>(a);
        return;
    }
    const int n4 = n >> 2;
    if (n4 <= 256 && n_rows >= 64 && !kq) {    // warp per row
        const int vpt = (n4 + 31) / 32;
        if (vpt <= 1) launch_warp<1>(a, s);
        else if (vpt <= 2) launch_warp<2>(a, s);
        else if (vpt <= 4) launch_warp<4>(a, s);
        else launch_warp<8>(a, s);
        return;
    }
    // CTA per row.  A handful of rows: as many threads as float4s (one load
    // per thread, shortest dependency chain).  Many rows: 256 threads so that
    // several CTAs share an SM.
    int threads = 256;
    if (n_rows < 296) {
        threads = ((n4 + 31) / 32) * 32;
        if (threads > 1024) threads = 1024;
        if (threads < 32) threads = 32;
    }
    const int vpt = (n4 + threads - 1) / threads;
    if (vpt <= 1) launch_cta<1>(a, threads, s);
    else if (vpt <= 2) launch_cta<2>(a, threads, s);
    else if (vpt <= 4) launch_cta<4>(a, threads, s);
    else launch_cta<8>(a, threads, s);
}

}  // namespace ds4b200
