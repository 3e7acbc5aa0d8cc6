// quant.cu — the activation quantisers that sit between the row ops of this library
// and the reference's quantised matvecs: Q8_0 in split form (int8 values + one f32 scale
// per 32 elements, cuda/dense_q8.cu:122-152) and Q8_K (per 256 elements: int8 values, f32
// scale, 16 partial sums, cuda/moe_iq2_pair.cu:159-235).  Integer outputs are bit-exact.
//
// Data movement: 128-bit loads, 32-bit (char4) stores; a Q8_0 block is 8 consecutive
// lanes (3 shuffles), a Q8_K block is one warp holding two float4 per lane.
#include "device_utils.cuh"
#include "kernels.cuh"
#include "q8k_device.cuh"

namespace ds4b200 {
namespace {

__device__ __forceinline__ int q8_round(float v) {
    const int q = __float2int_rn(v);           // ties to even, like lrintf
    return q > 127 ? 127 : (q < -128 ? -128 : q);
}

// n4 float4s, 8 per block.  Every lane of a warp takes part in the shuffles; lanes past
// the end carry zeros and store nothing.
__global__ void quantize_q8_0_kernel(const float *__restrict__ x, int8_t *__restrict__ xq,
                                     float *__restrict__ xscale, int64_t n4) {
    const int64_t rounded = (n4 + 31) & ~(int64_t)31;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < rounded;
         i += (int64_t)gridDim.x * blockDim.x) {
        const float4 v = (i < n4) ? ld_stream4(x + 4 * i) : make_float4(0.f, 0.f, 0.f, 0.f);
        float amax = amax4(v);
#pragma unroll
        for (int off = 4; off > 0; off >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
        float d, id;
        q8_0_block_scale(amax, d, id);
        if (i < n4) {
            reinterpret_cast<uint32_t *>(xq)[i] = q8_pack4_sat(v.x * id, v.y * id, v.z * id, v.w * id);
            if ((i & 7) == 0) xscale[i >> 3] = d;
        }
    }
}

// One warp per NB consecutive 256-element blocks: for each block lane l holds elements 4l..4l+3 and
// 128+4l..128+4l+3.  All 2*NB loads of a lane are issued before the first block is quantised, so a
// thread keeps 32*NB bytes in flight instead of 32.  `max` is the element of largest magnitude, the
// first one in index order on ties.
template <int NB>
__global__ void __launch_bounds__(256)
quantize_q8_K_kernel(const float *__restrict__ x, int8_t *__restrict__ xq, float *__restrict__ xscale,
                     int16_t *__restrict__ xbsums, int64_t n_blocks) {
    const int lane = threadIdx.x & 31;
    const int64_t b0 = ((int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5)) * NB;
    if (b0 >= n_blocks) return;
    float4 v[NB][2];
#pragma unroll
    for (int i = 0; i < NB; ++i) {
        if (b0 + i < n_blocks) {
            const float *xb = x + (b0 + i) * 256;
            v[i][0] = ld_stream4(xb + 4 * lane);
            v[i][1] = ld_stream4(xb + 128 + 4 * lane);
        }
    }
#pragma unroll
    for (int i = 0; i < NB; ++i) {
        const int64_t b = b0 + i;
        if (b >= n_blocks) break;
        const float e[8] = {v[i][0].x, v[i][0].y, v[i][0].z, v[i][0].w, v[i][1].x, v[i][1].y, v[i][1].z, v[i][1].w};
        q8k_block_store(e, lane, xq + b * 256, xscale + b, xbsums + b * 16);
    }
}

// Scalar forms for buffers without 16-byte (input) / 4-byte (output) alignment.
__global__ void quantize_q8_0_scalar_kernel(const float *x, int8_t *xq, float *xscale, int64_t n_blocks) {
    const int lane = threadIdx.x & 31;
    const int64_t b = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (b >= n_blocks) return;
    const float v = x[b * 32 + lane];
    const float d = warp_max(fabsf(v)) / 127.0f;
    const float id = (d != 0.0f) ? 1.0f / d : 0.0f;
    xq[b * 32 + lane] = (int8_t)q8_round(v * id);
    if (lane == 0) xscale[b] = d;
}

}  // namespace

void quantize_q8_0_rows(const float *x, int8_t *xq, float *xscale, int64_t n_blocks, cudaStream_t s) {
    if (n_blocks <= 0) return;
    if (aligned16(x) && (reinterpret_cast<uintptr_t>(xq) & 3u) == 0) {
        const int64_t n4 = n_blocks * 8;
        int64_t blocks = (n4 + 255) / 256;
        if (blocks > 148 * 16) blocks = 148 * 16;
        quantize_q8_0_kernel<<<(unsigned)blocks, 256, 0, s>>>(x, xq, xscale, n4);
    } else {
        quantize_q8_0_scalar_kernel<<<(unsigned)((n_blocks + 7) / 8), 256, 0, s>>>(x, xq, xscale, n_blocks);
    }
}

void quantize_q8_K_rows(const float *x, int8_t *xq, float *xscale, int16_t *xbsums, int64_t n_blocks,
                        cudaStream_t s) {
    if (n_blocks <= 0) return;
    // few blocks: one per warp (more warps); many: four per warp (more bytes in flight per thread)
    if (n_blocks < 148 * 64)
        quantize_q8_K_kernel<1><<<(unsigned)((n_blocks + 7) / 8), 256, 0, s>>>(x, xq, xscale, xbsums, n_blocks);
    else
        quantize_q8_K_kernel<4><<<(unsigned)((n_blocks + 31) / 32), 256, 0, s>>>(x, xq, xscale, xbsums, n_blocks);
}

}  // namespace ds4b200
