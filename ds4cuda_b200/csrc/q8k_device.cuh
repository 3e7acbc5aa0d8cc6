// q8k_device.cuh — the Q8_K block quantiser as a warp-collective device function, shared by
// the stand-alone quantiser and by the SwiGLU kernel that quantises its own output
// (cuda/moe_iq2_pair.cu:159-235 of the reference: per 256 elements int8 values, one f32 scale,
// 16 partial sums; `max` is the element of largest magnitude, the first one on ties).
#pragma once

#include "device_utils.cuh"

namespace ds4b200 {

__device__ __forceinline__ int q8k_round(float v) {
    const int q = __float2int_rn(v);           // ties to even, like lrintf
    return q > 127 ? 127 : (q < -128 ? -128 : q);
}
__device__ __forceinline__ uint32_t q8k_pack4(int a, int b, int c, int d) {
    return (uint32_t)(a & 0xff) | ((uint32_t)(b & 0xff) << 8) | ((uint32_t)(c & 0xff) << 16) |
           ((uint32_t)(d & 0xff) << 24);
}

// iscale = -127 / max and d = 1 / iscale as the IEEE quotients (cuda/moe_iq2_pair.cu:196-206), branch-free for
// maxima between 1e-30 and 1e30 in magnitude: reciprocal by one Newton step, quotient with an exact residual
// correction (both checked against the plain expressions for every mantissa in that range).
__device__ __forceinline__ void q8k_block_scale(float smax, float &iscale, float &d) {
    const float as = fabsf(smax);
    if (as > 1.0e-30f && as < 1.0e30f) {
        iscale = div_with_rcp(-127.0f, smax, rcp_newton(smax));
        d = rcp_newton(iscale);
    } else {
        iscale = -127.0f / smax;
        d = 1.0f / iscale;
    }
}

// One warp, one block: lane l holds elements 4l..4l+3 in e[0..3] and 128+4l..128+4l+3 in
// e[4..7].  Writes qb[256], *scale_b and sums_b[16].
__device__ __forceinline__ void q8k_block_store(const float (&e)[8], int lane, int8_t *qb, float *scale_b,
                                                int16_t *sums_b) {
    // largest magnitude of the block
    const float a_lo = fmaxf(fmaxf(fabsf(e[0]), fabsf(e[1])), fmaxf(fabsf(e[2]), fabsf(e[3])));
    const float a_hi = fmaxf(fmaxf(fabsf(e[4]), fabsf(e[5])), fmaxf(fabsf(e[6]), fabsf(e[7])));
    float amax = fmaxf(a_lo, a_hi);
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
    if (amax == 0.0f) {
        reinterpret_cast<uint32_t *>(qb)[lane] = 0u;
        reinterpret_cast<uint32_t *>(qb)[32 + lane] = 0u;
        if (lane < 16) sums_b[lane] = 0;
        if (lane == 0) *scale_b = 0.0f;
        return;
    }
    // the first element in index order that has it: elements 4l..4l+3 of every lane come before 128+4l..,
    // so the lowest lane with a hit in its low quad wins, else the lowest lane with one in its high quad
    const unsigned lo_lanes = __ballot_sync(0xffffffffu, a_lo == amax);
    const unsigned hi_lanes = __ballot_sync(0xffffffffu, a_hi == amax);
    const bool in_lo = lo_lanes != 0u;
    const int src = __ffs(in_lo ? lo_lanes : hi_lanes) - 1;
    const float c0 = in_lo ? e[0] : e[4], c1 = in_lo ? e[1] : e[5], c2 = in_lo ? e[2] : e[6], c3 = in_lo ? e[3] : e[7];
    float mine = c3;
    mine = fabsf(c2) == amax ? c2 : mine;
    mine = fabsf(c1) == amax ? c1 : mine;
    mine = fabsf(c0) == amax ? c0 : mine;
    const float smax = __shfl_sync(0xffffffffu, mine, src);
    float iscale, dq;
    q8k_block_scale(smax, iscale, dq);
    const uint32_t p0 = q8_pack4_sat(iscale * e[0], iscale * e[1], iscale * e[2], iscale * e[3]);
    const uint32_t p1 = q8_pack4_sat(iscale * e[4], iscale * e[5], iscale * e[6], iscale * e[7]);
    reinterpret_cast<uint32_t *>(qb)[lane] = p0;
    reinterpret_cast<uint32_t *>(qb)[32 + lane] = p1;
    // 16 consecutive values = 4 consecutive lanes of one half; a lane's four bytes add up in one dp4a
    int s0 = __dp4a((int)p0, 0x01010101, 0), s1 = __dp4a((int)p1, 0x01010101, 0);
    s0 += __shfl_xor_sync(0xffffffffu, s0, 1); s1 += __shfl_xor_sync(0xffffffffu, s1, 1);
    s0 += __shfl_xor_sync(0xffffffffu, s0, 2); s1 += __shfl_xor_sync(0xffffffffu, s1, 2);
    if ((lane & 3) == 0) {
        sums_b[lane >> 2] = (int16_t)s0;
        sums_b[8 + (lane >> 2)] = (int16_t)s1;
    }
    if (lane == 0) *scale_b = dq;
}

}  // namespace ds4b200
