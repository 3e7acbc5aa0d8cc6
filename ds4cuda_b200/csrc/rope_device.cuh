// rope_device.cuh — the device side of the tail YaRN RoPE shared by the kernels that
// rotate rows: parameters as plain floats, the (cos, sin) multipliers of one pair
// (cuda/rope.cu:165-200 of the reference, same expression shapes so that nvcc contracts
// the same FMAs), and the 2x2 rotation.
#pragma once

#include "device_utils.cuh"
#include "../../include/ds4b200.h"

namespace ds4b200 {

struct RopeDev {
    float freq_base, theta_scale, freq_scale, ext_factor, attn_factor, corr_low, corr_high;
};

__device__ __forceinline__ float rope_theta_scale(const RopeDev &p, int n_rot) {
    return p.theta_scale > 0.0f ? p.theta_scale : powf(p.freq_base, -2.0f / (float)n_rot);
}

// cos/sin multipliers of tail pair k given theta_extrap for that pair.
__device__ __forceinline__ void rope_cs(const RopeDev &p, int k, float theta_extrap, bool inverse,
                                        float &c, float &s) {
    const float theta_interp = p.freq_scale * theta_extrap;
    float theta = theta_interp;
    float mscale = p.attn_factor;
    if (p.ext_factor != 0.0f) {
        const float y = ((float)k - p.corr_low) / fmaxf(0.001f, p.corr_high - p.corr_low);
        const float ramp_mix = (1.0f - fminf(1.0f, fmaxf(0.0f, y))) * p.ext_factor;
        theta = theta_interp * (1.0f - ramp_mix) + theta_extrap * ramp_mix;
        mscale *= 1.0f + 0.1f * logf(1.0f / p.freq_scale);
    }
    c = cosf(theta) * mscale;
    s = sinf(theta) * mscale;
    if (inverse) s = -s;
}

// x0*c - x1*s and x0*s + x1*c with the roundings spelled out: x0 rounds x1*s and fuses x0*c
// into the subtraction, x1 rounds x0*s and fuses x1*c into the addition.  That is what the
// reference's expressions (cuda/rope.cu:199-200) compile to (checked bit for bit against its
// kernel on the GPU); written with intrinsics the result does not depend on what the
// surrounding code lets the compiler fuse.
__device__ __forceinline__ void rotate(float &x0, float &x1, float c, float s) {
    const float a = x0, b = x1;
    x0 = __fmaf_rn(a, c, -__fmul_rn(b, s));
    x1 = __fmaf_rn(b, c, __fmul_rn(a, s));
}

inline RopeDev to_dev(const ds4b200_rope_params &p) {
    return RopeDev{p.freq_base, p.theta_scale, p.freq_scale, p.ext_factor,
                   p.attn_factor, p.corr_low, p.corr_high};
}

}  // namespace ds4b200
