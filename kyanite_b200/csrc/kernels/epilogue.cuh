// The activation a contraction's epilogue applies to  accumulator + addends.
#pragma once
#include "../kernels.h"

namespace kn {

__device__ __forceinline__ float apply_activation(float v, int act) {
    if (act == (int)Activation::Relu) return fmaxf(v, 0.0f);
    if (act == (int)Activation::Gelu) return v * 0.5f * (1.0f + erff(v * 0.70710678118654752440f));
    return v;
}

// GELU (erf form) for tensor-core epilogues, whose products carry 10-bit mantissas: erf by the rational approximation
// of Abramowitz & Stegun 7.1.26 (absolute error <= 1.5e-7; with the approximate reciprocal and exponential about
// 3e-7), 14 arithmetic instructions and two special-function ones instead of the ~50 of erff.  One epilogue warp per
// scheduler has to finish a tile's 128 x 256 elements under the MMAs of the next tile: with erff it did not.
__device__ __forceinline__ float gelu_erf_tensor_core(float v) {
    const float x = v * 0.70710678118654752440f, ax = fabsf(x);
    float t, e;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(t) : "f"(fmaf(0.3275911f, ax, 1.0f)));
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(ax * ax * -1.4426950408889634f));
    float poly = fmaf(t, 1.061405429f, -1.453152027f);
    poly = fmaf(poly, t, 1.421413741f);
    poly = fmaf(poly, t, -0.284496736f);
    poly = fmaf(poly, t, 0.254829592f);
    const float erf_abs = fmaf(-poly * t, e, 1.0f);
    const float half_v = 0.5f * v;
    return fmaf(half_v, copysignf(erf_abs, x), half_v);
}

}  // namespace kn
