// The activation a contraction's epilogue applies to  accumulator + addends.
#pragma once
#include "../kernels.h"

namespace kn {

__device__ __forceinline__ float apply_activation(float v, int act) {
    if (act == (int)Activation::Relu) return fmaxf(v, 0.0f);
    if (act == (int)Activation::Gelu) return v * 0.5f * (1.0f + erff(v * 0.70710678118654752440f));
    return v;
}

// GELU (erf form) for tensor-core epilogues, whose products carry 10-bit mantissas: erf(x) = 1 - 2^p(|x|) with p a
// degree-7 polynomial fitted to log2(erfc) on [0, 4.3] (weighted for the absolute error of erf: 1.3e-7; of GELU
// 6e-7, at f32 rounding level), |x| clamped there (erfc(4.3) = 1e-9).  Nine arithmetic instructions and ONE
// special-function one per value instead of the ~50 of erff: one epilogue warp per scheduler has to finish a tile's
// 128 x 256 values under the MMAs of the next tile, and the special-function unit (16 results per clock per SM) is
// what a 128 x 256 tile with two of them per value (Abramowitz & Stegun 7.1.26: a reciprocal and an exponential)
// spent 4 100 of its cycles on.
__device__ __forceinline__ float gelu_erf_tensor_core(float v) {
    const float x = v * 0.70710678118654752440f, ax = fminf(fabsf(x), 4.3f);
    float p = fmaf(9.577743185e-05f, ax, -4.308883508e-04f);
    p = fmaf(p, ax, -2.383739920e-03f);
    p = fmaf(p, ax, 2.955816872e-02f);
    p = fmaf(p, ax, -1.490336508e-01f);
    p = fmaf(p, ax, -9.183061123e-01f);
    p = fmaf(p, ax, -1.627916694e+00f);
    p = fmaf(p, ax, 1.044533846e-07f);
    float e;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(p));
    const float half_v = 0.5f * v;
    return fmaf(half_v, copysignf(1.0f - e, x), half_v);
}

}  // namespace kn
