// The activation a contraction's epilogue applies to  accumulator + addends.
#pragma once
#include "../kernels.h"

namespace kn {

__device__ __forceinline__ float apply_activation(float v, int act) {
    if (act == (int)Activation::Relu) return fmaxf(v, 0.0f);
    if (act == (int)Activation::Gelu) return v * 0.5f * (1.0f + erff(v * 0.70710678118654752440f));
    return v;
}

}  // namespace kn
