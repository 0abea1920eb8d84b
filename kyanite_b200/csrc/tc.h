// Tensor-core (tcgen05 / TMEM / TMA) contraction steps: preparation of TMA descriptors once the
// device pointers are known, and launch.
#pragma once
#include "plan.h"

namespace kn {

// Builds the TMA tensor maps of a step marked `tensor_core` (needs the patched device pointers).
void tc_prepare_step(Step& step);
// Launches a step marked `tensor_core`; returns a cudaError_t as int.
int tc_launch_step(const Step& step, cudaStream_t stream);

}  // namespace kn
