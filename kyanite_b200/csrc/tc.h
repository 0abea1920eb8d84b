// Tensor-core (tcgen05 / TMEM / TMA) contraction steps: preparation of TMA descriptors once the
// device pointers are known, and launch.
#pragma once
#include "plan.h"

namespace kn {

// Builds the TMA tensor maps of a step marked `tensor_core` (needs the patched device pointers).
// `status_word` is a device word the kernel raises when one of its bounded waits expires.
void tc_prepare_step(Step& step, uint32_t* status_word);
// Launches a step marked `tensor_core`; returns a cudaError_t as int.
int tc_launch_step(const Step& step, cudaStream_t stream);

// Stores the calling thread's error message (what kn_last_error returns).
void set_last_error(const std::string& message);

// Output tile of the convolution kernel: wb x hb x nb output positions (product 128).
bool tc_conv_tile(int oh, int ow, int* wb, int* hb, int* nb);

}  // namespace kn
