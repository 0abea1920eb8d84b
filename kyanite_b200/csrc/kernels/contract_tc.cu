// placeholder until the tcgen05 kernels land: no step is marked tensor_core yet
#include <cuda_runtime.h>

#include "../tc.h"

namespace kn {

void tc_prepare_step(Step&) { fail(KN_ERR_INTERNAL, "tensor-core step without a tensor-core kernel"); }
int tc_launch_step(const Step&, cudaStream_t) { return (int)cudaErrorNotSupported; }

}  // namespace kn
