// Programmatic dependent launch for every kernel of the step list.
//
// A step list is a chain of short kernels in one stream; launched the plain way, each kernel's launch
// latency and prologue (index arithmetic, barrier and tensor-memory set-up) start only when the previous
// grid has drained.  With the programmatic-stream-serialisation attribute the next grid is scheduled as
// soon as every CTA of the previous one has called `griddepcontrol.launch_dependents` (or exited), and it
// blocks in `griddepcontrol.wait` until the previous grid has completed and its writes are visible.  Every
// kernel therefore calls `pdl_enter()` before its first access to global memory; kernels with a set-up
// phase that touches no global memory call it after that phase.  The attribute is kept under stream
// capture: the captured graph carries programmatic edges between consecutive kernel nodes.
#pragma once
#include <cuda_runtime.h>

#include <utility>

namespace kn {

__device__ __forceinline__ void pdl_enter() {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
}

template <typename... Params, typename... Args>
inline void launch_pdl(void (*kernel)(Params...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    (void)cudaLaunchKernelEx(&cfg, kernel, Params(std::forward<Args>(args))...);   // a failure stays in cudaGetLastError()
}

}  // namespace kn
