// Host-side helpers shared by the tensor-core kernel files.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>

#include <cstdint>
#include <memory>

#include "../kernels.h"

namespace kn {

// Tiled tensor map over f32 data.  dims / strides innermost first, strides in elements (dims[0] has
// stride 1).  `operand`: 128-byte swizzle and round-to-TF32 on load (an MMA operand tile); otherwise a
// plain f32 tile without swizzle (an epilogue tile).
CUtensorMap tc_make_map(const void* base, int rank, const int64_t* dims, const int64_t* strides, const int* box, bool operand);
// The same for a TF32 operand whose M / N index is the contiguous one (MN-major): the 128-byte swizzle in 32-byte
// pieces, the only shared-memory layout the tensor cores take for such an operand of 32-bit elements.
CUtensorMap tc_make_map_mn_major(const void* base, int rank, const int64_t* dims, const int64_t* strides, const int* box);

// Tiled tensor map for bulk tensor STORES of plain f32 from a 128-byte-swizzled staging tile (inner box
// extent 32 floats).
CUtensorMap tc_make_store_map(const void* base, int rank, const int64_t* dims, const int64_t* strides, const int* box);

// Tiled tensor maps over f16 data (strides in ELEMENTS): an MMA operand tile (128-byte swizzle: inner box extent 64
// halves) when `operand`, else a plain row-major tile without swizzle (an epilogue tile).
CUtensorMap tc_make_map_f16(const void* base, int rank, const int64_t* dims, const int64_t* strides, const int* box, bool operand);

// Persistent matrix multiply (kernels/gemm_persistent.cu): null if the step does not qualify.
// `splits` > 1: K is cut into slices of `k_iters_slice` 32-wide blocks whose partial tiles go to g.scratch.
// `trace_words`: null, or 8 words of pinned host memory for the kernel's progress markers (KN_FLAG_TRACE_GEMM).
std::shared_ptr<void> gemm_persistent_prepare(const GemmParams& g, uint32_t* status_word, int splits, int k_iters_slice,
                                              uint32_t* trace_words = nullptr);
int gemm_persistent_launch(const void* launch, cudaStream_t stream);

// Matmul with a row softmax (attention scores, kernels/attn_softmax.cu): null if the step does not qualify.
bool attn_softmax_fits(int64_t batch, int64_t m, int64_t n, int64_t k);
std::shared_ptr<void> attn_softmax_prepare(const GemmParams& g, uint32_t* status_word);
int attn_softmax_launch(const void* launch, cudaStream_t stream);
// Scores, softmax and probabilities . V in one kernel (kernels/attention.cu): null if the step does not qualify.
bool attention_fits(int64_t batch, int64_t m, int64_t n, int64_t k, int64_t dv);
std::shared_ptr<void> attention_prepare(const GemmParams& g, uint32_t* status_word);
int attention_launch(const void* launch, cudaStream_t stream);

// Convolution chain (kernels/conv_chain.cu): launch data built once the device pointers are known.
std::shared_ptr<void> chain_prepare(const ConvChainParams& c, uint32_t* status_word);
int chain_launch(const void* launch, cudaStream_t stream);

}  // namespace kn
