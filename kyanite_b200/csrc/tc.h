// Tensor-core (tcgen05 / TMEM / TMA) contraction steps: preparation of TMA descriptors once the
// device pointers are known, and launch.
#pragma once
#include "plan.h"

namespace kn {

// Builds the TMA tensor maps of a step marked `tensor_core` (needs the patched device pointers).
// `status_word` is a device word the kernel raises when one of its bounded waits expires.
// `flags`: the plan's kn_options.flags (KN_FLAG_*).  `trace_words`: null, or 8 words of pinned host memory the
// persistent matmul kernel writes progress markers to (KN_FLAG_TRACE_GEMM).
void tc_prepare_step(Step& step, uint32_t* status_word, int flags, uint32_t* trace_words = nullptr);
// Launches a step marked `tensor_core`; returns a cudaError_t as int.
int tc_launch_step(const Step& step, cudaStream_t stream);

// Stores the calling thread's error message (what kn_last_error returns).
void set_last_error(const std::string& message);

// Column-block width the persistent matmul kernel picks for a matrix with n columns (kernels/gemm_persistent.cu).
int gemm_persistent_bn(int64_t n);

// Shapes the fused attention-scores kernel takes (kernels/attn_softmax.cu): pure host arithmetic.
bool attn_softmax_fits(int64_t batch, int64_t m, int64_t n, int64_t k);
bool attention_fits(int64_t batch, int64_t m, int64_t n, int64_t k, int64_t dv);   // (kernels/attention.cu)

// Output tile of the convolution kernel: wb x hb x nb output positions (product 128).
bool tc_conv_tile(int oh, int ow, int* wb, int* hb, int* nb);

// Shared-memory layout of the convolution-chain kernel (kernels/conv_chain.cu).  The images of one CTA
// are stored as one large zero-padded image, `gx` images side by side and `gy` such rows of images below
// one another: a row has `wp = gx * (w + 1)` positions (the position in front of each image row is the
// zero left of it and, being adjacent in memory, the zero right of the image row before it), there are
// `h + 1` rows per row of images (the first is the zero row shared with the images above), and one more
// zero row at the end.  With that, filter tap (r, s) of every output position is the position
// `(r - 1) * wp + (s - 1)` further on, a constant shift of the operand's start address.  Two 8x8 boards
// side by side need 144 accumulator columns (128 of them real pixels), stacked they would need 160.
struct ChainGeometry {
    int per_cta;      // images per CTA = gx * gy
    int gx, gy;
    int wp;           // positions per padded row
    int q_first;      // padded position of output column 0 (the first real pixel)
    int r_first;      // shared-memory row that holds position q_first: q_first rounded up to a multiple of 8, so
                      // that a column's swizzle phase (row & 7) does not depend on the geometry
    int n_mma;        // accumulator columns: padded positions q_first .. q_first + n_mma - 1
    int rows_alloc;   // 128-byte rows per 32-channel block of the activation buffer
    int slots;        // 16 KB filter tiles in flight
    int group;        // filter tiles per request (a whole tap = the layer's channel blocks)
    int smem_bytes;
};
// False if images of this size do not fit (then every layer stays its own step).  `c_blocks` = 32-channel
// blocks of the widest layer.  Pure host arithmetic.
bool tc_chain_geometry(int h, int w, int64_t n_img, int c_blocks, ChainGeometry* out);

}  // namespace kn
