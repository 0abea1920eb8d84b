// Launch-parameter blocks of the executor's kernels and their host launchers.
//
// A parameter block is plain data: the planner fills it without touching CUDA, the executor patches
// the device pointers in once the arena exists, and the launcher passes it by value as a
// `__grid_constant__` kernel argument (so it is also baked into a captured CUDA graph node).
// Strides are in elements and may be zero or negative.  Every tensor of rank > KN_DEV_MAX_RANK
// after axis merging is rejected by the planner.
#pragma once
#include <cstdint>

#include "common.h"

struct CUstream_st;
typedef CUstream_st* cudaStream_t;

namespace kn {

constexpr int DEV_MAX_RANK = 8;
constexpr int SCALAR_MAX_OPERANDS = 10;
constexpr int SCALAR_MAX_INSTR = 40;

// Gelu is the exact form  x * 0.5 * (1 + erf(x / sqrt(2)))
enum class Activation : int32_t { None = 0, Relu = 1, Gelu = 2 };

// ---- fused elementwise ("scalar") kernel: replaces kn-cuda-eval/src/autokernel/scalar.{rs,cu}.
// The body is a small register program instead of generated C source: slot i < n_loads holds the
// element loaded from operand load_operand[i]; instruction k writes slot n_loads + k.
struct ScalarInstr {
    uint8_t kind;    // 0 = constant, 1 = unary, 2 = binary
    uint8_t op;      // UnaryOp / BinaryOp
    uint8_t dtype;   // result dtype
    uint8_t from;    // operand dtype (differs from `dtype` only for casts)
    uint8_t a, b;    // operand slots
    uint16_t pad;
    uint64_t imm;    // constant: canonical element pattern
};

struct ScalarParams {
    int32_t rank, n_operands, n_loads, n_instr, n_stores;
    int32_t vec4;    // 1: every operand is f32 with innermost stride 1 (or 0) and 16-byte aligned rows; 2: the same as an
                     // accumulator program (below); 3: operands and values are f16 or f32, innermost stride 1 (or 0),
                     // 16-byte aligned rows, eight elements per access; 4: the same as an accumulator program; 5: an
                     // accumulator program whose operands and values are all f16 (runs on packed halves)
    int64_t total;   // element count
    int64_t dims[DEV_MAX_RANK];
    void* ptr[SCALAR_MAX_OPERANDS];
    int64_t strides[SCALAR_MAX_OPERANDS][DEV_MAX_RANK];
    uint8_t dtype[SCALAR_MAX_OPERANDS];
    uint8_t load_operand[SCALAR_MAX_OPERANDS];
    uint8_t store_operand[SCALAR_MAX_OPERANDS];
    uint8_t store_slot[SCALAR_MAX_OPERANDS];
    ScalarInstr instr[SCALAR_MAX_INSTR];
    // vec4 == 2: the same program as an accumulator program (built by the planner's allocate_registers, which
    // documents the micro-op format); `n_regs` = number of spill slots it uses (0..8).
    int32_t n_micro, n_regs;
    ScalarInstr micro[SCALAR_MAX_INSTR + 2 * SCALAR_MAX_OPERANDS];
};

// ---- reduce: replaces autokernel/reduce.{rs,cu}
struct ReduceParams {
    const void* in;
    void* out;
    uint8_t dtype, op;       // DType, ReduceOp
    int32_t kept_rank, red_rank;
    int64_t n_out, n_red;
    int64_t kept_dims[DEV_MAX_RANK], kept_in_strides[DEV_MAX_RANK], kept_out_strides[DEV_MAX_RANK];
    int64_t red_dims[DEV_MAX_RANK], red_strides[DEV_MAX_RANK];
    float mean_scale;        // Mean: the divisor, n_red as float (sum / count like the CPU path)
};

// ---- softmax / layernorm over one axis: replace autokernel/{softmax,layernorm}.{rs,cu}
struct RowParams {
    const float* in0;
    const float* in1;        // may be null.  layernorm: second input, same strides as in0.
                             // softmax: additive term (an attention mask) with strides of its own
    float* out;
    int32_t outer_rank;
    int64_t rows, len;
    int64_t outer_dims[DEV_MAX_RANK], in_strides[DEV_MAX_RANK], out_strides[DEV_MAX_RANK];
    int64_t in_axis_stride, out_axis_stride;
    int64_t in1_strides[DEV_MAX_RANK], in1_axis_stride;   // softmax only
    float scale;             // softmax: x = scale * in0 + in1
    float alpha0, alpha1;    // layernorm: x = alpha0 * in0 + alpha1 * in1
    float eps;
    int32_t half;            // 1: in0, in1 and out hold f16 elements (the pointers are reinterpreted); the
                             // statistics and the arithmetic stay f32, the result is rounded to f16 once
};

// ---- root-mean-square norm over the innermost axis:  out = x / sqrt(mean(x^2) + eps) * gain.  The IR has no such
// operation; the planner recognises the pow / mean / sqrt / div / mul subgraph (with the value casts around it in
// half-storage graphs) and this one kernel takes the place of five elementwise and reduce steps.
struct RmsNormParams {
    const void* in;          // [rows, len], rows `in_row_stride` elements apart, f32 or f16
    void* out;               // [rows, len] dense, f32 or f16
    const float* gain;       // [len] f32 with element stride `gain_stride`, or null
    int64_t rows, len, in_row_stride, out_row_stride, gain_stride;
    float eps;
    int32_t in_half, out_half;
};

// ---- gather along one axis with rank-1 indices: replaces autokernel/gather.{rs,cu}
struct GatherParams {
    const void* in;
    const void* idx;
    void* out;
    int32_t rank, axis, elem_size;
    uint8_t idx_dtype;
    int64_t total;           // output elements
    int64_t axis_in_size;    // valid index range; anything else writes 0
    int64_t idx_stride;
    int64_t out_dims[DEV_MAX_RANK], in_strides[DEV_MAX_RANK], out_strides[DEV_MAX_RANK];
};

// An operand of a matmul that is a head split or head merge of another tensor (attention): instead of a [batch, rows, k]
// matrix in memory it is a 4-D tensor (k', rows', x, y) with element strides, of which the operand tile at
// (K offset k0, row offset r0, batch entry bt) starts at coordinates
//     (k0 % kd,  r0 % rd,  k0 / kd + bt % bi,  r0 / rd + bt / bi).
// Head split ([B*S, H*D] read as [B*H, S, D]): dims (D, S, H, B), kd = K = D, rd = rows = S, bi = H.
// Head merge ([B*H, S, D] read as [B*S, H*D]): dims (D, S, H, B), kd = D, rd = S, bi = 1 (one batch entry).
// Persistent tensor-core kernel only; `sa` / `sb` are not used for such an operand.
struct GemmOperand4D {
    int32_t enabled;
    int32_t kd, rd, bi;
    int64_t dims[4], strides[4];
};

// ---- batched matrix multiply with fused epilogue  C = act(A.B + add1 + add2)
// replaces cublasSgemmStridedBatched (kn-cuda-sys/src/wrapper/group.rs:120-171) plus the scalar
// kernel that followed it for bias / activation.
struct GemmParams {
    const float* a;
    const float* b;
    float* c;
    const float* add1;       // optional addends with their own (broadcastable) strides
    const float* add2;
    int64_t batch, m, n, k;
    int64_t sa[3], sb[3], sc[3], s1[3], s2[3];   // (batch, row, col) strides
    int32_t act;
    int32_t round_tf32;      // round outputs to TF32 (they only feed tensor-core contractions)
    // tensor-core path only: K is cut into `splits` slices whose partial tiles go to `scratch`
    // ([batch][slice][m][n] f32) and are summed by a second kernel; 1 = no split
    int32_t splits;
    float* scratch;
    int32_t half;            // 1: A, B, C and the addends hold f16 elements (the pointers are reinterpreted); products
                             // accumulate in f32 and the result is rounded to f16 once.  `scratch` stays f32.
    // Implicit convolution operand (persistent tensor-core kernel only, f32 storage).  0: none.  1 / 2: the A / B
    // operand is not a matrix in memory: `a` / `b` points to a channels-last image tensor [batch][h][w][c] and row
    // `oy * conv_ow + ox` of batch entry `n` is the window of output position (oy, ox) of image n, K index
    // (tap_y * conv_s + tap_x) * conv_c + channel, zeros outside the image (stride-1 convolution as a matmul
    // without materialising the windows).  `sa` / `sb` are not used for that operand.
    GemmOperand4D a4, b4;    // head split / merge read in place (above)
    // Row softmax fused into the matmul (attention scores): C = softmax over each row of (softmax_scale * A.B), rows of
    // at most 512 columns, no addends, no activation (kernels/attn_softmax.cu; tensor cores only).
    // 2: the step goes on to C = softmax(...) . V without writing the probabilities: `values` is V^T, [batch][values_cols][n]
    // with element strides `values_strides` (the last is 1), C is [batch][m][values_cols] (kernels/attention.cu).
    int32_t row_softmax;
    float softmax_scale;
    // `values_mn`: `values` is V itself, [batch][n][values_cols] with the columns contiguous (strides as above), or, with
    // `v4`, a head split read in place (rows = keys, K = columns).
    const float* values;
    int64_t values_strides[3];
    int64_t values_cols;
    int32_t values_mn;
    GemmOperand4D v4;
    int32_t conv_operand;
    int32_t conv_c, conv_h, conv_w, conv_ow, conv_r, conv_s, conv_pad_y, conv_pad_x;
    int64_t conv_strides[3];   // element strides of the image tensor: image, row, pixel (channels are contiguous)
};

// ---- 2D convolution (cross-correlation, zero padding) with fused epilogue
// out = act(conv(in, filter) + add1 + add2); replaces cudnnConvolutionBiasActivationForward
// (kn-cuda-sys/src/wrapper/operation.rs:162-240).
struct ConvParams {
    const float* in;
    const float* filter;
    float* out;
    const float* add1;
    const float* add2;
    int32_t n, c, h, w, k, r, s, oh, ow, stride_y, stride_x, pad_y, pad_x;
    int64_t s_in[4], s_f[4], s_out[4], s1[4], s2[4];
    int32_t act;
    int32_t round_tf32;
};

// ---- a run of stride-1 3x3 same-padding convolutions executed by ONE kernel, activations resident
// in shared memory: layer l computes  act_l(conv(x_l, filter_l) + bias_l [+ held])  where x_0 = `in`,
// x_{l+1} = the layer's result and `held` is `in` or the last result flagged to be held (the skip
// connection of a residual block).  Results reach global memory only where a layer is flagged to store,
// and through the heads of the optional pointwise last layer.
constexpr int kMaxChainLayers = 64;
constexpr int kChainFlagRelu = 1, kChainFlagAddHeld = 2, kChainFlagHold = 4;
constexpr int kChainFlagStore = 8;       // the layer's result is written to `out` (always set on the last 3x3 layer
                                         // unless nothing outside the chain reads it)
constexpr int kChainFlagPointwise = 16;  // a 1x1 layer: one tap, c_blocks tiles
constexpr int kMaxChainHeads = 4;
struct ConvChainParams {
    const float* in;      // [n, c_in, h, w], any strides
    float* out;           // [n, k, h, w], any strides
    const float* tiles;   // filter tiles [tile][128 output channels][32 input channels] in the 128-byte-swizzled
                          // order of shared memory, TF32, layers back to back;
                          // within a layer tile = tap * c_blocks + channel block, tap = r * 3 + s
    const float* bias;    // [layer][128]
    int32_t n, c_in, k, h, w;
    int32_t n_layers;
    int64_t s_in[4], s_out[4];
    uint8_t flags[kMaxChainLayers];
    uint8_t c_blocks[kMaxChainLayers];   // 32-channel blocks of the layer's input
    // Heads: when n_heads > 0 the last layer is a pointwise layer whose output channels are several 1x1
    // convolutions of the last 3x3 result side by side (a policy and a value head, say); head i owns
    // channels [head_begin[i], head_begin[i + 1]) and has its own output tensor [n, channels, h, w].
    int32_t n_heads;
    int32_t head_begin[kMaxChainHeads + 1];
    float* head_out[kMaxChainHeads];
    int64_t head_s_out[kMaxChainHeads][4];
    uint8_t head_relu[kMaxChainHeads];
};

// ---- im2col for a convolution that runs as a matmul: col[n][oy*OW + ox][tap][c] = in[n][c][oy*sy + r - py][ox*sx + s - px]
// (tap = r * S + s), zero outside the image and for the padding channels c >= C up to c_pad.
struct Im2colParams {
    const float* in;     // [N, C, H, W], any strides
    float* col;          // [N, OH*OW, R*S, c_pad], dense
    int32_t n, c, h, w, r, s, oh, ow, stride_y, stride_x, pad_y, pad_x, c_pad;
    int64_t s_in[4];
};

// ---- sum of a dense tensor over the ranks of the executor's communicator (tensor-parallel graphs); no kernel of
// this library: the executor hands the buffers to ncclAllReduce on its stream, or copies in -> out without one
struct AllReduceParams {
    const void* in;
    void* out;
    int64_t count;     // elements
    uint8_t dtype;     // DType: F32 or F16
};

// All launchers enqueue on `stream` and return the cudaError_t of the launch as int.
int launch_scalar(const ScalarParams& p, cudaStream_t stream);
int launch_reduce(const ReduceParams& p, cudaStream_t stream);
int launch_softmax(const RowParams& p, cudaStream_t stream);      // dispatches on p.half
int launch_layernorm(const RowParams& p, cudaStream_t stream);
int launch_rmsnorm(const RmsNormParams& p, cudaStream_t stream);  // kernels/rows_f16.cu
int launch_softmax_f16(const RowParams& p, cudaStream_t stream);  // kernels/rows_f16.cu
int launch_layernorm_f16(const RowParams& p, cudaStream_t stream);
int launch_gather(const GatherParams& p, cudaStream_t stream);
int launch_im2col(const Im2colParams& p, cudaStream_t stream);
int launch_gemm_simt(const GemmParams& p, cudaStream_t stream);
int launch_conv_simt(const ConvParams& p, cudaStream_t stream);

}  // namespace kn
