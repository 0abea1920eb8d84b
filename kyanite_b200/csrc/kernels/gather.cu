// Gather along one axis with rank-1 indices of any integer type:
//   out[..., j, ...] = in[..., idx[j], ...]
// Elements move as raw 1/2/4/8-byte words, so the result is bit-exact for every dtype.  An index
// outside [0, axis size) writes zero, like the reference's `gather_kernel`
// (kn-cuda-eval/src/autokernel/gather.cu:46-49); its CPU path rejects such indices instead.
#include <cuda_runtime.h>

#include "../kernels.h"
#include "../scalar_ops.h"
#include "launch.cuh"

namespace kn {

namespace {

template <typename W>
__global__ void __launch_bounds__(256) gather_kernel(const __grid_constant__ GatherParams p) {
    pdl_enter();
    const int64_t step = (int64_t)gridDim.x * blockDim.x;
    for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < p.total; idx += step) {
        int64_t rem = idx, in_off = 0, out_off = 0;
        bool valid = true;
        for (int d = p.rank - 1; d >= 0; d--) {
            const int64_t dim = p.out_dims[d];
            const int64_t q = rem / dim;
            int64_t i = rem - q * dim;
            rem = q;
            out_off += i * p.out_strides[d];
            if (d == p.axis) {
                const uint64_t raw = load_bits(p.idx, (DType)p.idx_dtype, i * p.idx_stride);
                // signed types arrive sign-extended, so a negative index is a huge unsigned value
                valid = raw < (uint64_t)p.axis_in_size;
                i = valid ? (int64_t)raw : 0;
            }
            in_off += i * p.in_strides[d];
        }
        W v = valid ? ((const W*)p.in)[in_off] : W(0);
        ((W*)p.out)[out_off] = v;
    }
}

// Row gather (an embedding lookup): everything behind the gathered axis is one contiguous run of at
// least 16 bytes in both tensors.  One warp per output row: the index is read once, the row moves as
// 128-bit words.  `rows` = product of the extents up to and including the axis.
__global__ void __launch_bounds__(256) gather_rows_kernel(const __grid_constant__ GatherParams p, int64_t rows, int row_vec4) {
    pdl_enter();
    const int lane = threadIdx.x & 31;
    const int64_t warps = (int64_t)gridDim.x * (blockDim.x >> 5);
    // where a row comes from and goes to (the index load and the divisions are a dependent chain of their
    // own, so the next row's are resolved while the current row moves)
    auto locate = [&](int64_t row, int64_t& in_off, int64_t& out_off, bool& valid) {
        int64_t rem = row;
        in_off = 0;
        out_off = 0;
        valid = true;
        for (int d = p.axis; d >= 0; d--) {
            const int64_t dim = p.out_dims[d];
            const int64_t q = rem / dim;
            int64_t i = rem - q * dim;
            rem = q;
            out_off += i * p.out_strides[d];
            if (d == p.axis) {
                const uint64_t raw = load_bits(p.idx, (DType)p.idx_dtype, i * p.idx_stride);
                valid = raw < (uint64_t)p.axis_in_size;
                i = valid ? (int64_t)raw : 0;
            }
            in_off += i * p.in_strides[d];
        }
    };
    int64_t row = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= rows) return;
    int64_t in_off, out_off;
    bool valid;
    locate(row, in_off, out_off, valid);
    const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
    while (true) {
        const int64_t next = row + warps;
        int64_t n_in = 0, n_out = 0;
        bool n_valid = false;
        if (next < rows) locate(next, n_in, n_out, n_valid);
        const uint4* src = (const uint4*)((const char*)p.in + in_off * p.elem_size);
        uint4* dst = (uint4*)((char*)p.out + out_off * p.elem_size);
        // four 128-bit loads per lane in flight before the first store
        for (int e0 = lane; e0 < row_vec4; e0 += 128) {
            uint4 r[4];
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const int e = e0 + 32 * j;
                r[j] = (valid && e < row_vec4) ? __ldg(src + e) : zero;
            }
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const int e = e0 + 32 * j;
                if (e < row_vec4) __stcs(dst + e, r[j]);   // streaming store: the table, not the output, should stay in L2
            }
        }
        if (next >= rows) break;
        row = next;
        in_off = n_in;
        out_off = n_out;
        valid = n_valid;
    }
}

}  // namespace

int launch_gather(const GatherParams& p, cudaStream_t stream) {
    if (p.total == 0) return 0;
    {
        // dense tail behind the axis?
        int64_t inner = 1;
        bool dense = true;
        for (int d = p.rank - 1; d > p.axis; d--) {
            dense = dense && p.in_strides[d] == inner && p.out_strides[d] == inner;
            inner *= p.out_dims[d];
        }
        const int64_t row_bytes = inner * p.elem_size;
        dense = dense && row_bytes >= 64 && row_bytes % 16 == 0 && row_bytes / 16 < (1 << 30) && ((uintptr_t)p.in & 15) == 0 &&
                ((uintptr_t)p.out & 15) == 0;
        for (int d = 0; d <= p.axis && dense; d++)
            dense = (p.in_strides[d] * p.elem_size) % 16 == 0 && (p.out_strides[d] * p.elem_size) % 16 == 0;
        if (dense) {
            const int64_t rows = p.total / inner;
            int64_t blocks = (rows + 7) / 8;
            if (blocks > 148 * 16) blocks = 148 * 16;
            launch_pdl(gather_rows_kernel, dim3((unsigned)blocks), dim3(256), (size_t)(0), stream, p, rows, (int)(row_bytes / 16));
            return (int)cudaGetLastError();
        }
    }
    int64_t blocks = (p.total + 255) / 256;
    if (blocks > 148 * 8) blocks = 148 * 8;
    const unsigned grid = (unsigned)blocks;
    switch (p.elem_size) {
        case 1: launch_pdl(gather_kernel<uint8_t>, dim3(grid), dim3(256), (size_t)(0), stream, p); break;
        case 2: launch_pdl(gather_kernel<uint16_t>, dim3(grid), dim3(256), (size_t)(0), stream, p); break;
        case 4: launch_pdl(gather_kernel<uint32_t>, dim3(grid), dim3(256), (size_t)(0), stream, p); break;
        case 8: launch_pdl(gather_kernel<uint64_t>, dim3(grid), dim3(256), (size_t)(0), stream, p); break;
        default: return (int)cudaErrorInvalidValue;
    }
    return (int)cudaGetLastError();
}

// ------------------------------------------------------------------ im2col
namespace {

constexpr int kIm2colC = 128;   // channels per block

// One block: one filter tap, 32 output positions of one image, 128 channels (16 elements per thread in flight).  A source that is contiguous
// along W is read with the lanes along the positions and turned through shared memory so that the lanes
// run along the channels for the store (rows of 128 bytes); a channels-last source is read that way already.
__global__ void __launch_bounds__(256) im2col_kernel(const __grid_constant__ Im2colParams p, int p_tiles, int c_tiles, int channels_last) {
    pdl_enter();
    __shared__ float tile[kIm2colC][33];
    int rem = blockIdx.x;
    const int ct = rem % c_tiles;
    rem /= c_tiles;
    const int pt = rem % p_tiles;
    rem /= p_tiles;
    const int tap = rem % (p.r * p.s);
    const int n = rem / (p.r * p.s);
    const int r = tap / p.s, q = tap - r * p.s;
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    const int positions = p.oh * p.ow;
    const float* in = p.in + (int64_t)n * p.s_in[0];
    float* col = p.col + ((int64_t)n * positions * (p.r * p.s) + tap) * p.c_pad;
    const int p0 = pt * 32, c0 = ct * kIm2colC;
    if (!channels_last) {
        // this thread's position for the read: p0 + tx
        const int pos = p0 + tx;
        const int oy = pos / p.ow, ox = pos - oy * p.ow;
        const int iy = oy * p.stride_y + r - p.pad_y, ix = ox * p.stride_x + q - p.pad_x;
        const bool inside = pos < positions && iy >= 0 && iy < p.h && ix >= 0 && ix < p.w;
        const float* src = in + (int64_t)iy * p.s_in[2] + (int64_t)ix * p.s_in[3];
        float v[kIm2colC / 8];
#pragma unroll
        for (int j = 0; j < kIm2colC / 8; j++) {
            const int c = c0 + ty + 8 * j;
            v[j] = (inside && c < p.c) ? __ldg(src + (int64_t)c * p.s_in[1]) : 0.f;
        }
#pragma unroll
        for (int j = 0; j < kIm2colC / 8; j++) tile[ty + 8 * j][tx] = v[j];
        __syncthreads();
    }
    // store: lanes along the channels; jp picks the position (ty + 8 * jp), jc the 32-channel group
#pragma unroll
    for (int jp = 0; jp < 4; jp++) {
        const int pl = ty + 8 * jp, pos = p0 + pl;
        if (pos >= positions) continue;
        const float* src = nullptr;   // channels-last source: this position's pixel, or null outside the image
        if (channels_last) {
            const int oy = pos / p.ow, ox = pos - oy * p.ow;
            const int iy = oy * p.stride_y + r - p.pad_y, ix = ox * p.stride_x + q - p.pad_x;
            if (iy >= 0 && iy < p.h && ix >= 0 && ix < p.w) src = in + (int64_t)iy * p.s_in[2] + (int64_t)ix * p.s_in[3];
        }
        float* dst = col + (int64_t)pos * (p.r * p.s) * p.c_pad;
        float v[kIm2colC / 32];
#pragma unroll
        for (int jc = 0; jc < kIm2colC / 32; jc++) {
            const int cl = 32 * jc + tx, c = c0 + cl;
            if (channels_last) v[jc] = (src != nullptr && c < p.c) ? __ldg(src + (int64_t)c * p.s_in[1]) : 0.f;
            else v[jc] = tile[cl][pl];
        }
#pragma unroll
        for (int jc = 0; jc < kIm2colC / 32; jc++) {
            const int c = c0 + 32 * jc + tx;
            if (c < p.c_pad) dst[c] = v[jc];
        }
    }
}

}  // namespace

int launch_im2col(const Im2colParams& p, cudaStream_t stream) {
    const int64_t positions = (int64_t)p.oh * p.ow;
    if (p.n == 0 || positions == 0 || p.c_pad == 0) return 0;
    const int64_t p_tiles = (positions + 31) / 32, c_tiles = (p.c_pad + kIm2colC - 1) / kIm2colC;
    const int64_t blocks = p_tiles * c_tiles * p.r * p.s * p.n;
    if (blocks >= (1ll << 31)) return (int)cudaErrorInvalidValue;
    const int channels_last = (p.c <= 1 || p.s_in[1] == 1) ? 1 : 0;
    launch_pdl(im2col_kernel, dim3((unsigned)blocks), dim3(256), (size_t)0, stream, p, (int)p_tiles, (int)c_tiles, channels_last);
    return (int)cudaGetLastError();
}

}  // namespace kn
