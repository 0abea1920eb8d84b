// Softmax and layernorm over rows stored as f16 (the storage type of the LLaMA-shaped configuration; an
// extension: the reference's IR has no half type).  Same contract as the f32 kernels in rows.cu: the statistics
// and all arithmetic are f32, the row is read once and written once, and the result is rounded to f16 once.
//
//   rows_f16_vec_kernel        rows contiguous along the axis, a multiple of 8 long, 16-byte aligned: 128-bit
//                              accesses (8 halves), the row in registers; one warp per row up to 2048 elements,
//                              one block of 256 threads per row up to 16384
//   rows_f16_streaming_kernel  everything else (any strides, any length): three sweeps over the row
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <algorithm>

#include "../kernels.h"
#include "launch.cuh"

namespace kn {

namespace {

constexpr unsigned kFullMask = 0xFFFFFFFFu;

__device__ __forceinline__ float wmax(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(kFullMask, v, o));
    return v;
}
__device__ __forceinline__ float wsum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(kFullMask, v, o);
    return v;
}
template <int TPR, bool IS_MAX>
__device__ __forceinline__ float reduce_row(float v, float* smem) {
    v = IS_MAX ? wmax(v) : wsum(v);
    if (TPR == 32) return v;
    // (a block may hold several rows of TPR threads each: a row's warps are neighbours)
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    constexpr int kWarpsPerRow = TPR >> 5;
    const int first = (warp / kWarpsPerRow) * kWarpsPerRow;
    __syncthreads();
    if (lane == 0) smem[warp] = v;
    __syncthreads();
    float r = lane < kWarpsPerRow ? smem[first + lane] : (IS_MAX ? -INFINITY : 0.0f);
    return IS_MAX ? wmax(r) : wsum(r);
}

__device__ __forceinline__ void offsets(int64_t idx, int rank, const int64_t* dims, const int64_t* s0, const int64_t* s1,
                                        const int64_t* s2, int64_t& o0, int64_t& o1, int64_t& o2) {
    o0 = o1 = o2 = 0;
    for (int d = rank - 1; d >= 0; d--) {
        const int64_t dim = dims[d];
        const int64_t q = idx / dim;
        const int64_t i = idx - q * dim;
        idx = q;
        o0 += i * s0[d];
        o1 += i * s1[d];
        o2 += i * s2[d];
    }
}

__device__ __forceinline__ void unpack8(const uint4& u, float (&f)[8]) {
    const __half2* h = (const __half2*)&u;
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const float2 t = __half22float2(h[i]);
        f[2 * i] = t.x;
        f[2 * i + 1] = t.y;
    }
}
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
    uint4 u;
    __half2* h = (__half2*)&u;
#pragma unroll
    for (int i = 0; i < 4; i++) h[i] = __floats2half2_rn(f[2 * i], f[2 * i + 1]);
    return u;
}

// SOFTMAX: x = scale * in0 + in1 (in1 with strides of its own); else layernorm: x = alpha0 * in0 + alpha1 * in1
// (in1 with in0's strides).
template <bool SOFTMAX, int TPR, int ITEMS>
__global__ void __launch_bounds__(256) rows_f16_vec_kernel(const __grid_constant__ RowParams p) {
    pdl_enter();
    __shared__ float smem[8];
    const int rows_per_block = blockDim.x / TPR;
    const int64_t row = (int64_t)blockIdx.x * rows_per_block + threadIdx.x / TPR;
    const int t = threadIdx.x % TPR;
    const bool active = row < p.rows;
    int64_t oi = 0, oo = 0, o1 = 0;
    if (active) offsets(row, p.outer_rank, p.outer_dims, p.in_strides, p.out_strides, SOFTMAX ? p.in1_strides : p.in_strides, oi, oo, o1);
    const uint4* in0 = (const uint4*)((const __half*)p.in0 + oi);
    const uint4* in1 = p.in1 ? (const uint4*)((const __half*)p.in1 + o1) : nullptr;
    uint4* out = (uint4*)((__half*)p.out + oo);
    const int len8 = (int)(p.len >> 3);

    float v[ITEMS][8];
    const float pad = SOFTMAX ? -INFINITY : 0.f;
#pragma unroll
    for (int i = 0; i < ITEMS; i++) {
        const int e = i * TPR + t;
        if (active && e < len8) {
            unpack8(__ldg(in0 + e), v[i]);
            const float a0 = SOFTMAX ? p.scale : p.alpha0;
#pragma unroll
            for (int j = 0; j < 8; j++) v[i][j] *= a0;
        } else {
#pragma unroll
            for (int j = 0; j < 8; j++) v[i][j] = pad;
        }
    }
    if (in1 != nullptr) {
#pragma unroll
        for (int i = 0; i < ITEMS; i++) {
            const int e = i * TPR + t;
            if (active && e < len8) {
                float a[8];
                unpack8(__ldg(in1 + e), a);
                const float a1 = SOFTMAX ? 1.f : p.alpha1;
#pragma unroll
                for (int j = 0; j < 8; j++) v[i][j] += a1 * a[j];
            }
        }
    }
    if (SOFTMAX) {
        float mx = -INFINITY;
#pragma unroll
        for (int i = 0; i < ITEMS; i++)
#pragma unroll
            for (int j = 0; j < 8; j++) mx = fmaxf(mx, v[i][j]);
        mx = reduce_row<TPR, true>(mx, smem);
        float sum = 0.f;
#pragma unroll
        for (int i = 0; i < ITEMS; i++)
#pragma unroll
            for (int j = 0; j < 8; j++) {
                // (the hardware exponential: its error, about 2^-21 relative, is far below the f16 step the result
                // is rounded to; with half the bytes per element of an f32 row the exact expf would bound the kernel)
                v[i][j] = __expf(v[i][j] - mx);   // padding: exp(-inf) = 0
                sum += v[i][j];
            }
        sum = reduce_row<TPR, false>(sum, smem);
        if (!active) return;
        const float inv = 1.0f / sum;
#pragma unroll
        for (int i = 0; i < ITEMS; i++) {
            const int e = i * TPR + t;
            if (e < len8) {
#pragma unroll
                for (int j = 0; j < 8; j++) v[i][j] = v[i][j] * inv;
                out[e] = pack8(v[i]);
            }
        }
    } else {
        float sum = 0.f;
#pragma unroll
        for (int i = 0; i < ITEMS; i++)
#pragma unroll
            for (int j = 0; j < 8; j++) sum += v[i][j];
        const float n = (float)p.len;
        const float mean = reduce_row<TPR, false>(sum, smem) / n;
        float sq = 0.f;
#pragma unroll
        for (int i = 0; i < ITEMS; i++) {
            const int e = i * TPR + t;
#pragma unroll
            for (int j = 0; j < 8; j++) {
                v[i][j] -= mean;
                if (e < len8) sq += v[i][j] * v[i][j];
            }
        }
        const float var = reduce_row<TPR, false>(sq, smem) / n;
        const float inv = 1.0f / sqrtf(var + p.eps);
        if (!active) return;
#pragma unroll
        for (int i = 0; i < ITEMS; i++) {
            const int e = i * TPR + t;
            if (e < len8) {
#pragma unroll
                for (int j = 0; j < 8; j++) v[i][j] = v[i][j] * inv;
                out[e] = pack8(v[i]);
            }
        }
    }
}

template <bool SOFTMAX>
__global__ void __launch_bounds__(256) rows_f16_streaming_kernel(const __grid_constant__ RowParams p) {
    pdl_enter();
    __shared__ float smem[8];
    const int64_t row = blockIdx.x;
    int64_t oi, oo, o1;
    offsets(row, p.outer_rank, p.outer_dims, p.in_strides, p.out_strides, SOFTMAX ? p.in1_strides : p.in_strides, oi, oo, o1);
    const __half* in0 = (const __half*)p.in0 + oi;
    const __half* in1 = p.in1 ? (const __half*)p.in1 + o1 : nullptr;
    __half* out = (__half*)p.out + oo;
    const int64_t s1 = SOFTMAX ? p.in1_axis_stride : p.in_axis_stride;
    auto load = [&](int64_t e) {
        float x = (SOFTMAX ? p.scale : p.alpha0) * __half2float(in0[e * p.in_axis_stride]);
        if (in1) x += (SOFTMAX ? 1.f : p.alpha1) * __half2float(in1[e * s1]);
        return x;
    };
    if (SOFTMAX) {
        float mx = -INFINITY;
        for (int64_t e = threadIdx.x; e < p.len; e += 256) mx = fmaxf(mx, load(e));
        mx = reduce_row<256, true>(mx, smem);
        float sum = 0.f;
        for (int64_t e = threadIdx.x; e < p.len; e += 256) sum += expf(load(e) - mx);
        sum = reduce_row<256, false>(sum, smem);
        for (int64_t e = threadIdx.x; e < p.len; e += 256) out[e * p.out_axis_stride] = __float2half_rn(expf(load(e) - mx) / sum);
    } else {
        const float n = (float)p.len;
        float sum = 0.f;
        for (int64_t e = threadIdx.x; e < p.len; e += 256) sum += load(e);
        const float mean = reduce_row<256, false>(sum, smem) / n;
        float sq = 0.f;
        for (int64_t e = threadIdx.x; e < p.len; e += 256) {
            const float d = load(e) - mean;
            sq += d * d;
        }
        const float var = reduce_row<256, false>(sq, smem) / n;
        const float denom = sqrtf(var + p.eps);
        for (int64_t e = threadIdx.x; e < p.len; e += 256) out[e * p.out_axis_stride] = __float2half_rn((load(e) - mean) / denom);
    }
}

// One block of 256 threads per row at a time, the row (up to 16384 elements, a multiple of 8) in registers as f32: one
// read, one write.  The blocks are persistent and software-pipelined: the next row's loads are issued (as raw 128-bit
// registers) before this row's reduction, so a block always has a row in flight; with one short-lived block per row the
// load -> barrier -> barrier -> store chain left the memory system idle half of the time.
template <bool IN_HALF, bool OUT_HALF, int ITEMS>
__global__ void __launch_bounds__(256) rmsnorm_kernel(const __grid_constant__ RmsNormParams p) {
    pdl_enter();
    __shared__ float smem[8];
    constexpr int R = IN_HALF ? ITEMS : 2 * ITEMS;   // 128-bit loads per thread and row
    const int t = threadIdx.x;
    const int len8 = (int)(p.len >> 3);
    auto load_row = [&](int64_t row, uint4 (&raw)[R]) {
#pragma unroll
        for (int i = 0; i < ITEMS; i++) {
            const int e = i * 256 + t;
            if (e < len8) {
                if (IN_HALF) {
                    raw[i] = __ldg((const uint4*)((const __half*)p.in + row * p.in_row_stride) + e);
                } else {
                    const uint4* src = (const uint4*)((const float*)p.in + row * p.in_row_stride) + 2 * e;
                    raw[2 * i] = __ldg(src);
                    raw[2 * i + 1] = __ldg(src + 1);
                }
            }
        }
    };
    uint4 raw[R], next_raw[R];
    int64_t row = blockIdx.x;
    if (row < p.rows) load_row(row, raw);
    for (; row < p.rows; row += gridDim.x) {
        const int64_t next = row + gridDim.x;
        if (next < p.rows) load_row(next, next_raw);
        float v[ITEMS][8];
        float sq = 0.f;
#pragma unroll
        for (int i = 0; i < ITEMS; i++) {
            const int e = i * 256 + t;
            if (e < len8) {
                if (IN_HALF) {
                    unpack8(raw[i], v[i]);
                } else {
                    const float4 a = *(const float4*)&raw[2 * i], b = *(const float4*)&raw[2 * i + 1];
                    v[i][0] = a.x; v[i][1] = a.y; v[i][2] = a.z; v[i][3] = a.w;
                    v[i][4] = b.x; v[i][5] = b.y; v[i][6] = b.z; v[i][7] = b.w;
                }
#pragma unroll
                for (int j = 0; j < 8; j++) sq += v[i][j] * v[i][j];
            }
        }
        const float ms = reduce_row<256, false>(sq, smem) / (float)p.len;
        const float inv = 1.0f / sqrtf(ms + p.eps);
#pragma unroll
        for (int i = 0; i < ITEMS; i++) {
            const int e = i * 256 + t;
            if (e < len8) {
                if (p.gain != nullptr && p.gain_stride == 1) {
                    const float4 g0 = __ldg((const float4*)p.gain + 2 * e), g1 = __ldg((const float4*)p.gain + 2 * e + 1);
                    const float g[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
#pragma unroll
                    for (int j = 0; j < 8; j++) v[i][j] = v[i][j] * inv * g[j];
                } else {
#pragma unroll
                    for (int j = 0; j < 8; j++) {
                        float y = v[i][j] * inv;
                        if (p.gain != nullptr) y *= __ldg(p.gain + (int64_t)(e * 8 + j) * p.gain_stride);
                        v[i][j] = y;
                    }
                }
                if (OUT_HALF) {
                    *((uint4*)((__half*)p.out + row * p.out_row_stride) + e) = pack8(v[i]);
                } else {
                    float4* dst = (float4*)((float*)p.out + row * p.out_row_stride) + 2 * e;
                    dst[0] = make_float4(v[i][0], v[i][1], v[i][2], v[i][3]);
                    dst[1] = make_float4(v[i][4], v[i][5], v[i][6], v[i][7]);
                }
            }
        }
#pragma unroll
        for (int i = 0; i < R; i++) raw[i] = next_raw[i];
    }
}

template <bool IN_HALF, bool OUT_HALF, int ITEMS>
void launch_rmsnorm_items(const RmsNormParams& p, cudaStream_t stream) {
    // persistent blocks: as many as are resident at once on the 148 SMs
    int per_sm = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, rmsnorm_kernel<IN_HALF, OUT_HALF, ITEMS>, 256, 0) != cudaSuccess || per_sm < 1)
        per_sm = 1;
    const dim3 grid((unsigned)std::min<int64_t>(p.rows, (int64_t)148 * per_sm)), block(256);
    launch_pdl(rmsnorm_kernel<IN_HALF, OUT_HALF, ITEMS>, grid, block, (size_t)0, stream, p);
}

template <bool IN_HALF, bool OUT_HALF>
int launch_rmsnorm_t(const RmsNormParams& p, cudaStream_t stream) {
    const int items = (int)((p.len / 8 + 255) / 256);
    if (items <= 1) launch_rmsnorm_items<IN_HALF, OUT_HALF, 1>(p, stream);
    else if (items <= 2) launch_rmsnorm_items<IN_HALF, OUT_HALF, 2>(p, stream);
    else if (items <= 4) launch_rmsnorm_items<IN_HALF, OUT_HALF, 4>(p, stream);
    else launch_rmsnorm_items<IN_HALF, OUT_HALF, 8>(p, stream);
    return (int)cudaGetLastError();
}

bool vec_ok(const RowParams& p, bool softmax) {
    if (p.len % 8 != 0 || p.len > 16384 || p.in_axis_stride != 1 || p.out_axis_stride != 1) return false;
    if (((uintptr_t)p.in0 & 15) || ((uintptr_t)p.out & 15) || (p.in1 && ((uintptr_t)p.in1 & 15))) return false;
    if (p.in1 && softmax && p.in1_axis_stride != 1) return false;
    for (int d = 0; d < p.outer_rank; d++) {
        if (p.in_strides[d] % 8 != 0 || p.out_strides[d] % 8 != 0) return false;
        if (p.in1 && softmax && p.in1_strides[d] % 8 != 0) return false;
    }
    return true;
}

template <bool SOFTMAX>
int launch_rows(const RowParams& p, cudaStream_t stream) {
    if (p.rows == 0 || p.len == 0) return 0;
    if (p.rows > 0x7FFFFFFFll) return (int)cudaErrorInvalidValue;
    if (vec_ok(p, SOFTMAX)) {
        const int len8 = (int)(p.len / 8);
        if (len8 <= 128) {   // one warp per row, eight rows per block
            const unsigned grid = (unsigned)((p.rows + 7) / 8);
            const int items = (len8 + 31) / 32;
            if (items <= 1) launch_pdl(rows_f16_vec_kernel<SOFTMAX, 32, 1>, dim3(grid), dim3(256), (size_t)0, stream, p);
            else if (items <= 2) launch_pdl(rows_f16_vec_kernel<SOFTMAX, 32, 2>, dim3(grid), dim3(256), (size_t)0, stream, p);
            else launch_pdl(rows_f16_vec_kernel<SOFTMAX, 32, 4>, dim3(grid), dim3(256), (size_t)0, stream, p);
        } else if (len8 <= 256) {
            // Four warps per row, two rows per block.  One warp per row would hold 64 converted values plus the raw
            // loads per lane: more than 128 registers, so one block of 8 warps per SM and half the bandwidth
            // (measured on 2048-element rows: 0.54 of the copy bandwidth).
            const unsigned grid = (unsigned)((p.rows + 1) / 2);
            launch_pdl(rows_f16_vec_kernel<SOFTMAX, 128, 2>, dim3(grid), dim3(256), (size_t)0, stream, p);
        } else {             // one block per row
            const unsigned grid = (unsigned)p.rows;
            const int items = (len8 + 255) / 256;
            if (items <= 2) launch_pdl(rows_f16_vec_kernel<SOFTMAX, 256, 2>, dim3(grid), dim3(256), (size_t)0, stream, p);
            else if (items <= 4) launch_pdl(rows_f16_vec_kernel<SOFTMAX, 256, 4>, dim3(grid), dim3(256), (size_t)0, stream, p);
            else launch_pdl(rows_f16_vec_kernel<SOFTMAX, 256, 8>, dim3(grid), dim3(256), (size_t)0, stream, p);
        }
        return (int)cudaGetLastError();
    }
    launch_pdl(rows_f16_streaming_kernel<SOFTMAX>, dim3((unsigned)p.rows), dim3(256), (size_t)0, stream, p);
    return (int)cudaGetLastError();
}

}  // namespace

// The planner emits this step only for rows it has checked: len a multiple of 8 and at most 16384, rows 16-byte aligned.
int launch_rmsnorm(const RmsNormParams& p, cudaStream_t stream) {
    if (p.rows == 0 || p.len == 0) return 0;
    if (p.rows > 0x7FFFFFFFll || p.len % 8 != 0 || p.len > 16384) return (int)cudaErrorInvalidValue;
    if (p.in_half) return p.out_half ? launch_rmsnorm_t<true, true>(p, stream) : launch_rmsnorm_t<true, false>(p, stream);
    return p.out_half ? launch_rmsnorm_t<false, true>(p, stream) : launch_rmsnorm_t<false, false>(p, stream);
}

int launch_softmax_f16(const RowParams& p, cudaStream_t stream) { return launch_rows<true>(p, stream); }
int launch_layernorm_f16(const RowParams& p, cudaStream_t stream) { return launch_rows<false>(p, stream); }

}  // namespace kn
