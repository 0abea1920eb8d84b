// Row-wise kernels: reduce, softmax, layernorm.  They take the place of the reference's
// `reduce_kernel`, `softmax_kernel` and `layernorm_kernel` templates
// (kn-cuda-eval/src/autokernel/{reduce,softmax,layernorm}.cu).
//
// softmax / layernorm keep the whole row in registers between the statistics pass and the
// normalising pass, so global memory is read once and written once (the reference kernels re-read
// the row two or three times).  A row is owned by a warp (len <= 1024) or by a block
// (len <= 8192); longer rows fall back to a block that re-reads the row from L2 / HBM.
#include <cuda_runtime.h>

#include "../kernels.h"
#include "../scalar_ops.h"
#include "launch.cuh"

namespace kn {

namespace {

constexpr unsigned kFull = 0xFFFFFFFFu;

__device__ __forceinline__ void decode_offsets(int64_t idx, int rank, const int64_t* dims, const int64_t* s0,
                                                const int64_t* s1, int64_t& o0, int64_t& o1) {
    o0 = 0;
    o1 = 0;
    for (int d = rank - 1; d >= 0; d--) {
        const int64_t dim = dims[d];
        const int64_t q = idx / dim;
        const int64_t i = idx - q * dim;
        idx = q;
        o0 += i * s0[d];
        o1 += i * s1[d];
    }
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(kFull, v, o));
    return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(kFull, v, o);
    return v;
}

// Reduction across the `TPR` threads that own one row.  TPR == 32: a warp.  TPR == blockDim.x: the
// whole block through shared memory.
template <int TPR, bool IS_MAX>
__device__ __forceinline__ float row_reduce(float v, float* smem) {
    v = IS_MAX ? warp_max(v) : warp_sum(v);
    if (TPR == 32) return v;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    __syncthreads();   // protect smem reuse between consecutive reductions
    if (lane == 0) smem[warp] = v;
    __syncthreads();
    float r = lane < (TPR >> 5) ? smem[lane] : (IS_MAX ? -INFINITY : 0.0f);
    return IS_MAX ? warp_max(r) : warp_sum(r);
}

// ------------------------------------------------------------------ softmax
template <int TPR, int ITEMS>
__global__ void __launch_bounds__(256) softmax_cached_kernel(const __grid_constant__ RowParams p) {
    pdl_enter();
    __shared__ float smem[8];
    const int rows_per_block = blockDim.x / TPR;
    const int64_t row = (int64_t)blockIdx.x * rows_per_block + threadIdx.x / TPR;
    const int t = threadIdx.x % TPR;
    const bool active = row < p.rows;   // whole warps / blocks share `row`, so reductions stay converged
    int64_t oi = 0, oo = 0;
    if (active) decode_offsets(row, p.outer_rank, p.outer_dims, p.in_strides, p.out_strides, oi, oo);
    const float* in = p.in0 + oi;
    float* out = p.out + oo;
    const float* add = nullptr;
    if (p.in1 != nullptr && active) {
        int64_t o1, unused;
        decode_offsets(row, p.outer_rank, p.outer_dims, p.in1_strides, p.out_strides, o1, unused);
        add = p.in1 + o1;
    }

    float v[ITEMS];
    float mx = -INFINITY;
#pragma unroll
    for (int i = 0; i < ITEMS; i++) {
        const int64_t e = (int64_t)i * TPR + t;
        v[i] = (active && e < p.len) ? in[e * p.in_axis_stride] * p.scale + (add ? add[e * p.in1_axis_stride] : 0.f) : -INFINITY;
        mx = fmaxf(mx, v[i]);
    }
    mx = row_reduce<TPR, true>(mx, smem);
    float sum = 0.f;
#pragma unroll
    for (int i = 0; i < ITEMS; i++) {
        const int64_t e = (int64_t)i * TPR + t;
        v[i] = expf(v[i] - mx);
        if (e < p.len) sum += v[i];
    }
    sum = row_reduce<TPR, false>(sum, smem);
    if (!active) return;
#pragma unroll
    for (int i = 0; i < ITEMS; i++) {
        const int64_t e = (int64_t)i * TPR + t;
        if (e < p.len) out[e * p.out_axis_stride] = v[i] / sum;
    }
}

// rows longer than a block can keep in registers: three sweeps over global memory
__global__ void __launch_bounds__(256) softmax_streaming_kernel(const __grid_constant__ RowParams p) {
    pdl_enter();
    __shared__ float smem[8];
    const int64_t row = blockIdx.x;
    int64_t oi, oo;
    decode_offsets(row, p.outer_rank, p.outer_dims, p.in_strides, p.out_strides, oi, oo);
    const float* in = p.in0 + oi;
    float* out = p.out + oo;
    const float* add = nullptr;
    if (p.in1 != nullptr) {
        int64_t o1, unused;
        decode_offsets(row, p.outer_rank, p.outer_dims, p.in1_strides, p.out_strides, o1, unused);
        add = p.in1 + o1;
    }
    auto load = [&](int64_t e) { return in[e * p.in_axis_stride] * p.scale + (add ? add[e * p.in1_axis_stride] : 0.f); };
    float mx = -INFINITY;
    for (int64_t e = threadIdx.x; e < p.len; e += 256) mx = fmaxf(mx, load(e));
    mx = row_reduce<256, true>(mx, smem);
    float sum = 0.f;
    for (int64_t e = threadIdx.x; e < p.len; e += 256) sum += expf(load(e) - mx);
    sum = row_reduce<256, false>(sum, smem);
    for (int64_t e = threadIdx.x; e < p.len; e += 256) out[e * p.out_axis_stride] = expf(load(e) - mx) / sum;
}

// ------------------------------------------------------------------ layernorm
__device__ __forceinline__ float ln_load(const RowParams& p, const float* in0, const float* in1, int64_t e) {
    float x = p.alpha0 * in0[e * p.in_axis_stride];
    if (in1 != nullptr) x += p.alpha1 * in1[e * p.in_axis_stride];
    return x;
}

template <int TPR, int ITEMS>
__global__ void __launch_bounds__(256) layernorm_cached_kernel(const __grid_constant__ RowParams p) {
    pdl_enter();
    __shared__ float smem[8];
    const int rows_per_block = blockDim.x / TPR;
    const int64_t row = (int64_t)blockIdx.x * rows_per_block + threadIdx.x / TPR;
    const int t = threadIdx.x % TPR;
    const bool active = row < p.rows;
    int64_t oi = 0, oo = 0;
    if (active) decode_offsets(row, p.outer_rank, p.outer_dims, p.in_strides, p.out_strides, oi, oo);
    const float* in0 = p.in0 + oi;
    const float* in1 = p.in1 ? p.in1 + oi : nullptr;
    float* out = p.out + oo;

    float v[ITEMS];
    float sum = 0.f;
#pragma unroll
    for (int i = 0; i < ITEMS; i++) {
        const int64_t e = (int64_t)i * TPR + t;
        v[i] = (active && e < p.len) ? ln_load(p, in0, in1, e) : 0.f;
        sum += v[i];
    }
    const float n = (float)p.len;
    const float mean = row_reduce<TPR, false>(sum, smem) / n;
    float sq = 0.f;
#pragma unroll
    for (int i = 0; i < ITEMS; i++) {
        const int64_t e = (int64_t)i * TPR + t;
        v[i] -= mean;
        if (e < p.len) sq += v[i] * v[i];
    }
    const float var = row_reduce<TPR, false>(sq, smem) / n;
    const float denom = sqrtf(var + p.eps);
    if (!active) return;
#pragma unroll
    for (int i = 0; i < ITEMS; i++) {
        const int64_t e = (int64_t)i * TPR + t;
        if (e < p.len) out[e * p.out_axis_stride] = v[i] / denom;
    }
}

__global__ void __launch_bounds__(256) layernorm_streaming_kernel(const __grid_constant__ RowParams p) {
    pdl_enter();
    __shared__ float smem[8];
    const int64_t row = blockIdx.x;
    int64_t oi, oo;
    decode_offsets(row, p.outer_rank, p.outer_dims, p.in_strides, p.out_strides, oi, oo);
    const float* in0 = p.in0 + oi;
    const float* in1 = p.in1 ? p.in1 + oi : nullptr;
    float* out = p.out + oo;
    const float n = (float)p.len;
    float sum = 0.f;
    for (int64_t e = threadIdx.x; e < p.len; e += 256) sum += ln_load(p, in0, in1, e);
    const float mean = row_reduce<256, false>(sum, smem) / n;
    float sq = 0.f;
    for (int64_t e = threadIdx.x; e < p.len; e += 256) {
        const float d = ln_load(p, in0, in1, e) - mean;
        sq += d * d;
    }
    const float var = row_reduce<256, false>(sq, smem) / n;
    const float denom = sqrtf(var + p.eps);
    for (int64_t e = threadIdx.x; e < p.len; e += 256) out[e * p.out_axis_stride] = (ln_load(p, in0, in1, e) - mean) / denom;
}

// ------------------------------------------------------------------ 128-bit variants
// Rows that are contiguous along the axis, a multiple of 4 long and 16-byte aligned (the planner's dense
// tensors always are): every lane moves float4s, offsets are 32-bit, and the per-lane item count is exactly
// what the row needs.  One warp (TPR = 32) or one block (TPR = 256) per row, the row stays in registers
// between the statistics and the normalising pass: one read, one write.
template <int TPR, int ITEMS4>
__global__ void __launch_bounds__(256) softmax_vec4_kernel(const __grid_constant__ RowParams p) {
    pdl_enter();
    __shared__ float smem[8];
    const int rows_per_block = blockDim.x / TPR;
    const int64_t row = (int64_t)blockIdx.x * rows_per_block + threadIdx.x / TPR;
    const int t = threadIdx.x % TPR;
    const bool active = row < p.rows;
    int64_t oi = 0, oo = 0;
    if (active) decode_offsets(row, p.outer_rank, p.outer_dims, p.in_strides, p.out_strides, oi, oo);
    const float4* in = (const float4*)(p.in0 + oi);
    float4* out = (float4*)(p.out + oo);
    const int len4 = (int)(p.len >> 2);
    const float4* add = nullptr;
    if (p.in1 != nullptr && active) {
        int64_t o1, unused;
        decode_offsets(row, p.outer_rank, p.outer_dims, p.in1_strides, p.out_strides, o1, unused);
        add = (const float4*)(p.in1 + o1);
    }

    float4 v[ITEMS4];
    float mx = -INFINITY;
#pragma unroll
    for (int i = 0; i < ITEMS4; i++) {
        const int e = i * TPR + t;
        if (active && e < len4) {
            v[i] = __ldg(in + e);
            v[i].x *= p.scale; v[i].y *= p.scale; v[i].z *= p.scale; v[i].w *= p.scale;
        } else {
            v[i] = make_float4(-INFINITY, -INFINITY, -INFINITY, -INFINITY);
        }
    }
    // the additive term in a loop of its own: a branch inside the loop above would keep the compiler from
    // issuing all the row's loads back to back
    if (add != nullptr) {
#pragma unroll
        for (int i = 0; i < ITEMS4; i++) {
            const int e = i * TPR + t;
            if (e < len4) {
                const float4 a = __ldg(add + e);
                v[i].x += a.x; v[i].y += a.y; v[i].z += a.z; v[i].w += a.w;
            }
        }
    }
#pragma unroll
    for (int i = 0; i < ITEMS4; i++) mx = fmaxf(mx, fmaxf(fmaxf(v[i].x, v[i].y), fmaxf(v[i].z, v[i].w)));
    mx = row_reduce<TPR, true>(mx, smem);
    float sum = 0.f;
#pragma unroll
    for (int i = 0; i < ITEMS4; i++) {
        v[i].x = expf(v[i].x - mx); v[i].y = expf(v[i].y - mx); v[i].z = expf(v[i].z - mx); v[i].w = expf(v[i].w - mx);
        sum += (v[i].x + v[i].y) + (v[i].z + v[i].w);     // padding lanes hold exp(-inf) = 0
    }
    sum = row_reduce<TPR, false>(sum, smem);
    if (!active) return;
#pragma unroll
    for (int i = 0; i < ITEMS4; i++) {
        const int e = i * TPR + t;
        if (e < len4) out[e] = make_float4(v[i].x / sum, v[i].y / sum, v[i].z / sum, v[i].w / sum);
    }
}

template <int TPR, int ITEMS4>
__global__ void __launch_bounds__(TPR > 256 ? TPR : 256) layernorm_vec4_kernel(const __grid_constant__ RowParams p) {
    pdl_enter();
    __shared__ float smem[32];
    const int rows_per_block = blockDim.x / TPR;
    const int64_t row = (int64_t)blockIdx.x * rows_per_block + threadIdx.x / TPR;
    const int t = threadIdx.x % TPR;
    const bool active = row < p.rows;
    int64_t oi = 0, oo = 0;
    if (active) decode_offsets(row, p.outer_rank, p.outer_dims, p.in_strides, p.out_strides, oi, oo);
    const float4* in0 = (const float4*)(p.in0 + oi);
    const float4* in1 = p.in1 ? (const float4*)(p.in1 + oi) : nullptr;
    float4* out = (float4*)(p.out + oo);
    const int len4 = (int)(p.len >> 2);

    float4 v[ITEMS4];
    float sum = 0.f;
#pragma unroll
    for (int i = 0; i < ITEMS4; i++) {
        const int e = i * TPR + t;
        v[i] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (active && e < len4) {
            const float4 a = __ldg(in0 + e);
            v[i] = make_float4(p.alpha0 * a.x, p.alpha0 * a.y, p.alpha0 * a.z, p.alpha0 * a.w);
            if (in1 != nullptr) {
                const float4 b = __ldg(in1 + e);
                v[i].x += p.alpha1 * b.x; v[i].y += p.alpha1 * b.y; v[i].z += p.alpha1 * b.z; v[i].w += p.alpha1 * b.w;
            }
        }
        sum += (v[i].x + v[i].y) + (v[i].z + v[i].w);
    }
    const float n = (float)p.len;
    const float mean = row_reduce<TPR, false>(sum, smem) / n;
    float sq = 0.f;
#pragma unroll
    for (int i = 0; i < ITEMS4; i++) {
        const int e = i * TPR + t;
        v[i].x -= mean; v[i].y -= mean; v[i].z -= mean; v[i].w -= mean;
        if (e < len4) sq += (v[i].x * v[i].x + v[i].y * v[i].y) + (v[i].z * v[i].z + v[i].w * v[i].w);
    }
    const float var = row_reduce<TPR, false>(sq, smem) / n;
    const float denom = sqrtf(var + p.eps);
    if (!active) return;
#pragma unroll
    for (int i = 0; i < ITEMS4; i++) {
        const int e = i * TPR + t;
        if (e < len4) out[e] = make_float4(v[i].x / denom, v[i].y / denom, v[i].z / denom, v[i].w / denom);
    }
}

// A row too long for one block's registers (a group norm over a few groups of a large feature map: 64 rows of 81 920
// or 122 880 elements in the UNet-shaped graph): a thread-block cluster of CL CTAs takes the row, each CTA keeps a
// CL-th of it in registers, and the two statistics meet through distributed shared memory (every CTA publishes its
// partial sum in its own shared memory, a cluster barrier, every CTA adds the CL partials in the same order).  One
// read and one write of the row on CL times as many SMs as rows, where the streaming kernel sweeps global memory three
// times with one CTA per row (64 CTAs on 148 SMs: 218 GB/s measured).
template <int CL, int ITEMS4>
__global__ void __launch_bounds__(512) layernorm_cluster_kernel(const __grid_constant__ RowParams p) {
    pdl_enter();
    __shared__ float smem[32];
    __shared__ float partial[2];
    uint32_t rank;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(rank));
    const int64_t row = (int64_t)(blockIdx.x / CL);
    const int t = threadIdx.x;
    int64_t oi = 0, oo = 0;
    decode_offsets(row, p.outer_rank, p.outer_dims, p.in_strides, p.out_strides, oi, oo);
    const int len4 = (int)(p.len >> 2);
    const int part4 = (len4 + CL - 1) / CL;                 // float4s per CTA
    const int begin = (int)rank * part4, end = min(len4, begin + part4);
    const float4* in0 = (const float4*)(p.in0 + oi);
    const float4* in1 = p.in1 ? (const float4*)(p.in1 + oi) : nullptr;
    float4* out = (float4*)(p.out + oo);
    // the sum of the CL partials, identical in every CTA of the cluster
    auto cluster_sum = [&](float mine, int slot) -> float {
        if (t == 0) partial[slot] = mine;
        asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
        asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
        float total = 0.f;
        const uint32_t local = (uint32_t)__cvta_generic_to_shared(&partial[slot]);
#pragma unroll
        for (uint32_t c = 0; c < (uint32_t)CL; c++) {
            uint32_t remote;
            float v;
            asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local), "r"(c));
            asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(remote) : "memory");
            total += v;
        }
        return total;
    };

    float4 v[ITEMS4];
    float sum = 0.f;
#pragma unroll
    for (int i = 0; i < ITEMS4; i++) {
        const int e = begin + i * 512 + t;
        v[i] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (e < end) {
            const float4 a = __ldg(in0 + e);
            v[i] = make_float4(p.alpha0 * a.x, p.alpha0 * a.y, p.alpha0 * a.z, p.alpha0 * a.w);
            if (in1 != nullptr) {
                const float4 b = __ldg(in1 + e);
                v[i].x += p.alpha1 * b.x; v[i].y += p.alpha1 * b.y; v[i].z += p.alpha1 * b.z; v[i].w += p.alpha1 * b.w;
            }
        }
        sum += (v[i].x + v[i].y) + (v[i].z + v[i].w);
    }
    const float n = (float)p.len;
    const float mean = cluster_sum(row_reduce<512, false>(sum, smem), 0) / n;
    float sq = 0.f;
#pragma unroll
    for (int i = 0; i < ITEMS4; i++) {
        const int e = begin + i * 512 + t;
        v[i].x -= mean; v[i].y -= mean; v[i].z -= mean; v[i].w -= mean;
        if (e < end) sq += (v[i].x * v[i].x + v[i].y * v[i].y) + (v[i].z * v[i].z + v[i].w * v[i].w);
    }
    const float var = cluster_sum(row_reduce<512, false>(sq, smem), 1) / n;
    const float denom = sqrtf(var + p.eps);
#pragma unroll
    for (int i = 0; i < ITEMS4; i++) {
        const int e = begin + i * 512 + t;
        if (e < end) out[e] = make_float4(v[i].x / denom, v[i].y / denom, v[i].z / denom, v[i].w / denom);
    }
    // no CTA leaves while another may still read its partial sums
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

template <int CL, int ITEMS4>
static int launch_layernorm_cluster(const RowParams& p, cudaStream_t stream) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(p.rows * CL));
    cfg.blockDim = dim3(512);
    cfg.dynamicSmemBytes = 0;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    attr[1].id = cudaLaunchAttributeClusterDimension;
    attr[1].val.clusterDim.x = CL;
    attr[1].val.clusterDim.y = 1;
    attr[1].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 2;
    return (int)cudaLaunchKernelEx(&cfg, layernorm_cluster_kernel<CL, ITEMS4>, p);
}

// Sum / mean of f32 over a contiguous innermost axis: TPO threads per output, float4 loads.
template <int TPO>
__global__ void __launch_bounds__(256) reduce_f32_rows_kernel(const __grid_constant__ ReduceParams p) {
    pdl_enter();
    __shared__ float smem[8];
    const int outs_per_block = 256 / TPO;
    const int64_t o = (int64_t)blockIdx.x * outs_per_block + threadIdx.x / TPO;
    const int t = threadIdx.x % TPO;
    const bool active = o < p.n_out;
    const ReduceOp rop = (ReduceOp)p.op;
    int64_t oi = 0, oo = 0;
    if (active) decode_offsets(o, p.kept_rank, p.kept_dims, p.kept_in_strides, p.kept_out_strides, oi, oo);
    const float4* in = (const float4*)((const float*)p.in + oi);
    const int len4 = (int)(p.n_red >> 2);
    const bool is_max = rop == ReduceOp::Max, is_min = rop == ReduceOp::Min, is_prod = rop == ReduceOp::Prod;
    float acc = is_max ? -INFINITY : is_min ? INFINITY : is_prod ? 1.f : 0.f;
    if (active) {
        // four independent accumulators keep several loads in flight per lane
        float a0 = acc, a1 = acc, a2 = acc, a3 = acc;
        for (int e = t; e < len4; e += TPO) {
            const float4 x = __ldg(in + e);
            if (is_max) { a0 = fmaxf(a0, x.x); a1 = fmaxf(a1, x.y); a2 = fmaxf(a2, x.z); a3 = fmaxf(a3, x.w); }
            else if (is_min) { a0 = fminf(a0, x.x); a1 = fminf(a1, x.y); a2 = fminf(a2, x.z); a3 = fminf(a3, x.w); }
            else if (is_prod) { a0 *= x.x; a1 *= x.y; a2 *= x.z; a3 *= x.w; }
            else { a0 += x.x; a1 += x.y; a2 += x.z; a3 += x.w; }
        }
        if (is_max) acc = fmaxf(fmaxf(a0, a1), fmaxf(a2, a3));
        else if (is_min) acc = fminf(fminf(a0, a1), fminf(a2, a3));
        else if (is_prod) acc = (a0 * a1) * (a2 * a3);
        else acc = (a0 + a1) + (a2 + a3);
    }
    auto combine = [&](float x, float y) { return is_max ? fmaxf(x, y) : is_min ? fminf(x, y) : is_prod ? x * y : x + y; };
#pragma unroll
    for (int s = 16; s > 0; s >>= 1) acc = combine(acc, __shfl_xor_sync(kFull, acc, s));
    if (TPO > 32) {
        const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
        if (lane == 0) smem[warp] = acc;
        __syncthreads();
        acc = lane < (TPO >> 5) ? smem[lane] : (is_max ? -INFINITY : is_min ? INFINITY : is_prod ? 1.f : 0.f);
#pragma unroll
        for (int s = 16; s > 0; s >>= 1) acc = combine(acc, __shfl_xor_sync(kFull, acc, s));
    }
    if (active && t == 0) {
        if (rop == ReduceOp::Mean) acc = acc / p.mean_scale;
        ((float*)p.out)[oo] = acc;
    }
}

// ------------------------------------------------------------------ reduce
__device__ __forceinline__ uint64_t reduce_identity(ReduceOp op, DType d) {
    const bool is_float = d == DType::F32 || d == DType::F64 || d == DType::F16;
    switch (op) {
        case ReduceOp::Sum: case ReduceOp::Mean: return is_float ? float_pattern(d, 0.0) : 0ull;
        case ReduceOp::Prod: return is_float ? float_pattern(d, 1.0) : 1ull;
        default: break;
    }
    const bool want_max_value = op == ReduceOp::Min;   // identity of min is the largest value
    if (is_float) return float_pattern(d, want_max_value ? (double)INFINITY : -(double)INFINITY);
    switch (d) {
        case DType::I8: return (uint64_t)(int64_t)(want_max_value ? INT8_MAX : INT8_MIN);
        case DType::I16: return (uint64_t)(int64_t)(want_max_value ? INT16_MAX : INT16_MIN);
        case DType::I32: return (uint64_t)(int64_t)(want_max_value ? INT32_MAX : INT32_MIN);
        case DType::I64: return (uint64_t)(want_max_value ? INT64_MAX : INT64_MIN);
        case DType::U8: return want_max_value ? 0xFFull : 0ull;
        case DType::U16: return want_max_value ? 0xFFFFull : 0ull;
        case DType::U32: return want_max_value ? 0xFFFFFFFFull : 0ull;
        case DType::U64: return want_max_value ? ~0ull : 0ull;
        default: return want_max_value ? 1ull : 0ull;   // Bool
    }
}

__device__ __forceinline__ BinaryOp reduce_binary(ReduceOp op) {
    switch (op) {
        case ReduceOp::Sum: case ReduceOp::Mean: return BinaryOp::Add;
        case ReduceOp::Prod: return BinaryOp::Mul;
        case ReduceOp::Max: return BinaryOp::Max;
        default: return BinaryOp::Min;
    }
}

// TPO threads cooperate on one output element.
template <int TPO>
__global__ void __launch_bounds__(256) reduce_kernel(const __grid_constant__ ReduceParams p) {
    pdl_enter();
    __shared__ uint64_t smem[8];
    const int outs_per_block = 256 / TPO;
    const int64_t o = (int64_t)blockIdx.x * outs_per_block + threadIdx.x / TPO;
    const int t = threadIdx.x % TPO;
    const bool active = o < p.n_out;
    const DType d = (DType)p.dtype;
    const ReduceOp rop = (ReduceOp)p.op;
    const BinaryOp bop = reduce_binary(rop);

    int64_t oi = 0, oo = 0;
    if (active) decode_offsets(o, p.kept_rank, p.kept_dims, p.kept_in_strides, p.kept_out_strides, oi, oo);

    uint64_t acc = reduce_identity(rop, d);
    if (active) {
        for (int64_t r = t; r < p.n_red; r += TPO) {
            int64_t ri = 0, dummy = 0;
            decode_offsets(r, p.red_rank, p.red_dims, p.red_strides, p.red_strides, ri, dummy);
            acc = binary_bits(bop, d, acc, load_bits(p.in, d, oi + ri));
        }
    }
#pragma unroll
    for (int s = 16; s > 0; s >>= 1) acc = binary_bits(bop, d, acc, __shfl_xor_sync(kFull, acc, s));
    if (TPO > 32) {
        const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
        if (lane == 0) smem[warp] = acc;
        __syncthreads();
        acc = lane < (TPO >> 5) ? smem[lane] : reduce_identity(rop, d);
#pragma unroll
        for (int s = 16; s > 0; s >>= 1) acc = binary_bits(bop, d, acc, __shfl_xor_sync(kFull, acc, s));
    }
    if (active && t == 0) {
        if (rop == ReduceOp::Mean) acc = f32_to_bits(bits_to_f32(acc) / p.mean_scale);
        store_bits(p.out, d, oo, acc);
    }
}

}  // namespace

static bool row_vec4_ok_len(const RowParams& p, int64_t max_len) {
    if (p.len % 4 != 0 || p.in_axis_stride != 1 || p.out_axis_stride != 1 || p.len > max_len) return false;
    if (((uintptr_t)p.in0 & 15) || ((uintptr_t)p.out & 15) || (p.in1 && ((uintptr_t)p.in1 & 15))) return false;
    for (int d = 0; d < p.outer_rank; d++)
        if (p.in_strides[d] % 4 != 0 || p.out_strides[d] % 4 != 0) return false;
    return true;
}
static bool row_vec4_ok(const RowParams& p) { return row_vec4_ok_len(p, 8192); }

// softmax's additive term is read 128 bits at a time like the input
static bool softmax_vec4_ok(const RowParams& p) {
    if (!row_vec4_ok(p)) return false;
    if (p.in1 == nullptr) return true;
    if (p.in1_axis_stride != 1) return false;
    for (int d = 0; d < p.outer_rank; d++)
        if (p.in1_strides[d] % 4 != 0) return false;
    return true;
}

#define KN_ROW_VEC4_CASE(KERNEL, TPR, N)                     \
    case N: launch_pdl(KERNEL<TPR, N>, dim3(grid), dim3(256), (size_t)(0), stream, p); break;

#define KN_ROW_DISPATCH(KERNEL, VEC4, STREAMING, OK)                                                            \
    if (p.rows == 0 || p.len == 0) return 0;                                                                   \
    if (p.rows > 0x7FFFFFFFll) return (int)cudaErrorInvalidValue;                                              \
    const int64_t len = p.len;                                                                                 \
    if (OK(p)) {                                                                                               \
        const int len4 = (int)(len / 4);                                                                       \
        if (len4 > 256 && len4 <= 512) {                                                                       \
            /* four warps per row (a block of 128 threads), three or four float4 per thread */                  \
            const unsigned grid = (unsigned)p.rows;                                                            \
            if (len4 <= 384) launch_pdl(VEC4<128, 3>, dim3(grid), dim3(128), (size_t)(0), stream, p);           \
            else launch_pdl(VEC4<128, 4>, dim3(grid), dim3(128), (size_t)(0), stream, p);                       \
        } else if (len4 <= 512) {                                                                              \
            /* one warp per row, the row in registers (up to 8 float4 per lane) */                             \
            const unsigned grid = (unsigned)((p.rows + 7) / 8);                                                \
            const int items = (len4 + 31) / 32;                                                                \
            switch (items <= 8 ? items : (items + 1) / 2 * 2) {                                                \
                KN_ROW_VEC4_CASE(VEC4, 32, 1) KN_ROW_VEC4_CASE(VEC4, 32, 2) KN_ROW_VEC4_CASE(VEC4, 32, 3)      \
                KN_ROW_VEC4_CASE(VEC4, 32, 4) KN_ROW_VEC4_CASE(VEC4, 32, 5) KN_ROW_VEC4_CASE(VEC4, 32, 6)      \
                KN_ROW_VEC4_CASE(VEC4, 32, 7) KN_ROW_VEC4_CASE(VEC4, 32, 10) KN_ROW_VEC4_CASE(VEC4, 32, 12)    \
                KN_ROW_VEC4_CASE(VEC4, 32, 14) KN_ROW_VEC4_CASE(VEC4, 32, 16)                                  \
                default: launch_pdl(VEC4<32, 8>, dim3(grid), dim3(256), (size_t)(0), stream, p); break;                                      \
            }                                                                                                  \
        } else {                                                                                               \
            const unsigned grid = (unsigned)p.rows;                                                            \
            switch ((len4 + 255) / 256) {                                                                      \
                KN_ROW_VEC4_CASE(VEC4, 256, 2) KN_ROW_VEC4_CASE(VEC4, 256, 3) KN_ROW_VEC4_CASE(VEC4, 256, 4)   \
                KN_ROW_VEC4_CASE(VEC4, 256, 5) KN_ROW_VEC4_CASE(VEC4, 256, 6) KN_ROW_VEC4_CASE(VEC4, 256, 7)   \
                default: launch_pdl(VEC4<256, 8>, dim3(grid), dim3(256), (size_t)(0), stream, p); break;                                     \
            }                                                                                                  \
        }                                                                                                      \
        return (int)cudaGetLastError();                                                                        \
    }                                                                                                          \
    if (len <= 1024) {                                                                                         \
        const int rows_per_block = 8;                                                                          \
        const unsigned grid = (unsigned)((p.rows + rows_per_block - 1) / rows_per_block);                      \
        if (len <= 32) launch_pdl(KERNEL<32, 1>, dim3(grid), dim3(256), (size_t)(0), stream, p);                                             \
        else if (len <= 64) launch_pdl(KERNEL<32, 2>, dim3(grid), dim3(256), (size_t)(0), stream, p);                                        \
        else if (len <= 128) launch_pdl(KERNEL<32, 4>, dim3(grid), dim3(256), (size_t)(0), stream, p);                                       \
        else if (len <= 256) launch_pdl(KERNEL<32, 8>, dim3(grid), dim3(256), (size_t)(0), stream, p);                                       \
        else if (len <= 512) launch_pdl(KERNEL<32, 16>, dim3(grid), dim3(256), (size_t)(0), stream, p);                                      \
        else launch_pdl(KERNEL<32, 32>, dim3(grid), dim3(256), (size_t)(0), stream, p);                                                      \
    } else if (len <= 8192) {                                                                                  \
        const unsigned grid = (unsigned)p.rows;                                                                \
        if (len <= 2048) launch_pdl(KERNEL<256, 8>, dim3(grid), dim3(256), (size_t)(0), stream, p);                                          \
        else if (len <= 4096) launch_pdl(KERNEL<256, 16>, dim3(grid), dim3(256), (size_t)(0), stream, p);                                    \
        else launch_pdl(KERNEL<256, 32>, dim3(grid), dim3(256), (size_t)(0), stream, p);                                                     \
    } else {                                                                                                   \
        launch_pdl(STREAMING, dim3((unsigned)p.rows), dim3(256), (size_t)(0), stream, p);                                                    \
    }                                                                                                          \
    return (int)cudaGetLastError();

int launch_softmax(const RowParams& p, cudaStream_t stream) {
    if (p.half) return launch_softmax_f16(p, stream);
    KN_ROW_DISPATCH(softmax_cached_kernel, softmax_vec4_kernel, softmax_streaming_kernel, softmax_vec4_ok)
}

int launch_layernorm(const RowParams& p, cudaStream_t stream) {
    if (p.half) return launch_layernorm_f16(p, stream);
    // Rows of 8193..49152 elements (a group norm over [channels / groups, H, W]): one block of 512 threads per
    // row with the row in registers, one read and one write, instead of three sweeps by the streaming kernel.
    if (p.rows > 0 && p.rows <= 0x7FFFFFFFll && p.len > 8192 && p.len <= 49152 && row_vec4_ok_len(p, 49152)) {
        const int items = (int)((p.len / 4 + 511) / 512);
        const unsigned grid = (unsigned)p.rows;
        if (items <= 8) launch_pdl(layernorm_vec4_kernel<512, 8>, dim3(grid), dim3(512), (size_t)0, stream, p);
        else if (items <= 12) launch_pdl(layernorm_vec4_kernel<512, 12>, dim3(grid), dim3(512), (size_t)0, stream, p);
        else if (items <= 16) launch_pdl(layernorm_vec4_kernel<512, 16>, dim3(grid), dim3(512), (size_t)0, stream, p);
        else if (items <= 20) launch_pdl(layernorm_vec4_kernel<512, 20>, dim3(grid), dim3(512), (size_t)0, stream, p);
        else launch_pdl(layernorm_vec4_kernel<512, 24>, dim3(grid), dim3(512), (size_t)0, stream, p);
        return (int)cudaGetLastError();
    }
    // Longer rows, up to 8 x 49152 elements: a cluster of two, four or eight CTAs per row (see layernorm_cluster_kernel).
    // The smallest cluster whose slices fit in registers, unless that leaves SMs without a CTA (few rows: the group
    // norms of a small batch), in which case a larger one.
    if (p.rows > 0 && p.rows <= (1 << 24) && p.len > 49152 && p.len <= 8 * 49152 && row_vec4_ok_len(p, 8 * 49152)) {
        int cl = 8;
        for (int c : {4, 2})
            if ((p.len + c - 1) / c <= 49152 && p.rows * c >= 2 * 148) cl = c;
        const int items = (int)(((p.len / 4 + cl - 1) / cl + 511) / 512);
#define KN_LN_CLUSTER(CL)                                                          \
        if (cl == CL) {                                                            \
            if (items <= 8) return launch_layernorm_cluster<CL, 8>(p, stream);     \
            if (items <= 16) return launch_layernorm_cluster<CL, 16>(p, stream);   \
            return launch_layernorm_cluster<CL, 24>(p, stream);                    \
        }
        KN_LN_CLUSTER(2) KN_LN_CLUSTER(4) KN_LN_CLUSTER(8)
#undef KN_LN_CLUSTER
    }
    KN_ROW_DISPATCH(layernorm_cached_kernel, layernorm_vec4_kernel, layernorm_streaming_kernel, row_vec4_ok)
}

int launch_reduce(const ReduceParams& p, cudaStream_t stream) {
    if (p.n_out == 0) return 0;
    // f32 over one contiguous, 16-byte-aligned axis: the 128-bit kernel
    bool rows = (DType)p.dtype == DType::F32 && p.red_rank == 1 && p.red_strides[0] == 1 && p.n_red % 4 == 0 && p.n_red >= 128 &&
                p.n_red < (1ll << 31) && ((uintptr_t)p.in & 15) == 0 && p.n_out <= 0x7FFFFFFFll;
    for (int d = 0; d < p.kept_rank && rows; d++) rows = p.kept_in_strides[d] % 4 == 0;
    if (rows) {
        if (p.n_red >= 8192) launch_pdl(reduce_f32_rows_kernel<256>, dim3((unsigned)p.n_out), dim3(256), (size_t)(0), stream, p);
        else launch_pdl(reduce_f32_rows_kernel<32>, dim3((unsigned)((p.n_out + 7) / 8)), dim3(256), (size_t)(0), stream, p);
        return (int)cudaGetLastError();
    }
    if (p.n_red >= 2048) {
        if (p.n_out > 0x7FFFFFFFll) return (int)cudaErrorInvalidValue;
        launch_pdl(reduce_kernel<256>, dim3((unsigned)p.n_out), dim3(256), (size_t)(0), stream, p);
    } else {
        const int64_t grid = (p.n_out + 7) / 8;
        if (grid > 0x7FFFFFFFll) return (int)cudaErrorInvalidValue;
        launch_pdl(reduce_kernel<32>, dim3((unsigned)grid), dim3(256), (size_t)(0), stream, p);
    }
    return (int)cudaGetLastError();
}

}  // namespace kn
