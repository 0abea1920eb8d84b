// Exact-f32 contraction kernels on the SIMT pipes: batched matrix multiply and 2D convolution
// (as an implicit GEMM) with the fused `act(x + add1 + add2)` epilogue.
//
// These serve KN_MATH_F32 and every contraction shape the tensor-core kernels do not take
// (arbitrary operand strides, stride/padding combinations, tiny extents).  Operands are addressed
// through their element strides, so transposed, sliced, flipped or broadcast inputs need no copy.
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "../kernels.h"
#include <utility>

#include "epilogue.cuh"
#include "launch.cuh"

namespace kn {

namespace {

constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4;

__device__ __forceinline__ float apply_epilogue(float v, int act, int round_tf32) {
    v = apply_activation(v, act);
    if (round_tf32) {
        uint32_t u;
        asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(u) : "f"(v));
        v = __uint_as_float(u);
    }
    return v;
}

struct GemmProblem {
    GemmParams p;
    __device__ int64_t M() const { return p.m; }
    __device__ int64_t N() const { return p.n; }
    __device__ int64_t K() const { return p.k; }
    __device__ bool a_k_fast() const { return p.sa[2] == 1; }
    __device__ bool b_k_fast() const { return p.sb[1] == 1; }
    __device__ float load_a(int64_t b, int64_t m, int64_t k) const { return p.a[b * p.sa[0] + m * p.sa[1] + k * p.sa[2]]; }
    __device__ float load_b(int64_t b, int64_t k, int64_t n) const { return p.b[b * p.sb[0] + k * p.sb[1] + n * p.sb[2]]; }
    __device__ void store(int64_t b, int64_t m, int64_t n, float acc) const {
        if (p.add1) acc += p.add1[b * p.s1[0] + m * p.s1[1] + n * p.s1[2]];
        if (p.add2) acc += p.add2[b * p.s2[0] + m * p.s2[1] + n * p.s2[2]];
        p.c[b * p.sc[0] + m * p.sc[1] + n * p.sc[2]] = apply_epilogue(acc, p.act, p.round_tf32);
    }
};

// The same problem with f16 storage: operands and addends are converted on load, products accumulate in f32,
// the result is rounded to f16 once.
struct GemmProblemHalf {
    GemmParams p;
    __device__ int64_t M() const { return p.m; }
    __device__ int64_t N() const { return p.n; }
    __device__ int64_t K() const { return p.k; }
    __device__ bool a_k_fast() const { return p.sa[2] == 1; }
    __device__ bool b_k_fast() const { return p.sb[1] == 1; }
    __device__ float load_a(int64_t b, int64_t m, int64_t k) const {
        return __half2float(((const __half*)p.a)[b * p.sa[0] + m * p.sa[1] + k * p.sa[2]]);
    }
    __device__ float load_b(int64_t b, int64_t k, int64_t n) const {
        return __half2float(((const __half*)p.b)[b * p.sb[0] + k * p.sb[1] + n * p.sb[2]]);
    }
    __device__ void store(int64_t b, int64_t m, int64_t n, float acc) const {
        if (p.add1) acc += __half2float(((const __half*)p.add1)[b * p.s1[0] + m * p.s1[1] + n * p.s1[2]]);
        if (p.add2) acc += __half2float(((const __half*)p.add2)[b * p.s2[0] + m * p.s2[1] + n * p.s2[2]]);
        ((__half*)p.c)[b * p.sc[0] + m * p.sc[1] + n * p.sc[2]] = __float2half_rn(apply_activation(acc, p.act));
    }
};

struct ConvProblem {
    ConvParams p;
    __device__ int64_t M() const { return (int64_t)p.n * p.oh * p.ow; }
    __device__ int64_t N() const { return p.k; }
    __device__ int64_t K() const { return (int64_t)p.c * p.r * p.s; }
    __device__ bool a_k_fast() const { return false; }
    __device__ bool b_k_fast() const { return true; }
    __device__ float load_a(int64_t, int64_t m, int64_t kk) const {
        const int ox = (int)(m % p.ow);
        const int64_t t = m / p.ow;
        const int oy = (int)(t % p.oh);
        const int64_t img = t / p.oh;
        const int fx = (int)(kk % p.s);
        const int64_t u = kk / p.s;
        const int fy = (int)(u % p.r);
        const int64_t ci = u / p.r;
        const int iy = oy * p.stride_y + fy - p.pad_y;
        const int ix = ox * p.stride_x + fx - p.pad_x;
        if (iy < 0 || iy >= p.h || ix < 0 || ix >= p.w) return 0.0f;
        return p.in[img * p.s_in[0] + ci * p.s_in[1] + iy * p.s_in[2] + ix * p.s_in[3]];
    }
    __device__ float load_b(int64_t, int64_t kk, int64_t n) const {
        const int fx = (int)(kk % p.s);
        const int64_t u = kk / p.s;
        const int fy = (int)(u % p.r);
        const int64_t ci = u / p.r;
        return p.filter[n * p.s_f[0] + ci * p.s_f[1] + fy * p.s_f[2] + fx * p.s_f[3]];
    }
    __device__ void store(int64_t, int64_t m, int64_t n, float acc) const {
        const int64_t ox = m % p.ow;
        const int64_t t = m / p.ow;
        const int64_t oy = t % p.oh;
        const int64_t img = t / p.oh;
        if (p.add1) acc += p.add1[img * p.s1[0] + n * p.s1[1] + oy * p.s1[2] + ox * p.s1[3]];
        if (p.add2) acc += p.add2[img * p.s2[0] + n * p.s2[1] + oy * p.s2[2] + ox * p.s2[3]];
        p.out[img * p.s_out[0] + n * p.s_out[1] + oy * p.s_out[2] + ox * p.s_out[3]] = apply_epilogue(acc, p.act, p.round_tf32);
    }
};

template <class Problem>
__global__ void __launch_bounds__(256) contract_simt_kernel(const __grid_constant__ Problem prob) {
    pdl_enter();
    __shared__ float As[BK][BM + 4];
    __shared__ float Bs[BK][BN + 4];
    const int64_t M = prob.M(), N = prob.N(), K = prob.K();
    const int64_t batch = blockIdx.z;
    const int64_t m0 = (int64_t)blockIdx.x * BM, n0 = (int64_t)blockIdx.y * BN;
    const int tid = threadIdx.x;
    const int tx = tid % (BN / TN), ty = tid / (BN / TN);
    const bool a_k_fast = prob.a_k_fast(), b_k_fast = prob.b_k_fast();

    float acc[TM][TN];
#pragma unroll
    for (int i = 0; i < TM; i++)
#pragma unroll
        for (int j = 0; j < TN; j++) acc[i][j] = 0.0f;

    for (int64_t k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
        for (int i = 0; i < (BM * BK) / 256; i++) {
            const int e = tid + i * 256;
            const int mm = a_k_fast ? e / BK : e % BM;
            const int kk = a_k_fast ? e % BK : e / BM;
            const int64_t m = m0 + mm, k = k0 + kk;
            As[kk][mm] = (m < M && k < K) ? prob.load_a(batch, m, k) : 0.0f;
        }
#pragma unroll
        for (int i = 0; i < (BN * BK) / 256; i++) {
            const int e = tid + i * 256;
            const int nn = b_k_fast ? e / BK : e % BN;
            const int kk = b_k_fast ? e % BK : e / BN;
            const int64_t n = n0 + nn, k = k0 + kk;
            Bs[kk][nn] = (n < N && k < K) ? prob.load_b(batch, k, n) : 0.0f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < BK; kk++) {
            float a[TM], b[TN];
#pragma unroll
            for (int i = 0; i < TM; i++) a[i] = As[kk][ty * TM + i];
#pragma unroll
            for (int j = 0; j < TN; j++) b[j] = Bs[kk][tx * TN + j];
#pragma unroll
            for (int i = 0; i < TM; i++)
#pragma unroll
                for (int j = 0; j < TN; j++) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < TM; i++) {
        const int64_t m = m0 + ty * TM + i;
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < TN; j++) {
            const int64_t n = n0 + tx * TN + j;
            if (n < N) prob.store(batch, m, n, acc[i][j]);
        }
    }
}

template <class Problem>
int launch(const Problem& prob, int64_t M, int64_t N, int64_t batch, cudaStream_t stream) {
    if (M == 0 || N == 0 || batch == 0) return 0;
    const int64_t gx = (M + BM - 1) / BM, gy = (N + BN - 1) / BN;
    if (gy > 65535 || batch > 65535 || gx > 0x7FFFFFFFll) return (int)cudaErrorInvalidValue;
    dim3 grid((unsigned)gx, (unsigned)gy, (unsigned)batch);
    launch_pdl(contract_simt_kernel<Problem>, dim3(grid), dim3(256), (size_t)(0), stream, prob);
    return (int)cudaGetLastError();
}

// Matrix multiply with very few output columns (a classifier head, n <= 8): a 64 x 64 tile would leave
// almost every thread idle and walk K serially, so one warp takes one output row instead, its lanes
// stride through K (coalesced when K is the fast axis of both operands) and a shuffle tree sums them.
constexpr int kSkinnyMaxN = 8;

__global__ void __launch_bounds__(256) gemm_skinny_kernel(const __grid_constant__ GemmParams p) {
    pdl_enter();
    const int lane = threadIdx.x & 31;
    const int64_t row_id = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row_id >= p.batch * p.m) return;
    const int64_t b = row_id / p.m, m = row_id - b * p.m;
    const float* a = p.a + b * p.sa[0] + m * p.sa[1];
    const float* w = p.b + b * p.sb[0];
    float acc[kSkinnyMaxN];
#pragma unroll
    for (int n = 0; n < kSkinnyMaxN; n++) acc[n] = 0.f;
    const bool wide = p.sa[2] == 1 && p.sb[1] == 1 && (p.k & 3) == 0 && (((uintptr_t)a | (uintptr_t)w) & 15) == 0 && (p.sb[2] & 3) == 0;
    if (wide) {
        // both operands contiguous along K: 128-bit loads, two per lane in flight for each operand row
        const int64_t k4 = p.k >> 2;
        const float4* a4 = (const float4*)a;
#pragma unroll 2
        for (int64_t k = lane; k < k4; k += 32) {
            const float4 x = __ldg(a4 + k);
#pragma unroll
            for (int n = 0; n < kSkinnyMaxN; n++)
                if (n < p.n) {
                    const float4 y = __ldg((const float4*)(w + n * p.sb[2]) + k);
                    acc[n] = fmaf(x.x, y.x, fmaf(x.y, y.y, fmaf(x.z, y.z, fmaf(x.w, y.w, acc[n]))));
                }
        }
    } else {
#pragma unroll 4
        for (int64_t k = lane; k < p.k; k += 32) {
            const float x = a[k * p.sa[2]];
#pragma unroll
            for (int n = 0; n < kSkinnyMaxN; n++)
                if (n < p.n) acc[n] = fmaf(x, w[k * p.sb[1] + n * p.sb[2]], acc[n]);
        }
    }
#pragma unroll
    for (int n = 0; n < kSkinnyMaxN; n++)
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) acc[n] += __shfl_xor_sync(0xffffffffu, acc[n], off);
#pragma unroll
    for (int n = 0; n < kSkinnyMaxN; n++) {
        if (n < p.n && lane == n) {
            float v = acc[n];
            if (p.add1) v += p.add1[b * p.s1[0] + m * p.s1[1] + n * p.s1[2]];
            if (p.add2) v += p.add2[b * p.s2[0] + m * p.s2[1] + n * p.s2[2]];
            p.c[b * p.sc[0] + m * p.sc[1] + n * p.sc[2]] = apply_epilogue(v, p.act, p.round_tf32);
        }
    }
}

}  // namespace

int launch_gemm_simt(const GemmParams& p, cudaStream_t stream) {
    if (p.half) return launch(GemmProblemHalf{p}, p.m, p.n, p.batch, stream);
    if (p.n >= 1 && p.n <= kSkinnyMaxN && p.k >= 32 && p.batch * p.m > 0) {
        const int64_t rows = p.batch * p.m;
        launch_pdl(gemm_skinny_kernel, dim3((unsigned)((rows + 7) / 8)), dim3(256), (size_t)(0), stream, p);
        return (int)cudaGetLastError();
    }
    if (p.m >= 1 && p.m <= kSkinnyMaxN && p.k >= 32 && p.batch * p.n > 0) {
        // few output ROWS (a single token through a linear layer): the same kernel on the transposed problem,
        // C^T = B^T . A^T, one warp per output column
        GemmParams t = p;
        t.a = p.b;
        t.b = p.a;
        t.m = p.n;
        t.n = p.m;
        const int64_t sa[3] = {p.sb[0], p.sb[2], p.sb[1]}, sb[3] = {p.sa[0], p.sa[2], p.sa[1]};
        for (int i = 0; i < 3; i++) {
            t.sa[i] = sa[i];
            t.sb[i] = sb[i];
        }
        std::swap(t.sc[1], t.sc[2]);
        std::swap(t.s1[1], t.s1[2]);
        std::swap(t.s2[1], t.s2[2]);
        const int64_t rows = t.batch * t.m;
        launch_pdl(gemm_skinny_kernel, dim3((unsigned)((rows + 7) / 8)), dim3(256), (size_t)(0), stream, t);
        return (int)cudaGetLastError();
    }
    return launch(GemmProblem{p}, p.m, p.n, p.batch, stream);
}

int launch_conv_simt(const ConvParams& p, cudaStream_t stream) {
    return launch(ConvProblem{p}, (int64_t)p.n * p.oh * p.ow, p.k, 1, stream);
}

}  // namespace kn
