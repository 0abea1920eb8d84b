// Fused elementwise kernels: one launch evaluates a whole Unary/Binary expression tree over N
// strided operands (any rank, stride 0 = broadcast, negative = flip) and doubles as the strided
// copy.  Takes the place of the reference's runtime-compiled `scalar_kernel`
// (kn-cuda-eval/src/autokernel/scalar.cu:13-26): the expression arrives as a register program in
// the launch parameters instead of generated source.
//
// Two variants:
//   scalar_generic_kernel  any dtype mix, one element per thread iteration, 64-bit value slots.
//   scalar_vec4_kernel     all-f32 programs whose operands are contiguous (or broadcast) along the
//                          innermost axis: 128-bit loads and stores, four elements per iteration.
#include <cuda_runtime.h>

#include "../kernels.h"
#include "../scalar_ops.h"

namespace kn {

namespace {

constexpr int kThreads = 256;
constexpr int kSlots = SCALAR_MAX_OPERANDS + SCALAR_MAX_INSTR;

template <typename I>
__global__ void __launch_bounds__(kThreads) scalar_generic_kernel(const __grid_constant__ ScalarParams p) {
    const I total = (I)p.total;
    const I step = (I)gridDim.x * (I)blockDim.x;
    for (I idx = (I)blockIdx.x * (I)blockDim.x + (I)threadIdx.x; idx < total; idx += step) {
        int64_t off[SCALAR_MAX_OPERANDS];
#pragma unroll
        for (int o = 0; o < SCALAR_MAX_OPERANDS; o++) off[o] = 0;
        I rem = idx;
        for (int d = p.rank - 1; d >= 0; d--) {
            const I dim = (I)p.dims[d];
            const I q = rem / dim;
            const int64_t i = (int64_t)(rem - q * dim);
            rem = q;
            for (int o = 0; o < p.n_operands; o++) off[o] += i * p.strides[o][d];
        }

        uint64_t slot[kSlots];
        for (int l = 0; l < p.n_loads; l++) {
            const int o = p.load_operand[l];
            slot[l] = load_bits(p.ptr[o], (DType)p.dtype[o], off[o]);
        }
        for (int k = 0; k < p.n_instr; k++) {
            const ScalarInstr in = p.instr[k];
            uint64_t r;
            if (in.kind == 0) r = in.imm;
            else if (in.kind == 1) r = unary_bits((UnaryOp)in.op, (DType)in.from, (DType)in.dtype, slot[in.a]);
            else r = binary_bits((BinaryOp)in.op, (DType)in.dtype, slot[in.a], slot[in.b]);
            slot[p.n_loads + k] = r;
        }
        for (int s = 0; s < p.n_stores; s++) {
            const int o = p.store_operand[s];
            store_bits(p.ptr[o], (DType)p.dtype[o], off[o], slot[p.store_slot[s]]);
        }
    }
}

__device__ __forceinline__ float4 splat(float v) { return make_float4(v, v, v, v); }

template <typename I>
__global__ void __launch_bounds__(kThreads) scalar_vec4_kernel(const __grid_constant__ ScalarParams p) {
    const int last = p.rank - 1;
    const I inner4 = (I)(p.dims[last] >> 2);
    const I total4 = (I)(p.total >> 2);
    const I step = (I)gridDim.x * (I)blockDim.x;
    for (I idx = (I)blockIdx.x * (I)blockDim.x + (I)threadIdx.x; idx < total4; idx += step) {
        int64_t off[SCALAR_MAX_OPERANDS];
        I rem = idx / inner4;
        const int64_t inner = (int64_t)(idx - rem * inner4) * 4;
#pragma unroll
        for (int o = 0; o < SCALAR_MAX_OPERANDS; o++) off[o] = 0;
        for (int o = 0; o < p.n_operands; o++) off[o] = inner * p.strides[o][last];
        for (int d = last - 1; d >= 0; d--) {
            const I dim = (I)p.dims[d];
            const I q = rem / dim;
            const int64_t i = (int64_t)(rem - q * dim);
            rem = q;
            for (int o = 0; o < p.n_operands; o++) off[o] += i * p.strides[o][d];
        }

        float4 slot[kSlots];
        for (int l = 0; l < p.n_loads; l++) {
            const int o = p.load_operand[l];
            const float* src = (const float*)p.ptr[o] + off[o];
            slot[l] = p.strides[o][last] == 0 ? splat(__ldg(src)) : __ldg((const float4*)src);
        }
        for (int k = 0; k < p.n_instr; k++) {
            const ScalarInstr in = p.instr[k];
            float4 r;
            if (in.kind == 0) {
                r = splat(bits_to_f32(in.imm));
            } else if (in.kind == 1) {
                const float4 a = slot[in.a];
                const UnaryOp op = (UnaryOp)in.op;
                r = make_float4(f32_unary(op, a.x), f32_unary(op, a.y), f32_unary(op, a.z), f32_unary(op, a.w));
            } else {
                const float4 a = slot[in.a], b = slot[in.b];
                const BinaryOp op = (BinaryOp)in.op;
                r = make_float4(f32_binary(op, a.x, b.x), f32_binary(op, a.y, b.y), f32_binary(op, a.z, b.z),
                                f32_binary(op, a.w, b.w));
            }
            slot[p.n_loads + k] = r;
        }
        for (int s = 0; s < p.n_stores; s++) {
            const int o = p.store_operand[s];
            *(float4*)((float*)p.ptr[o] + off[o]) = slot[p.store_slot[s]];
        }
    }
}

int grid_for(int64_t work_items) {
    int64_t blocks = (work_items + kThreads - 1) / kThreads;
    const int64_t cap = 148 * 8;   // 8 resident blocks of 256 threads per SM
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    return (int)blocks;
}

}  // namespace

int launch_scalar(const ScalarParams& p, cudaStream_t stream) {
    if (p.total == 0) return 0;
    if (p.vec4) {
        const int64_t total4 = p.total >> 2;
        if (total4 < (1ll << 31)) scalar_vec4_kernel<uint32_t><<<grid_for(total4), kThreads, 0, stream>>>(p);
        else scalar_vec4_kernel<uint64_t><<<grid_for(total4), kThreads, 0, stream>>>(p);
    } else {
        if (p.total < (1ll << 31)) scalar_generic_kernel<uint32_t><<<grid_for(p.total), kThreads, 0, stream>>>(p);
        else scalar_generic_kernel<uint64_t><<<grid_for(p.total), kThreads, 0, stream>>>(p);
    }
    return (int)cudaGetLastError();
}

}  // namespace kn
