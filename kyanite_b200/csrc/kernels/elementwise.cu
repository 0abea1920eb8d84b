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
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <mutex>

#include "../kernels.h"
#include "../scalar_ops.h"
#include "launch.cuh"

namespace kn {

namespace {

constexpr int kThreads = 256;
constexpr int kSlots = SCALAR_MAX_OPERANDS + SCALAR_MAX_INSTR;

template <typename I>
__global__ void __launch_bounds__(kThreads) scalar_generic_kernel(const __grid_constant__ ScalarParams p) {
    pdl_enter();
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
    pdl_enter();
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

// Programs over f16 and f32 values (the half-storage graphs: RoPE, SwiGLU, residual adds, the casts around a norm):
// operands contiguous (or broadcast) along the innermost axis, eight elements per thread and iteration, so an
// f16 operand moves as one 128-bit access and an f32 operand as two.  Values are carried as f32; an instruction
// whose result type is f16 rounds its result to f16 (the storage semantics: every f16 value is rounded once per
// operation), so the numbers equal the one-element-at-a-time kernel's.
struct F8 {
    float v[8];
};

__device__ __forceinline__ F8 load8(const void* base, DType dt, int64_t off, bool broadcast) {
    F8 r;
    if (dt == DType::F16) {
        const __half* src = (const __half*)base + off;
        if (broadcast) {
            const float x = __half2float(__ldg(src));
#pragma unroll
            for (int i = 0; i < 8; i++) r.v[i] = x;
        } else {
            const uint4 u = __ldg((const uint4*)src);
            const __half2* h = (const __half2*)&u;
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const float2 t = __half22float2(h[i]);
                r.v[2 * i] = t.x;
                r.v[2 * i + 1] = t.y;
            }
        }
    } else {
        const float* src = (const float*)base + off;
        if (broadcast) {
            const float x = __ldg(src);
#pragma unroll
            for (int i = 0; i < 8; i++) r.v[i] = x;
        } else {
            const float4 a = __ldg((const float4*)src), b = __ldg((const float4*)src + 1);
            r.v[0] = a.x; r.v[1] = a.y; r.v[2] = a.z; r.v[3] = a.w;
            r.v[4] = b.x; r.v[5] = b.y; r.v[6] = b.z; r.v[7] = b.w;
        }
    }
    return r;
}

__device__ __forceinline__ void store8(void* base, DType dt, int64_t off, const F8& x) {
    if (dt == DType::F16) {
        uint4 u;
        __half2* h = (__half2*)&u;
#pragma unroll
        for (int i = 0; i < 4; i++) h[i] = __floats2half2_rn(x.v[2 * i], x.v[2 * i + 1]);
        *(uint4*)((__half*)base + off) = u;
    } else {
        float4* dst = (float4*)((float*)base + off);
        dst[0] = make_float4(x.v[0], x.v[1], x.v[2], x.v[3]);
        dst[1] = make_float4(x.v[4], x.v[5], x.v[6], x.v[7]);
    }
}

template <typename I>
__global__ void __launch_bounds__(kThreads) scalar_vec8_kernel(const __grid_constant__ ScalarParams p) {
    pdl_enter();
    const int last = p.rank - 1;
    const I inner8 = (I)(p.dims[last] >> 3);
    const I total8 = (I)(p.total >> 3);
    const I step = (I)gridDim.x * (I)blockDim.x;
    for (I idx = (I)blockIdx.x * (I)blockDim.x + (I)threadIdx.x; idx < total8; idx += step) {
        int64_t off[SCALAR_MAX_OPERANDS];
        I rem = idx / inner8;
        const int64_t inner = (int64_t)(idx - rem * inner8) * 8;
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

        F8 slot[kSlots];
        for (int l = 0; l < p.n_loads; l++) {
            const int o = p.load_operand[l];
            slot[l] = load8(p.ptr[o], (DType)p.dtype[o], off[o], p.strides[o][last] == 0);
        }
        for (int k = 0; k < p.n_instr; k++) {
            const ScalarInstr in = p.instr[k];
            F8 r;
            if (in.kind == 0) {
                const float c = (DType)in.dtype == DType::F16 ? f16_bits_to_f32((uint16_t)in.imm) : bits_to_f32(in.imm);
#pragma unroll
                for (int i = 0; i < 8; i++) r.v[i] = c;
            } else if (in.kind == 1) {
                const F8 a = slot[in.a];
                const UnaryOp op = (UnaryOp)in.op;
                if (op == UnaryOp::ValueCast) r = a;   // f16 <-> f32: the value; rounding to f16 happens below
                else {
#pragma unroll
                    for (int i = 0; i < 8; i++) r.v[i] = f32_unary(op, a.v[i]);
                }
            } else {
                const F8 a = slot[in.a], b = slot[in.b];
                const BinaryOp op = (BinaryOp)in.op;
#pragma unroll
                for (int i = 0; i < 8; i++) r.v[i] = f32_binary(op, a.v[i], b.v[i]);
            }
            if ((DType)in.dtype == DType::F16 && in.kind != 0) {
#pragma unroll
                for (int i = 0; i < 8; i++) r.v[i] = __half2float(__float2half_rn(r.v[i]));
            }
            slot[p.n_loads + k] = r;
        }
        for (int s = 0; s < p.n_stores; s++) {
            const int o = p.store_operand[s];
            store8(p.ptr[o], (DType)p.dtype[o], off[o], slot[p.store_slot[s]]);
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

// Accumulator-program variant of the 128-bit kernel.  The slot arrays above are indexed with run-time
// indices and therefore live in local memory, which makes every instruction of the program a round trip
// through L1, and selecting among registers with switches costs more instructions than the arithmetic.
// Here every micro-op leaves its result in an accumulator that IS a register; only values that are needed
// again later are also copied to a numbered spill slot in shared memory ([slot][position][thread] float4:
// conflict-free 128-bit accesses, and the run-time slot number is just an address).  Every thread carries V
// consecutive float4 positions through the program; all loads of the program are issued first.
constexpr int kRegOperandsF32 = 4, kRegOperandsMixed = 6;   // operand addresses kept in registers

template <int V>
struct Vec {
    float4 v[V];
};

template <int V, typename F>
__device__ __forceinline__ void map1(Vec<V>& acc, const Vec<V>& a, F f) {
#pragma unroll
    for (int i = 0; i < V; i++) acc.v[i] = make_float4(f(a.v[i].x), f(a.v[i].y), f(a.v[i].z), f(a.v[i].w));
}
template <int V, typename F>
__device__ __forceinline__ void map2(Vec<V>& acc, const Vec<V>& a, const Vec<V>& b, F f) {
#pragma unroll
    for (int i = 0; i < V; i++)
        acc.v[i] = make_float4(f(a.v[i].x, b.v[i].x), f(a.v[i].y, b.v[i].y), f(a.v[i].z, b.v[i].z), f(a.v[i].w, b.v[i].w));
}

template <int V>
__device__ __forceinline__ void unary_v(UnaryOp op, Vec<V>& acc, const Vec<V>& a) {
    switch (op) {   // uniform: one branch per micro-op, the loops over positions and lanes are inside
        case UnaryOp::Abs: map1(acc, a, [](float x) { return fabsf(x); }); break;
        case UnaryOp::Neg: map1(acc, a, [](float x) { return -x; }); break;
        case UnaryOp::Exp: map1(acc, a, [](float x) { return expf(x); }); break;
        case UnaryOp::Sqrt: map1(acc, a, [](float x) { return sqrtf(x); }); break;
        case UnaryOp::Sigmoid: map1(acc, a, [](float x) { return 1.0f / (1.0f + expf(-x)); }); break;
        case UnaryOp::Tanh: map1(acc, a, [](float x) { return tanhf(x); }); break;
        case UnaryOp::Erf: map1(acc, a, [](float x) { return erff(x); }); break;
        case UnaryOp::ValueCast: acc = a; break;   // between f16 and f32 values, which travel as f32 (mixed programs only)
        default: map1(acc, a, [op](float x) { return f32_unary(op, x); }); break;
    }
}
template <int V>
__device__ __forceinline__ void binary_v(BinaryOp op, Vec<V>& acc, const Vec<V>& a, const Vec<V>& b) {
    switch (op) {
        case BinaryOp::Add: map2(acc, a, b, [](float x, float y) { return x + y; }); break;
        case BinaryOp::Sub: map2(acc, a, b, [](float x, float y) { return x - y; }); break;
        case BinaryOp::Mul: map2(acc, a, b, [](float x, float y) { return x * y; }); break;
        case BinaryOp::Div: map2(acc, a, b, [](float x, float y) { return x / y; }); break;
        case BinaryOp::Min: map2(acc, a, b, [](float x, float y) { return fminf(x, y); }); break;
        case BinaryOp::Max: map2(acc, a, b, [](float x, float y) { return fmaxf(x, y); }); break;
        default: map2(acc, a, b, [](float x, float y) { return powf(x, y); }); break;
    }
}

// round to f16 and back: the value an f16-typed result is stored as
__device__ __forceinline__ float round_f16(float x) { return __half2float(__float2half_rn(x)); }

// MIXED: operands and values may be f16 as well as f32 (V is even then).  Values travel as f32; an f16 operand is
// converted on load and store (four elements = 8 bytes per position), and a micro-op whose result type is f16
// rounds its result to f16, which is what storing every intermediate as f16 would give.
template <int V, bool RANK1, bool MIXED>
__global__ void __launch_bounds__(kThreads) scalar_acc_kernel(const __grid_constant__ ScalarParams p) {
    constexpr int kRegOperands = MIXED ? kRegOperandsMixed : kRegOperandsF32;
    pdl_enter();
    extern __shared__ float4 spill[];   // [slot][position][thread]
    const int last = p.rank - 1;
    const uint32_t inner_v = (uint32_t)(p.dims[last] / (4 * V));   // groups of V float4 along the innermost axis
    const uint32_t total_v = (uint32_t)(p.total / (4 * V));
    const uint32_t step = gridDim.x * blockDim.x;
    uint32_t inner_bytes[kRegOperands];   // bytes between two consecutive float4 positions (0 = broadcast)
    bool is_half[kRegOperands];
#pragma unroll
    for (int o = 0; o < kRegOperands; o++) {
        is_half[o] = MIXED && o < p.n_operands && (DType)p.dtype[o] == DType::F16;
        inner_bytes[o] = o < p.n_operands && p.strides[o][last] != 0 ? (is_half[o] ? 8u : 16u) : 0u;
    }
    float4* const my_spill = spill + threadIdx.x;
    auto slot_read = [&](int slot, Vec<V>& out) {
#pragma unroll
        for (int v = 0; v < V; v++) out.v[v] = my_spill[(slot * V + v) * kThreads];
    };

    for (uint32_t g = blockIdx.x * blockDim.x + threadIdx.x; g < total_v; g += step) {
        uint32_t off[kRegOperands];   // element offset of the group's first position
        if (RANK1) {
#pragma unroll
            for (int o = 0; o < kRegOperands; o++) off[o] = inner_bytes[o] ? g * (uint32_t)(4 * V) : 0u;
        } else {
            uint32_t rem = g / inner_v;
            const uint32_t inner = (g - rem * inner_v) * (uint32_t)(4 * V);
#pragma unroll
            for (int o = 0; o < kRegOperands; o++) off[o] = inner_bytes[o] ? inner : 0u;
            for (int d = last - 1; d >= 0; d--) {
                const uint32_t dim = (uint32_t)p.dims[d];
                const uint32_t q = rem / dim;
                const uint32_t i = rem - q * dim;
                rem = q;
#pragma unroll
                for (int o = 0; o < kRegOperands; o++)
                    if (o < p.n_operands) off[o] += i * (uint32_t)p.strides[o][d];
            }
        }
        const char* base[kRegOperands];
#pragma unroll
        for (int o = 0; o < kRegOperands; o++)
            base[o] = o < p.n_operands ? (const char*)p.ptr[o] + (size_t)off[o] * (is_half[o] ? 2u : 4u) : nullptr;
        auto operand = [&](int o, uint32_t* stride_bytes, bool* half) -> const char* {
            switch (o) {
                case 0: *stride_bytes = inner_bytes[0]; *half = is_half[0]; return base[0];
                case 1: *stride_bytes = inner_bytes[1]; *half = is_half[1]; return base[1];
                case 2: *stride_bytes = inner_bytes[2]; *half = is_half[2]; return base[2];
                case 3: *stride_bytes = inner_bytes[3]; *half = is_half[3]; return base[3];
                case 4: *stride_bytes = inner_bytes[kRegOperands - 2]; *half = is_half[kRegOperands - 2]; return base[kRegOperands - 2];
                default: *stride_bytes = inner_bytes[kRegOperands - 1]; *half = is_half[kRegOperands - 1]; return base[kRegOperands - 1];
            }
        };
        if (MIXED) {
            // The micro-ops run in program order, and each load is converted (and parked in its slot) before the
            // next one is issued, so a thread has one operand's 32 bytes in flight at a time: too few to cover
            // DRAM latency with 2-byte elements.  The later operands' lines are therefore requested into L2 now
            // (the loads come first in the program), and with a one-dimensional index space so is the next
            // iteration's first operand.  (Requesting every operand of the next iteration as well measured slower.)
            for (int k = 1; k < p.n_micro && p.micro[k].kind == 3; k++) {
                uint32_t sb;
                bool half;
                const char* src = operand(p.micro[k].a, &sb, &half);
                if (sb) asm volatile("prefetch.global.L2 [%0];" ::"l"(src));
            }
            if (RANK1 && g + step < total_v && p.micro[0].kind == 3) {
                uint32_t sb;
                bool half;
                const char* src = operand(p.micro[0].a, &sb, &half);
                if (sb) asm volatile("prefetch.global.L2 [%0];" ::"l"(src + (size_t)step * (4 * V) * (half ? 2u : 4u)));
            }
        }
        auto imm_value = [&](const ScalarInstr& in) {
            return MIXED && (DType)in.dtype == DType::F16 ? f16_bits_to_f32((uint16_t)in.imm) : bits_to_f32(in.imm);
        };

        Vec<V> acc;
#pragma unroll
        for (int v = 0; v < V; v++) acc.v[v] = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int k = 0; k < p.n_micro; k++) {
            const ScalarInstr in = p.micro[k];
            Vec<V> a = acc, b = acc;
            if (in.kind != 0 && in.kind != 3 && in.a != 255) slot_read(in.a, a);
            switch (in.kind) {
                case 0:
#pragma unroll
                    for (int v = 0; v < V; v++) acc.v[v] = splat(imm_value(in));
                    break;
                case 1:
                    if (MIXED && (DType)in.dtype == DType::F16 && (UnaryOp)in.op == UnaryOp::Sigmoid)
                        // the result is rounded to f16 below: the hardware exponential and reciprocal (errors near
                        // 2^-21) are exact enough, and the exact ones would bound a kernel that moves 2-byte elements
                        map1(acc, a, [](float x) { return __fdividef(1.0f, 1.0f + __expf(-x)); });
                    else
                        unary_v<V>((UnaryOp)in.op, acc, a);
                    break;
                case 2:
                    if (in.b != 255) slot_read(in.b, b);
                    binary_v<V>((BinaryOp)in.op, acc, a, b);
                    break;
                case 3: {
                    uint32_t sb;
                    bool half;
                    const char* src = operand(in.a, &sb, &half);
                    if (MIXED && half) {
                        if (sb) {
                            // 8 halves (two positions) per 128-bit load
#pragma unroll
                            for (int v = 0; v < V; v += 2) {
                                const uint4 u = __ldg((const uint4*)(src + v * 8));
                                const __half2* h = (const __half2*)&u;
                                const float2 f0 = __half22float2(h[0]), f1 = __half22float2(h[1]), f2 = __half22float2(h[2]),
                                             f3 = __half22float2(h[3]);
                                acc.v[v] = make_float4(f0.x, f0.y, f1.x, f1.y);
                                acc.v[v + 1] = make_float4(f2.x, f2.y, f3.x, f3.y);
                            }
                        } else {
                            const float4 x = splat(__half2float(__ldg((const __half*)src)));
#pragma unroll
                            for (int v = 0; v < V; v++) acc.v[v] = x;
                        }
                    } else if (sb) {
#pragma unroll
                        for (int v = 0; v < V; v++) acc.v[v] = __ldg((const float4*)(src + v * 16));
                    } else {
                        const float4 x = splat(__ldg((const float*)src));
#pragma unroll
                        for (int v = 0; v < V; v++) acc.v[v] = x;
                    }
                    break;
                }
                case 4: {
                    uint32_t sb;
                    bool half;
                    char* dst = const_cast<char*>(operand(in.b, &sb, &half));
                    if (MIXED && half) {
#pragma unroll
                        for (int v = 0; v < V; v += 2) {
                            uint4 u;
                            __half2* h = (__half2*)&u;
                            h[0] = __floats2half2_rn(a.v[v].x, a.v[v].y);
                            h[1] = __floats2half2_rn(a.v[v].z, a.v[v].w);
                            h[2] = __floats2half2_rn(a.v[v + 1].x, a.v[v + 1].y);
                            h[3] = __floats2half2_rn(a.v[v + 1].z, a.v[v + 1].w);
                            *(uint4*)(dst + v * 8) = u;
                        }
                    } else {
#pragma unroll
                        for (int v = 0; v < V; v++) *(float4*)(dst + v * 16) = a.v[v];
                    }
                    break;
                }
                case 5:
#pragma unroll
                    for (int v = 0; v < V; v++) b.v[v] = splat(imm_value(in));
                    binary_v<V>((BinaryOp)in.op, acc, a, b);
                    break;
                default:
#pragma unroll
                    for (int v = 0; v < V; v++) b.v[v] = splat(imm_value(in));
                    binary_v<V>((BinaryOp)in.op, acc, b, a);
                    break;
            }
            // (bit 8 of `pad`: only f16 stores read this result, and their rounding is the same rounding)
            if (MIXED && (DType)in.dtype == DType::F16 && !(in.pad & 0x100) && (in.kind == 1 || in.kind == 2 || in.kind >= 5)) {
#pragma unroll
                for (int v = 0; v < V; v++) {
                    const float2 lo = __half22float2(__floats2half2_rn(acc.v[v].x, acc.v[v].y));
                    const float2 hi = __half22float2(__floats2half2_rn(acc.v[v].z, acc.v[v].w));
                    acc.v[v] = make_float4(lo.x, lo.y, hi.x, hi.y);
                }
            }
            if ((in.pad & 0xFF) != 255) {
#pragma unroll
                for (int v = 0; v < V; v++) my_spill[((int)(in.pad & 0xFF) * V + v) * kThreads] = acc.v[v];
            }
        }
    }
}

template <int V, bool MIXED>
int launch_acc(const ScalarParams& p, cudaStream_t stream) {
    const int64_t groups = p.total / (4 * V);
    const int grid = grid_for(groups);
    const size_t smem = (size_t)p.n_regs * V * kThreads * sizeof(float4);
    static std::mutex mu;
    static bool done[64] = {false};   // (one set per instantiation of this template)
    int device = 0;
    cudaGetDevice(&device);
    {
        std::lock_guard<std::mutex> lock(mu);
        if (device >= 0 && device < 64 && !done[device]) {
            cudaError_t e1 = cudaFuncSetAttribute(scalar_acc_kernel<V, true, MIXED>, cudaFuncAttributeMaxDynamicSharedMemorySize, 128 * 1024);
            cudaError_t e2 = cudaFuncSetAttribute(scalar_acc_kernel<V, false, MIXED>, cudaFuncAttributeMaxDynamicSharedMemorySize, 128 * 1024);
            if (e1 != cudaSuccess) return (int)e1;
            if (e2 != cudaSuccess) return (int)e2;
            done[device] = true;
        }
    }
    if (p.rank == 1) launch_pdl(scalar_acc_kernel<V, true, MIXED>, dim3(grid), dim3(kThreads), (size_t)(smem), stream, p);
    else launch_pdl(scalar_acc_kernel<V, false, MIXED>, dim3(grid), dim3(kThreads), (size_t)(smem), stream, p);
    return (int)cudaGetLastError();
}

// ---------------------------------------------------------------- accumulator programs over f16 only
// Every operand and every value of the program is f16.  Values then travel as packed halves (eight per 128-bit
// register) and add / subtract / multiply / min / max run as half2 instructions: an f16 <-> f32 conversion issues at
// a fraction of the arithmetic rate, and the f32 route spends several per element (SwiGLU ran at 0.46 of the copy
// bandwidth on them).  The result is the same bit for bit: an IEEE half operation rounds the exact result once, the
// oracle rounds it to f32 and then to f16, and for + - x that double rounding is innocuous because 24 >= 2 * 11 + 2
// significand bits.  Everything else (division, powers, transcendental unaries) converts, computes in f32 and rounds.
template <int V>
struct VecH {
    uint4 v[V];   // 8 halves each
};

__device__ __forceinline__ uint4 splat_h(uint16_t bits) {
    const uint32_t w = (uint32_t)bits * 0x00010001u;
    return make_uint4(w, w, w, w);
}
template <typename F>
__device__ __forceinline__ uint4 map_h2(const uint4& a, const uint4& b, F f) {
    uint4 r;
    const __half2* x = (const __half2*)&a;
    const __half2* y = (const __half2*)&b;
    __half2* o = (__half2*)&r;
#pragma unroll
    for (int i = 0; i < 4; i++) o[i] = f(x[i], y[i]);
    return r;
}
// through f32: 8 halves -> two float4 -> f -> rounded back
template <typename F>
__device__ __forceinline__ uint4 via_f32(const uint4& a, const uint4& b, F f) {
    const __half2* x = (const __half2*)&a;
    const __half2* y = (const __half2*)&b;
    uint4 r;
    __half2* o = (__half2*)&r;
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const float2 p = __half22float2(x[i]), q = __half22float2(y[i]);
        o[i] = __floats2half2_rn(f(p.x, q.x), f(p.y, q.y));
    }
    return r;
}

template <int V>
__device__ __forceinline__ void unary_h(UnaryOp op, VecH<V>& acc, const VecH<V>& a) {
#pragma unroll
    for (int i = 0; i < V; i++) {
        switch (op) {   // uniform
            case UnaryOp::Neg: acc.v[i] = map_h2(a.v[i], a.v[i], [](__half2 x, __half2) { return __hneg2(x); }); break;
            case UnaryOp::Abs: acc.v[i] = map_h2(a.v[i], a.v[i], [](__half2 x, __half2) { return __habs2(x); }); break;
            // (the hardware exponential and reciprocal, errors near 2^-21: the result is rounded to f16)
            case UnaryOp::Sigmoid: acc.v[i] = via_f32(a.v[i], a.v[i], [](float x, float) { return __fdividef(1.0f, 1.0f + __expf(-x)); }); break;
            case UnaryOp::ValueCast: acc.v[i] = a.v[i]; break;
            default: acc.v[i] = via_f32(a.v[i], a.v[i], [op](float x, float) { return f32_unary(op, x); }); break;
        }
    }
}
template <int V>
__device__ __forceinline__ void binary_h(BinaryOp op, VecH<V>& acc, const VecH<V>& a, const VecH<V>& b) {
#pragma unroll
    for (int i = 0; i < V; i++) {
        switch (op) {   // uniform
            case BinaryOp::Add: acc.v[i] = map_h2(a.v[i], b.v[i], [](__half2 x, __half2 y) { return __hadd2_rn(x, y); }); break;
            case BinaryOp::Sub: acc.v[i] = map_h2(a.v[i], b.v[i], [](__half2 x, __half2 y) { return __hsub2_rn(x, y); }); break;
            case BinaryOp::Mul: acc.v[i] = map_h2(a.v[i], b.v[i], [](__half2 x, __half2 y) { return __hmul2_rn(x, y); }); break;
            case BinaryOp::Min: acc.v[i] = map_h2(a.v[i], b.v[i], [](__half2 x, __half2 y) { return __hmin2(x, y); }); break;
            case BinaryOp::Max: acc.v[i] = map_h2(a.v[i], b.v[i], [](__half2 x, __half2 y) { return __hmax2(x, y); }); break;
            case BinaryOp::Div: acc.v[i] = via_f32(a.v[i], b.v[i], [](float x, float y) { return x / y; }); break;
            default: acc.v[i] = via_f32(a.v[i], b.v[i], [](float x, float y) { return powf(x, y); }); break;
        }
    }
}

template <int V, bool RANK1>
__global__ void __launch_bounds__(kThreads) scalar_h2_kernel(const __grid_constant__ ScalarParams p) {
    constexpr int kRegOperands = kRegOperandsMixed;
    pdl_enter();
    extern __shared__ float4 spill[];   // [slot][position][thread], 16 bytes = 8 halves per entry
    uint4* const my_spill = (uint4*)spill + threadIdx.x;
    const int last = p.rank - 1;
    const uint32_t inner_v = (uint32_t)(p.dims[last] / (8 * V));   // groups of V positions along the innermost axis
    const uint32_t total_v = (uint32_t)(p.total / (8 * V));
    const uint32_t step = gridDim.x * blockDim.x;
    bool strided[kRegOperands];   // false = broadcast along the innermost axis
#pragma unroll
    for (int o = 0; o < kRegOperands; o++) strided[o] = o < p.n_operands && p.strides[o][last] != 0;
    auto slot_read = [&](int slot, VecH<V>& out) {
#pragma unroll
        for (int v = 0; v < V; v++) out.v[v] = my_spill[(slot * V + v) * kThreads];
    };

    for (uint32_t g = blockIdx.x * blockDim.x + threadIdx.x; g < total_v; g += step) {
        uint32_t off[kRegOperands];   // element offset of the group's first position
        if (RANK1) {
#pragma unroll
            for (int o = 0; o < kRegOperands; o++) off[o] = strided[o] ? g * (uint32_t)(8 * V) : 0u;
        } else {
            uint32_t rem = g / inner_v;
            const uint32_t inner = (g - rem * inner_v) * (uint32_t)(8 * V);
#pragma unroll
            for (int o = 0; o < kRegOperands; o++) off[o] = strided[o] ? inner : 0u;
            for (int d = last - 1; d >= 0; d--) {
                const uint32_t dim = (uint32_t)p.dims[d];
                const uint32_t q = rem / dim;
                const uint32_t i = rem - q * dim;
                rem = q;
#pragma unroll
                for (int o = 0; o < kRegOperands; o++)
                    if (o < p.n_operands) off[o] += i * (uint32_t)p.strides[o][d];
            }
        }
        const __half* base[kRegOperands];
#pragma unroll
        for (int o = 0; o < kRegOperands; o++) base[o] = o < p.n_operands ? (const __half*)p.ptr[o] + off[o] : nullptr;
        auto operand = [&](int o, bool* is_strided) -> const __half* {
            switch (o) {
                case 0: *is_strided = strided[0]; return base[0];
                case 1: *is_strided = strided[1]; return base[1];
                case 2: *is_strided = strided[2]; return base[2];
                case 3: *is_strided = strided[3]; return base[3];
                case 4: *is_strided = strided[4]; return base[4];
                default: *is_strided = strided[5]; return base[5];
            }
        };

        VecH<V> acc;
#pragma unroll
        for (int v = 0; v < V; v++) acc.v[v] = make_uint4(0u, 0u, 0u, 0u);
        for (int k = 0; k < p.n_micro; k++) {
            const ScalarInstr in = p.micro[k];
            VecH<V> a = acc, b = acc;
            if (in.kind != 0 && in.kind != 3 && in.a != 255) slot_read(in.a, a);
            switch (in.kind) {
                case 0:
#pragma unroll
                    for (int v = 0; v < V; v++) acc.v[v] = splat_h((uint16_t)in.imm);
                    break;
                case 1:
                    unary_h<V>((UnaryOp)in.op, acc, a);
                    break;
                case 2:
                    if (in.b != 255) slot_read(in.b, b);
                    binary_h<V>((BinaryOp)in.op, acc, a, b);
                    break;
                case 3: {
                    bool st;
                    const __half* src = operand(in.a, &st);
                    if (st) {
#pragma unroll
                        for (int v = 0; v < V; v++) acc.v[v] = __ldg((const uint4*)src + v);
                    } else {
                        const uint4 x = splat_h(__half_as_ushort(__ldg(src)));
#pragma unroll
                        for (int v = 0; v < V; v++) acc.v[v] = x;
                    }
                    break;
                }
                case 4: {
                    bool st;
                    __half* dst = const_cast<__half*>(operand(in.b, &st));
#pragma unroll
                    for (int v = 0; v < V; v++) *((uint4*)dst + v) = a.v[v];
                    break;
                }
                case 5:
#pragma unroll
                    for (int v = 0; v < V; v++) b.v[v] = splat_h((uint16_t)in.imm);
                    binary_h<V>((BinaryOp)in.op, acc, a, b);
                    break;
                default:
#pragma unroll
                    for (int v = 0; v < V; v++) b.v[v] = splat_h((uint16_t)in.imm);
                    binary_h<V>((BinaryOp)in.op, acc, b, a);
                    break;
            }
            if ((in.pad & 0xFF) != 255) {
#pragma unroll
                for (int v = 0; v < V; v++) my_spill[((int)(in.pad & 0xFF) * V + v) * kThreads] = acc.v[v];
            }
        }
    }
}

template <int V>
int launch_h2(const ScalarParams& p, cudaStream_t stream) {
    const int64_t groups = p.total / (8 * V);
    const int grid = grid_for(groups);
    const size_t smem = (size_t)p.n_regs * V * kThreads * sizeof(uint4);
    static std::mutex mu;
    static bool done[64] = {false};   // (one set per instantiation of this template)
    int device = 0;
    cudaGetDevice(&device);
    {
        std::lock_guard<std::mutex> lock(mu);
        if (device >= 0 && device < 64 && !done[device]) {
            cudaError_t e1 = cudaFuncSetAttribute(scalar_h2_kernel<V, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 128 * 1024);
            cudaError_t e2 = cudaFuncSetAttribute(scalar_h2_kernel<V, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 128 * 1024);
            if (e1 != cudaSuccess) return (int)e1;
            if (e2 != cudaSuccess) return (int)e2;
            done[device] = true;
        }
    }
    if (p.rank == 1) launch_pdl(scalar_h2_kernel<V, true>, dim3(grid), dim3(kThreads), (size_t)(smem), stream, p);
    else launch_pdl(scalar_h2_kernel<V, false>, dim3(grid), dim3(kThreads), (size_t)(smem), stream, p);
    return (int)cudaGetLastError();
}

// ---------------------------------------------------------------- transposing copy
// A plain copy of 4-byte elements whose source is contiguous along one axis (s) and whose destination is
// contiguous along another (t): a [batch, k, n] matmul operand rewritten K-contiguous, a head split.
// Read by the generic kernel, one side of it touches a 32-byte sector per element.  Here a block moves a
// 32 x 64 tile through shared memory: rows of 128 bytes on both sides, eight loads per thread in flight.
constexpr int kTransposeT = 64;   // tile extent along t (32 along s)
struct TransposeParams {
    const void* src;                // elements of 4 bytes (transpose_copy_kernel<uint32_t>) or 2 bytes (<uint16_t>: f16 storage)
    void* dst;
    int64_t ns, nt;                 // extents of the two axes
    int64_t src_t_stride, dst_s_stride;
    int64_t tiles_s, tiles_t;
    int32_t n_outer;
    int64_t outer_dims[DEV_MAX_RANK], outer_src[DEV_MAX_RANK], outer_dst[DEV_MAX_RANK];
};

template <typename T>
__global__ void __launch_bounds__(256) transpose_copy_kernel(const __grid_constant__ TransposeParams q) {
    pdl_enter();
    __shared__ T tile[kTransposeT][33 + (sizeof(T) == 2 ? 1 : 0)];   // (odd number of 4-byte words per row either way)
    int64_t rem = blockIdx.x;
    const int64_t ts = rem % q.tiles_s;
    rem /= q.tiles_s;
    const int64_t tt = rem % q.tiles_t;
    rem /= q.tiles_t;
    int64_t src_off = 0, dst_off = 0;
    for (int d = q.n_outer - 1; d >= 0; d--) {
        const int64_t i = rem % q.outer_dims[d];
        rem /= q.outer_dims[d];
        src_off += i * q.outer_src[d];
        dst_off += i * q.outer_dst[d];
    }
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    const int64_t s0 = ts * 32, t0 = tt * kTransposeT;
    T r[kTransposeT / 8];
#pragma unroll
    for (int j = 0; j < kTransposeT / 8; j++) {
        const int64_t t = t0 + ty + 8 * j, s2 = s0 + tx;
        r[j] = (t < q.nt && s2 < q.ns) ? __ldg((const T*)q.src + src_off + s2 + t * q.src_t_stride) : (T)0;
    }
#pragma unroll
    for (int j = 0; j < kTransposeT / 8; j++) tile[ty + 8 * j][tx] = r[j];
    __syncthreads();
#pragma unroll
    for (int h = 0; h < kTransposeT / 32; h++) {
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const int64_t s2 = s0 + ty + 8 * j, t = t0 + 32 * h + tx;
            if (t < q.nt && s2 < q.ns) ((T*)q.dst)[dst_off + t + s2 * q.dst_s_stride] = tile[32 * h + tx][ty + 8 * j];
        }
    }
}

// Fills `q` and returns true if `p` is such a copy.
bool as_transpose(const ScalarParams& p, TransposeParams& q) {
    if (p.n_operands != 2 || p.n_loads != 1 || p.n_instr != 0 || p.n_stores != 1 || p.rank < 2) return false;
    const int src = p.load_operand[0], dst = p.store_operand[0];
    if (src == dst || p.store_slot[0] != 0 || p.dtype[src] != p.dtype[dst]) return false;
    const DType dt = (DType)p.dtype[src];
    if (dtype_size(dt) != 4 && dtype_size(dt) != 2) return false;
    int s_axis = -1, t_axis = -1;
    for (int d = 0; d < p.rank; d++) {
        if (p.dims[d] <= 1) continue;
        if (p.strides[src][d] == 1 && s_axis < 0) s_axis = d;
        if (p.strides[dst][d] == 1 && t_axis < 0) t_axis = d;
    }
    if (s_axis < 0 || t_axis < 0 || s_axis == t_axis) return false;
    if (p.dims[s_axis] < 16 || p.dims[t_axis] < 16) return false;
    q.src = p.ptr[src];
    q.dst = p.ptr[dst];
    q.ns = p.dims[s_axis];
    q.nt = p.dims[t_axis];
    q.src_t_stride = p.strides[src][t_axis];
    q.dst_s_stride = p.strides[dst][s_axis];
    q.tiles_s = (q.ns + 31) / 32;
    q.tiles_t = (q.nt + kTransposeT - 1) / kTransposeT;
    q.n_outer = 0;
    int64_t blocks = q.tiles_s * q.tiles_t;
    for (int d = 0; d < p.rank; d++) {
        if (d == s_axis || d == t_axis || p.dims[d] <= 1) continue;
        q.outer_dims[q.n_outer] = p.dims[d];
        q.outer_src[q.n_outer] = p.strides[src][d];
        q.outer_dst[q.n_outer] = p.strides[dst][d];
        q.n_outer++;
        blocks *= p.dims[d];
    }
    return blocks < (1ll << 31);
}

}  // namespace

int launch_scalar(const ScalarParams& p, cudaStream_t stream) {
    if (p.total == 0) return 0;
    if (p.vec4 != 2 && p.vec4 != 4 && p.vec4 != 5) {
        TransposeParams q;
        if (as_transpose(p, q)) {
            int64_t blocks = q.tiles_s * q.tiles_t;
            for (int d = 0; d < q.n_outer; d++) blocks *= q.outer_dims[d];
            if (dtype_size((DType)p.dtype[p.load_operand[0]]) == 2)
                launch_pdl(transpose_copy_kernel<uint16_t>, dim3((unsigned)blocks), dim3(256), (size_t)0, stream, q);
            else
                launch_pdl(transpose_copy_kernel<uint32_t>, dim3((unsigned)blocks), dim3(256), (size_t)0, stream, q);
            return (int)cudaGetLastError();
        }
    }
    if (p.vec4 == 2) {
        // V consecutive float4 positions per thread: as many as the innermost extent and the spill slots
        // (n_regs * V * 4 KB of shared memory per block) allow
        const int64_t inner4 = p.dims[p.rank - 1] / 4;
        if (inner4 % 4 == 0 && p.n_regs <= 4) return launch_acc<4, false>(p, stream);
        if (inner4 % 2 == 0) return launch_acc<2, false>(p, stream);
        return launch_acc<1, false>(p, stream);
    } else if (p.vec4 == 5) {
        // an accumulator program over f16 only: packed halves, eight per position (the innermost extent is a multiple
        // of 8, the planner's condition); four positions per thread when the extent and the spill slots allow
        const int64_t inner8 = p.dims[p.rank - 1] / 8;
        if (inner8 % 4 == 0 && p.n_regs <= 4) return launch_h2<4>(p, stream);
        if (inner8 % 2 == 0) return launch_h2<2>(p, stream);
        return launch_h2<1>(p, stream);
    } else if (p.vec4 == 4) {
        // f16 / f32 mix as an accumulator program: the innermost extent is a multiple of 8 (the planner's condition)
        const int64_t inner4 = p.dims[p.rank - 1] / 4;
        if (inner4 % 4 == 0 && p.n_regs <= 4) return launch_acc<4, true>(p, stream);
        return launch_acc<2, true>(p, stream);
    } else if (p.vec4 == 3) {
        const int64_t total8 = p.total >> 3;
        if (total8 < (1ll << 31)) launch_pdl(scalar_vec8_kernel<uint32_t>, dim3(grid_for(total8)), dim3(kThreads), (size_t)(0), stream, p);
        else launch_pdl(scalar_vec8_kernel<uint64_t>, dim3(grid_for(total8)), dim3(kThreads), (size_t)(0), stream, p);
    } else if (p.vec4) {
        const int64_t total4 = p.total >> 2;
        if (total4 < (1ll << 31)) launch_pdl(scalar_vec4_kernel<uint32_t>, dim3(grid_for(total4)), dim3(kThreads), (size_t)(0), stream, p);
        else launch_pdl(scalar_vec4_kernel<uint64_t>, dim3(grid_for(total4)), dim3(kThreads), (size_t)(0), stream, p);
    } else {
        if (p.total < (1ll << 31)) launch_pdl(scalar_generic_kernel<uint32_t>, dim3(grid_for(p.total)), dim3(kThreads), (size_t)(0), stream, p);
        else launch_pdl(scalar_generic_kernel<uint64_t>, dim3(grid_for(p.total)), dim3(kThreads), (size_t)(0), stream, p);
    }
    return (int)cudaGetLastError();
}

}  // namespace kn
