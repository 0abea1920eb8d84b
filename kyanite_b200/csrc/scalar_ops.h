// Element semantics shared by host constant folding and the device kernels.
//
// Values travel as canonical 64-bit patterns: signed ints sign-extended, unsigned ints and Bool
// zero-extended, F32 in the low 32 bits, F16 in the low 16 bits, F64 in all 64 bits.
//
// The semantics restate the reference's scalar maps: `UnaryOp::map` / `BinaryOp::map`
// (kn-graph/src/graph.rs:1649-1734), `DScalar::value_cast` / `bit_cast`
// (kn-graph/src/dtype.rs:323-392) and Bool arithmetic (dtype.rs:726-757).  Two deliberate
// differences, both also present in the reference's own GPU path: `erf` is the library `erff`
// instead of the CPU's 3e-7 polynomial (kn-cuda-eval/src/planner.rs:1130-1149), and integer
// division by zero yields 0 instead of aborting.
#pragma once
#include <cmath>
#include <cstdint>

#include "common.h"

#ifdef __CUDACC__
#define KN_HD __host__ __device__ __forceinline__
#else
#define KN_HD inline
#endif

namespace kn {

KN_HD float bits_to_f32(uint64_t b) {
    uint32_t u = (uint32_t)b;
    float f;
#ifdef __CUDA_ARCH__
    f = __uint_as_float(u);
#else
    memcpy(&f, &u, 4);
#endif
    return f;
}
KN_HD uint64_t f32_to_bits(float f) {
    uint32_t u;
#ifdef __CUDA_ARCH__
    u = __float_as_uint(f);
#else
    memcpy(&u, &f, 4);
#endif
    return (uint64_t)u;
}
KN_HD double bits_to_f64(uint64_t b) {
    double d;
#ifdef __CUDA_ARCH__
    d = __longlong_as_double((long long)b);
#else
    memcpy(&d, &b, 8);
#endif
    return d;
}
KN_HD uint64_t f64_to_bits(double d) {
    uint64_t u;
#ifdef __CUDA_ARCH__
    u = (uint64_t)__double_as_longlong(d);
#else
    memcpy(&u, &d, 8);
#endif
    return u;
}

// IEEE binary16 <-> binary32 (round to nearest even), written out so host and device agree.
KN_HD float f16_bits_to_f32(uint16_t h) {
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1Fu;
    uint32_t man = h & 0x3FFu;
    uint32_t out;
    if (exp == 0) {
        if (man == 0) {
            out = sign;
        } else {
            int e = -1;
            do { man <<= 1; e++; } while ((man & 0x400u) == 0);
            out = sign | ((uint32_t)(127 - 15 - e) << 23) | ((man & 0x3FFu) << 13);
        }
    } else if (exp == 31) {
        out = sign | 0x7F800000u | (man << 13);
    } else {
        out = sign | ((exp + 127 - 15) << 23) | (man << 13);
    }
    return bits_to_f32(out);
}
KN_HD uint16_t f32_to_f16_bits(float f) {
    uint32_t x = (uint32_t)f32_to_bits(f);
    uint32_t sign = (x >> 16) & 0x8000u;
    uint32_t ax = x & 0x7FFFFFFFu;
    if (ax >= 0x7F800000u) return (uint16_t)(sign | 0x7C00u | (ax > 0x7F800000u ? 0x200u : 0u));
    if (ax >= 0x477FF000u) return (uint16_t)(sign | 0x7C00u);   // rounds to inf
    if (ax < 0x33000001u) return (uint16_t)sign;                // rounds to zero
    int32_t exp = (int32_t)(ax >> 23) - 127;
    uint32_t man = (ax & 0x7FFFFFu) | 0x800000u;
    int shift;
    uint32_t hexp;
    if (exp < -14) { shift = 13 + (-14 - exp); hexp = 0; } else { shift = 13; hexp = (uint32_t)(exp + 15); }
    uint32_t half_man = man >> shift;
    uint32_t rem = man & ((1u << shift) - 1u);
    uint32_t halfway = 1u << (shift - 1);
    uint32_t res = (hexp << 10) + (hexp ? (half_man & 0x3FFu) : half_man);
    if (rem > halfway || (rem == halfway && (res & 1u))) res++;
    return (uint16_t)(sign | res);
}

// canonical pattern of an arithmetic result of type `d` held in a wider integer
KN_HD uint64_t canon_int(DType d, uint64_t v) {
    switch (d) {
        case DType::I8: return (uint64_t)(int64_t)(int8_t)v;
        case DType::I16: return (uint64_t)(int64_t)(int16_t)v;
        case DType::I32: return (uint64_t)(int64_t)(int32_t)v;
        case DType::U8: return v & 0xFFull;
        case DType::U16: return v & 0xFFFFull;
        case DType::U32: return v & 0xFFFFFFFFull;
        case DType::Bool: return v ? 1ull : 0ull;
        default: return v;
    }
}

// numeric value of a float-typed pattern as double / pattern of a double rounded to float type `d`
KN_HD double float_value(DType d, uint64_t b) {
    if (d == DType::F32) return (double)bits_to_f32(b);
    if (d == DType::F16) return (double)f16_bits_to_f32((uint16_t)b);
    return bits_to_f64(b);
}
KN_HD uint64_t float_pattern(DType d, double v) {
    if (d == DType::F32) return f32_to_bits((float)v);
    if (d == DType::F16) return (uint64_t)f32_to_f16_bits((float)v);
    return f64_to_bits(v);
}

// low 64 bits of `trunc(x)` saturated to the i128 range, NaN -> 0 (Rust `f64 as i128` then wrap)
KN_HD uint64_t f64_to_wrapped_int(double x) {
    if (x != x) return 0;
    double ax = fabs(x);
    if (ax < 9223372036854775808.0) return (uint64_t)(int64_t)x;
    if (ax >= 1.7014118346046923e38) return x > 0 ? ~0ull : 0ull;   // i128::MAX / i128::MIN
    uint64_t b = f64_to_bits(ax);
    int e = (int)((b >> 52) & 0x7FF) - 1075;                         // value = m * 2^e, e >= 11 here
    uint64_t m = (b & 0xFFFFFFFFFFFFFull) | (1ull << 52);
    uint64_t lo = e >= 64 ? 0ull : (m << e);
    return x < 0 ? (uint64_t)(0 - lo) : lo;
}

KN_HD uint64_t value_cast_bits(DType from, DType to, uint64_t x) {
    bool from_float = from == DType::F32 || from == DType::F64 || from == DType::F16;
    bool to_float = to == DType::F32 || to == DType::F64 || to == DType::F16;
    if (from_float) {
        double yf = float_value(from, x);
        if (to_float) return float_pattern(to, yf);
        if (to == DType::Bool) return (yf != 0.0) ? 1ull : 0ull;
        return canon_int(to, f64_to_wrapped_int(yf));
    }
    // integer or bool source: canonical pattern is already the i128 value's low 64 bits
    if (to_float) {
        double yf = (from == DType::U64) ? (double)x : (double)(int64_t)x;
        return float_pattern(to, yf);
    }
    if (to == DType::Bool) return x != 0 ? 1ull : 0ull;
    return canon_int(to, x);
}

KN_HD uint64_t bit_cast_bits(DType to, uint64_t x) {
    // same byte width on both sides: re-canonicalise the raw bytes for the target type
    switch (to) {
        case DType::F32: return x & 0xFFFFFFFFull;
        case DType::F16: return x & 0xFFFFull;
        case DType::F64: return x;
        default: return canon_int(to, x);
    }
}

template <typename F>
KN_HD F float_unary(UnaryOp op, F x) {
    switch (op) {
        case UnaryOp::Abs: return fabs(x);
        case UnaryOp::Neg: return -x;
        case UnaryOp::Sin: return sin(x);
        case UnaryOp::Cos: return cos(x);
        case UnaryOp::Exp: return exp(x);
        case UnaryOp::Log: return log(x);
        case UnaryOp::Sqrt: return sqrt(x);
        case UnaryOp::Sigmoid: return (F)1 / ((F)1 + exp(-x));
        case UnaryOp::Tanh: return tanh(x);
        case UnaryOp::Erf: return erf(x);
        case UnaryOp::Mish: return x * tanh(log1p(exp(x)));
        case UnaryOp::Softplus: return log1p(exp(-fabs(x))) + fmax(x, (F)0);
        default: return x;
    }
}

KN_HD float f32_unary(UnaryOp op, float x) {
    switch (op) {
        case UnaryOp::Abs: return fabsf(x);
        case UnaryOp::Neg: return -x;
        case UnaryOp::Sin: return sinf(x);
        case UnaryOp::Cos: return cosf(x);
        case UnaryOp::Exp: return expf(x);
        case UnaryOp::Log: return logf(x);
        case UnaryOp::Sqrt: return sqrtf(x);
        case UnaryOp::Sigmoid: return 1.0f / (1.0f + expf(-x));
        case UnaryOp::Tanh: return tanhf(x);
        case UnaryOp::Erf: return erff(x);
        case UnaryOp::Mish: return x * tanhf(log1pf(expf(x)));
        case UnaryOp::Softplus: return log1pf(expf(-fabsf(x))) + fmaxf(x, 0.0f);
        default: return x;
    }
}

KN_HD float f32_binary(BinaryOp op, float a, float b) {
    switch (op) {
        case BinaryOp::Add: return a + b;
        case BinaryOp::Sub: return a - b;
        case BinaryOp::Mul: return a * b;
        case BinaryOp::Div: return a / b;
        case BinaryOp::Min: return fminf(a, b);   // NaN-ignoring, like Rust's f32::min
        case BinaryOp::Max: return fmaxf(a, b);
        case BinaryOp::Pow: return powf(a, b);
    }
    return a;
}

// `from` is the operand dtype, `to` the result dtype (they differ only for casts)
KN_HD uint64_t unary_bits(UnaryOp op, DType from, DType to, uint64_t x) {
    if (op == UnaryOp::ValueCast) return value_cast_bits(from, to, x);
    if (op == UnaryOp::BitCast) return bit_cast_bits(to, x);
    switch (from) {
        case DType::F32: return f32_to_bits(f32_unary(op, bits_to_f32(x)));
        case DType::F64: return f64_to_bits(float_unary<double>(op, bits_to_f64(x)));
        case DType::F16: return (uint64_t)f32_to_f16_bits(f32_unary(op, f16_bits_to_f32((uint16_t)x)));
        default: {
            // signed integers: wrapping abs / neg
            int64_t v = (int64_t)x;
            if (op == UnaryOp::Abs) return canon_int(from, (uint64_t)(v < 0 ? (0 - (uint64_t)v) : (uint64_t)v));
            if (op == UnaryOp::Neg) return canon_int(from, 0 - (uint64_t)v);
            return x;
        }
    }
}

KN_HD uint64_t binary_bits(BinaryOp op, DType d, uint64_t a, uint64_t b) {
    switch (d) {
        case DType::F32: return f32_to_bits(f32_binary(op, bits_to_f32(a), bits_to_f32(b)));
        case DType::F16:
            return (uint64_t)f32_to_f16_bits(f32_binary(op, f16_bits_to_f32((uint16_t)a), f16_bits_to_f32((uint16_t)b)));
        case DType::F64: {
            double x = bits_to_f64(a), y = bits_to_f64(b), r;
            switch (op) {
                case BinaryOp::Add: r = x + y; break;
                case BinaryOp::Sub: r = x - y; break;
                case BinaryOp::Mul: r = x * y; break;
                case BinaryOp::Div: r = x / y; break;
                case BinaryOp::Min: r = fmin(x, y); break;
                case BinaryOp::Max: r = fmax(x, y); break;
                default: r = pow(x, y); break;
            }
            return f64_to_bits(r);
        }
        case DType::Bool: {
            bool x = a != 0, y = b != 0, r;
            switch (op) {
                case BinaryOp::Add: case BinaryOp::Max: r = x || y; break;
                case BinaryOp::Mul: case BinaryOp::Min: r = x && y; break;
                case BinaryOp::Sub: case BinaryOp::Div: r = x && !y; break;
                default: r = x; break;
            }
            return r ? 1ull : 0ull;
        }
        default: break;
    }
    bool is_signed = d == DType::I8 || d == DType::I16 || d == DType::I32 || d == DType::I64;
    uint64_t r;
    switch (op) {
        case BinaryOp::Add: r = a + b; break;
        case BinaryOp::Sub: r = a - b; break;
        case BinaryOp::Mul: r = a * b; break;
        case BinaryOp::Div:
            if (b == 0) { r = 0; }
            else if (is_signed) {
                int64_t x = (int64_t)a, y = (int64_t)b;
                r = (y == -1) ? (0 - (uint64_t)x) : (uint64_t)(x / y);
            } else { r = a / b; }
            break;
        case BinaryOp::Min: r = is_signed ? (uint64_t)((int64_t)a < (int64_t)b ? (int64_t)a : (int64_t)b) : (a < b ? a : b); break;
        case BinaryOp::Max: r = is_signed ? (uint64_t)((int64_t)a > (int64_t)b ? (int64_t)a : (int64_t)b) : (a > b ? a : b); break;
        default: r = a; break;
    }
    return canon_int(d, r);
}

KN_HD uint64_t load_bits(const void* base, DType d, int64_t idx) {
    switch (d) {
        case DType::F32: case DType::U32: return (uint64_t)((const uint32_t*)base)[idx];
        case DType::I32: return (uint64_t)(int64_t)((const int32_t*)base)[idx];
        case DType::F64: case DType::U64: case DType::I64: return ((const uint64_t*)base)[idx];
        case DType::I16: return (uint64_t)(int64_t)((const int16_t*)base)[idx];
        case DType::U16: case DType::F16: return (uint64_t)((const uint16_t*)base)[idx];
        case DType::I8: return (uint64_t)(int64_t)((const int8_t*)base)[idx];
        case DType::Bool: return ((const uint8_t*)base)[idx] ? 1ull : 0ull;
        default: return (uint64_t)((const uint8_t*)base)[idx];
    }
}

KN_HD void store_bits(void* base, DType d, int64_t idx, uint64_t v) {
    switch (d) {
        case DType::F32: case DType::U32: case DType::I32: ((uint32_t*)base)[idx] = (uint32_t)v; break;
        case DType::F64: case DType::U64: case DType::I64: ((uint64_t*)base)[idx] = v; break;
        case DType::I16: case DType::U16: case DType::F16: ((uint16_t*)base)[idx] = (uint16_t)v; break;
        default: ((uint8_t*)base)[idx] = (uint8_t)v; break;
    }
}

}  // namespace kn
