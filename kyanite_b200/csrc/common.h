// Shared basics: dtypes, scalar values, error type.
#pragma once
#include <cstdint>
#include <cstring>
#include <stdexcept>
#include <string>
#include <vector>

namespace kn {

// Element types of the graph IR.  0..10 are the reference's types in its declaration order
// (kn-graph/src/dtype.rs:25-37); F16 is a storage-only extension.
enum class DType : uint8_t { F32 = 0, F64, I8, I16, I32, I64, U8, U16, U32, U64, Bool, F16, COUNT };

inline int dtype_size(DType d) {
    switch (d) {
        case DType::F32: case DType::I32: case DType::U32: return 4;
        case DType::F64: case DType::I64: case DType::U64: return 8;
        case DType::I16: case DType::U16: case DType::F16: return 2;
        case DType::I8: case DType::U8: case DType::Bool: return 1;
        default: return 0;
    }
}
inline bool dtype_is_float(DType d) { return d == DType::F32 || d == DType::F64 || d == DType::F16; }
inline bool dtype_is_int(DType d) { return d >= DType::I8 && d <= DType::U64; }
inline bool dtype_is_signed(DType d) {
    return dtype_is_float(d) || d == DType::I8 || d == DType::I16 || d == DType::I32 || d == DType::I64;
}
const char* dtype_name(DType d);

enum class UnaryOp : uint8_t { Abs = 0, Neg, Sin, Cos, Exp, Log, Sqrt, Sigmoid, Tanh, Erf, Mish, Softplus, ValueCast, BitCast };
enum class BinaryOp : uint8_t { Add = 0, Sub, Mul, Div, Min, Max, Pow };
enum class ReduceOp : uint8_t { Sum = 0, Mean, Prod, Max, Min };

// Every failure inside the library is reported as this exception and converted to a status code
// plus a thread-local message at the C boundary; nothing aborts the process or traps the device.
struct Error : std::runtime_error {
    int code;
    Error(int code_, const std::string& msg) : std::runtime_error(msg), code(code_) {}
};

[[noreturn]] void fail(int code, const std::string& msg);

#define KN_CHECK(cond, code, msg)                       \
    do {                                                \
        if (!(cond)) ::kn::fail((code), (msg));         \
    } while (0)

}  // namespace kn
