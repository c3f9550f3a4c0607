// Device-side datatype traits, reduction operators and 16-byte vector packs shared by the
// local reduction kernels and the NVLink collectives.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <type_traits>

#include "xccl/xccl.h"

namespace xccl {
namespace dev {

// Accumulator type: 16-bit floats accumulate in fp32, everything else in its own type.
template <typename T> struct Traits {
    using acc = T;
    static constexpr bool is_float = false;
    __device__ __forceinline__ static acc up(T v) { return v; }
    __device__ __forceinline__ static T   down(acc v) { return v; }
};
template <> struct Traits<float> {
    using acc = float;
    static constexpr bool is_float = true;
    __device__ __forceinline__ static acc   up(float v) { return v; }
    __device__ __forceinline__ static float down(acc v) { return v; }
};
template <> struct Traits<double> {
    using acc = double;
    static constexpr bool is_float = true;
    __device__ __forceinline__ static acc    up(double v) { return v; }
    __device__ __forceinline__ static double down(acc v) { return v; }
};
template <> struct Traits<__half> {
    using acc = float;
    static constexpr bool is_float = true;
    __device__ __forceinline__ static acc    up(__half v) { return __half2float(v); }
    __device__ __forceinline__ static __half down(acc v) { return __float2half_rn(v); }
};
template <> struct Traits<__nv_bfloat16> {
    using acc = float;
    static constexpr bool is_float = true;
    __device__ __forceinline__ static acc           up(__nv_bfloat16 v) { return __bfloat162float(v); }
    __device__ __forceinline__ static __nv_bfloat16 down(acc v) { return __float2bfloat16_rn(v); }
};

// Runtime operator on accumulators. The branch is uniform across the grid.
template <typename A, bool kFloat> struct Apply;
template <typename A> struct Apply<A, true> {
    __device__ __forceinline__ static A f(int op, A x, A y)
    {
        switch (op) {
        case XCCL_OP_MAX: return x > y ? x : y;
        case XCCL_OP_MIN: return x < y ? x : y;
        case XCCL_OP_PROD: return x * y;
        default: return x + y;
        }
    }
};
template <typename A> struct Apply<A, false> {
    __device__ __forceinline__ static A f(int op, A x, A y)
    {
        switch (op) {
        case XCCL_OP_MAX: return x > y ? x : y;
        case XCCL_OP_MIN: return x < y ? x : y;
        case XCCL_OP_PROD: return (A)(x * y);
        case XCCL_OP_LAND: return (A)(x && y);
        case XCCL_OP_LOR: return (A)(x || y);
        case XCCL_OP_LXOR: return (A)((!x) != (!y));
        case XCCL_OP_AND:
        case XCCL_OP_BAND: return (A)(x & y);
        case XCCL_OP_OR:
        case XCCL_OP_BOR: return (A)(x | y);
        case XCCL_OP_XOR:
        case XCCL_OP_BXOR: return (A)(x ^ y);
        default: return (A)(x + y);
        }
    }
};

// kSum = true compiles the operator away for the hot sum path.
template <typename T, bool kSum>
__device__ __forceinline__ typename Traits<T>::acc combine(int op, typename Traits<T>::acc x, typename Traits<T>::acc y)
{
    if (kSum) {
        return x + y;
    }
    return Apply<typename Traits<T>::acc, Traits<T>::is_float>::f(op, x, y);
}

// E elements of T moved as one aligned unit (16 bytes for the input side).
template <typename T, int E> struct alignas((sizeof(T) * E) >= 16 ? 16 : (sizeof(T) * E)) Pack {
    T v[E];
};
template <typename T> struct PackOf {
    static constexpr int E = 16 / (int)sizeof(T);
    using type             = Pack<T, E>;
};

// Conversion of an accumulator to an output element, with optional scaling.
template <typename O, typename A> __device__ __forceinline__ O to_out(A v) { return Traits<O>::down((typename Traits<O>::acc)v); }

template <typename A> __device__ __forceinline__ A scaled(A v, float scale, bool do_scale)
{
    if (!do_scale) {
        return v;
    }
    if constexpr (std::is_integral<A>::value) {
        return (A)((float)v * scale);
    } else {
        return (A)(v * (A)scale);
    }
}

}  // namespace dev

// Host-side dispatch from (input dtype, output dtype) to template arguments. Output differs
// from input only for the float casts used by gradient epilogues.
#define XCCL_DISPATCH_IO(in_dt, out_dt, ...)                                                             \
    [&]() -> xccl_status_t {                                                                             \
        xccl_dt_t _o = ((out_dt) == XCCL_DT_UNSUPPORTED || (out_dt) == XCCL_DT_LAST_PREDEFINED) ? (in_dt) : (out_dt); \
        if (_o == (in_dt)) {                                                                             \
            switch (in_dt) {                                                                             \
            case XCCL_DT_INT8: { using T = int8_t; using O = T; __VA_ARGS__ }                  \
            case XCCL_DT_INT16: { using T = int16_t; using O = T; __VA_ARGS__ }                \
            case XCCL_DT_INT32: { using T = int32_t; using O = T; __VA_ARGS__ }                \
            case XCCL_DT_INT64: { using T = int64_t; using O = T; __VA_ARGS__ }                \
            case XCCL_DT_UINT8: { using T = uint8_t; using O = T; __VA_ARGS__ }                \
            case XCCL_DT_UINT16: { using T = uint16_t; using O = T; __VA_ARGS__ }              \
            case XCCL_DT_UINT32: { using T = uint32_t; using O = T; __VA_ARGS__ }              \
            case XCCL_DT_UINT64: { using T = uint64_t; using O = T; __VA_ARGS__ }              \
            case XCCL_DT_FLOAT16: { using T = __half; using O = T; __VA_ARGS__ }               \
            case XCCL_DT_BFLOAT16: { using T = __nv_bfloat16; using O = T; __VA_ARGS__ }       \
            case XCCL_DT_FLOAT32: { using T = float; using O = T; __VA_ARGS__ }                \
            case XCCL_DT_FLOAT64: { using T = double; using O = T; __VA_ARGS__ }               \
            default: return XCCL_ERR_UNSUPPORTED;                                                        \
            }                                                                                            \
        }                                                                                                \
        if ((in_dt) == XCCL_DT_FLOAT32 && _o == XCCL_DT_BFLOAT16) { using T = float; using O = __nv_bfloat16; __VA_ARGS__ } \
        if ((in_dt) == XCCL_DT_FLOAT32 && _o == XCCL_DT_FLOAT16) { using T = float; using O = __half; __VA_ARGS__ }         \
        if ((in_dt) == XCCL_DT_BFLOAT16 && _o == XCCL_DT_FLOAT32) { using T = __nv_bfloat16; using O = float; __VA_ARGS__ } \
        if ((in_dt) == XCCL_DT_FLOAT16 && _o == XCCL_DT_FLOAT32) { using T = __half; using O = float; __VA_ARGS__ }         \
        return XCCL_ERR_UNSUPPORTED;                                                                     \
    }()

}  // namespace xccl
