// Host reductions for every datatype the API names (the reference covers int16/32/64, float
// and double only: src/utils/reduce.h:14-140). 16-bit floats are accumulated in fp32 and
// rounded once per output element, which is also what the GPU kernels do, so this file is
// their oracle.
#include <algorithm>
#include <cstdint>
#include <cstring>
#include <type_traits>

#include "mem.h"

namespace xccl {

namespace {

struct Half {
    uint16_t bits;
};
struct BFloat {
    uint16_t bits;
};

inline float to_float(Half h)
{
    _Float16 v;
    std::memcpy(&v, &h.bits, 2);
    return (float)v;
}
inline Half from_float(float f, Half *)
{
    _Float16 v = (_Float16)f;
    Half     h;
    std::memcpy(&h.bits, &v, 2);
    return h;
}
inline float to_float(BFloat b)
{
    uint32_t u = (uint32_t)b.bits << 16;
    float    f;
    std::memcpy(&f, &u, 4);
    return f;
}
inline BFloat from_float(float f, BFloat *)
{
    uint32_t u;
    std::memcpy(&u, &f, 4);
    if ((u & 0x7fffffffu) > 0x7f800000u) {
        return BFloat{(uint16_t)((u >> 16) | 0x40)};  // quiet NaN
    }
    u += 0x7fffu + ((u >> 16) & 1u);  // round to nearest even
    return BFloat{(uint16_t)(u >> 16)};
}

template <typename T> struct Acc { using type = T; };
template <> struct Acc<Half> { using type = float; };
template <> struct Acc<BFloat> { using type = float; };

template <typename T> inline typename Acc<T>::type load(const T &v) { return v; }
template <> inline float load<Half>(const Half &v) { return to_float(v); }
template <> inline float load<BFloat>(const BFloat &v) { return to_float(v); }

template <typename T> inline T store(typename Acc<T>::type v) { return (T)v; }
template <> inline Half store<Half>(float v) { return from_float(v, (Half *)nullptr); }
template <> inline BFloat store<BFloat>(float v) { return from_float(v, (BFloat *)nullptr); }

struct OpMax  { template <typename A> static A f(A x, A y) { return x > y ? x : y; } };
struct OpMin  { template <typename A> static A f(A x, A y) { return x < y ? x : y; } };
struct OpSum  { template <typename A> static A f(A x, A y) { return x + y; } };
struct OpProd { template <typename A> static A f(A x, A y) { return x * y; } };
struct OpLand { template <typename A> static A f(A x, A y) { return (A)(x && y); } };
struct OpLor  { template <typename A> static A f(A x, A y) { return (A)(x || y); } };
struct OpLxor { template <typename A> static A f(A x, A y) { return (A)((!x) != (!y)); } };
struct OpBand { template <typename A> static A f(A x, A y) { return x & y; } };
struct OpBor  { template <typename A> static A f(A x, A y) { return x | y; } };
struct OpBxor { template <typename A> static A f(A x, A y) { return x ^ y; } };

template <typename T, typename Op>
void run(const void *a_, const void *vecs_, void *dst_, size_t n_vectors, size_t count, size_t stride_bytes)
{
    using A       = typename Acc<T>::type;
    const T *a    = (const T *)a_;
    T       *dst  = (T *)dst_;
    for (size_t i = 0; i < count; i++) {
        A acc = load<T>(a[i]);
        for (size_t k = 0; k < n_vectors; k++) {
            const T *v = (const T *)((const char *)vecs_ + k * stride_bytes);
            acc        = Op::template f<A>(acc, load<T>(v[i]));
        }
        dst[i] = store<T>(acc);
    }
}

template <typename T>
xccl_status_t run_arith(xccl_op_t op, const void *a, const void *v, void *d, size_t n, size_t c, size_t s)
{
    switch (op) {
    case XCCL_OP_MAX: run<T, OpMax>(a, v, d, n, c, s); return XCCL_OK;
    case XCCL_OP_MIN: run<T, OpMin>(a, v, d, n, c, s); return XCCL_OK;
    case XCCL_OP_SUM: run<T, OpSum>(a, v, d, n, c, s); return XCCL_OK;
    case XCCL_OP_PROD: run<T, OpProd>(a, v, d, n, c, s); return XCCL_OK;
    default: return XCCL_ERR_UNSUPPORTED;
    }
}

template <typename T>
xccl_status_t run_integer(xccl_op_t op, const void *a, const void *v, void *d, size_t n, size_t c, size_t s)
{
    switch (op) {
    case XCCL_OP_LAND: run<T, OpLand>(a, v, d, n, c, s); return XCCL_OK;
    case XCCL_OP_LOR: run<T, OpLor>(a, v, d, n, c, s); return XCCL_OK;
    case XCCL_OP_LXOR: run<T, OpLxor>(a, v, d, n, c, s); return XCCL_OK;
    case XCCL_OP_AND:
    case XCCL_OP_BAND: run<T, OpBand>(a, v, d, n, c, s); return XCCL_OK;
    case XCCL_OP_OR:
    case XCCL_OP_BOR: run<T, OpBor>(a, v, d, n, c, s); return XCCL_OK;
    case XCCL_OP_XOR:
    case XCCL_OP_BXOR: run<T, OpBxor>(a, v, d, n, c, s); return XCCL_OK;
    default: return run_arith<T>(op, a, v, d, n, c, s);
    }
}

}  // namespace

bool host_reduce_supported(xccl_dt_t dt, xccl_op_t op)
{
    bool arith = (op == XCCL_OP_MAX || op == XCCL_OP_MIN || op == XCCL_OP_SUM || op == XCCL_OP_PROD);
    bool logic = (op >= XCCL_OP_AND && op <= XCCL_OP_BXOR);
    switch (dt) {
    case XCCL_DT_INT8: case XCCL_DT_INT16: case XCCL_DT_INT32: case XCCL_DT_INT64:
    case XCCL_DT_UINT8: case XCCL_DT_UINT16: case XCCL_DT_UINT32: case XCCL_DT_UINT64:
        return arith || logic;
    case XCCL_DT_FLOAT16: case XCCL_DT_FLOAT32: case XCCL_DT_FLOAT64: case XCCL_DT_BFLOAT16:
        return arith;
    default:
        return false;
    }
}

xccl_status_t host_reduce_multi(const void *a, const void *v, void *d, size_t n, size_t c, size_t s, xccl_dt_t dt,
                                xccl_op_t op)
{
    switch (dt) {
    case XCCL_DT_INT8: return run_integer<int8_t>(op, a, v, d, n, c, s);
    case XCCL_DT_INT16: return run_integer<int16_t>(op, a, v, d, n, c, s);
    case XCCL_DT_INT32: return run_integer<int32_t>(op, a, v, d, n, c, s);
    case XCCL_DT_INT64: return run_integer<int64_t>(op, a, v, d, n, c, s);
    case XCCL_DT_UINT8: return run_integer<uint8_t>(op, a, v, d, n, c, s);
    case XCCL_DT_UINT16: return run_integer<uint16_t>(op, a, v, d, n, c, s);
    case XCCL_DT_UINT32: return run_integer<uint32_t>(op, a, v, d, n, c, s);
    case XCCL_DT_UINT64: return run_integer<uint64_t>(op, a, v, d, n, c, s);
    case XCCL_DT_FLOAT16: return run_arith<Half>(op, a, v, d, n, c, s);
    case XCCL_DT_BFLOAT16: return run_arith<BFloat>(op, a, v, d, n, c, s);
    case XCCL_DT_FLOAT32: return run_arith<float>(op, a, v, d, n, c, s);
    case XCCL_DT_FLOAT64: return run_arith<double>(op, a, v, d, n, c, s);
    default: return XCCL_ERR_UNSUPPORTED;
    }
}

namespace {
template <typename T, typename O> void scale_cast(const void *src_, void *dst_, size_t count, float scale)
{
    const T *src = (const T *)src_;
    O       *dst = (O *)dst_;
    for (size_t i = 0; i < count; i++) {
        auto v = load<T>(src[i]);
        if constexpr (std::is_integral<decltype(v)>::value) {
            dst[i] = store<O>((typename Acc<O>::type)((float)v * scale));
        } else {
            dst[i] = store<O>((typename Acc<O>::type)(v * (decltype(v))scale));
        }
    }
}
}  // namespace

// dst[i] = out_cast(scale * src[i]): the host form of the fused collective epilogue.
xccl_status_t host_scale_cast(const void *src, xccl_dt_t dt, void *dst, xccl_dt_t out_dt, size_t count, float scale)
{
    if (out_dt == XCCL_DT_UNSUPPORTED || out_dt == XCCL_DT_LAST_PREDEFINED) out_dt = dt;
    if (out_dt == dt) {
        switch (dt) {
        case XCCL_DT_INT8: scale_cast<int8_t, int8_t>(src, dst, count, scale); return XCCL_OK;
        case XCCL_DT_INT16: scale_cast<int16_t, int16_t>(src, dst, count, scale); return XCCL_OK;
        case XCCL_DT_INT32: scale_cast<int32_t, int32_t>(src, dst, count, scale); return XCCL_OK;
        case XCCL_DT_INT64: scale_cast<int64_t, int64_t>(src, dst, count, scale); return XCCL_OK;
        case XCCL_DT_UINT8: scale_cast<uint8_t, uint8_t>(src, dst, count, scale); return XCCL_OK;
        case XCCL_DT_UINT16: scale_cast<uint16_t, uint16_t>(src, dst, count, scale); return XCCL_OK;
        case XCCL_DT_UINT32: scale_cast<uint32_t, uint32_t>(src, dst, count, scale); return XCCL_OK;
        case XCCL_DT_UINT64: scale_cast<uint64_t, uint64_t>(src, dst, count, scale); return XCCL_OK;
        case XCCL_DT_FLOAT16: scale_cast<Half, Half>(src, dst, count, scale); return XCCL_OK;
        case XCCL_DT_BFLOAT16: scale_cast<BFloat, BFloat>(src, dst, count, scale); return XCCL_OK;
        case XCCL_DT_FLOAT32: scale_cast<float, float>(src, dst, count, scale); return XCCL_OK;
        case XCCL_DT_FLOAT64: scale_cast<double, double>(src, dst, count, scale); return XCCL_OK;
        default: return XCCL_ERR_UNSUPPORTED;
        }
    }
    if (dt == XCCL_DT_FLOAT32 && out_dt == XCCL_DT_BFLOAT16) { scale_cast<float, BFloat>(src, dst, count, scale); return XCCL_OK; }
    if (dt == XCCL_DT_FLOAT32 && out_dt == XCCL_DT_FLOAT16) { scale_cast<float, Half>(src, dst, count, scale); return XCCL_OK; }
    if (dt == XCCL_DT_BFLOAT16 && out_dt == XCCL_DT_FLOAT32) { scale_cast<BFloat, float>(src, dst, count, scale); return XCCL_OK; }
    if (dt == XCCL_DT_FLOAT16 && out_dt == XCCL_DT_FLOAT32) { scale_cast<Half, float>(src, dst, count, scale); return XCCL_OK; }
    return XCCL_ERR_UNSUPPORTED;
}

xccl_status_t host_reduce(const void *a, const void *b, void *dst, size_t count, xccl_dt_t dt, xccl_op_t op)
{
    return host_reduce_multi(a, b, dst, 1, count, 0, dt, op);
}

}  // namespace xccl
