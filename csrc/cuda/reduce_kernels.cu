// Local element-wise reductions on device buffers for sm_100a.
//
//   dst[i] = out_cast(scale * (a[i] op v_0[i] op ... op v_{n-1}[i]))
//
// One kernel covers the pairwise (n = 1) and the multi-vector form. It is bandwidth bound, so
// it moves 16 bytes per thread per access, keeps the running value in registers (fp32 for
// 16-bit floats) and issues the loads of all vectors of a pack before combining them.
// The reference has two scalar kernels for this (src/utils/cuda/kernels/xccl_cuda_reduce.cu:17-39,
// src/utils/cuda/kernels/xccl_cuda_reduce_multi.cu:17-44) limited to int16/32/64, float, double.
#include "cuda_common.h"
#include "dev_types.cuh"
#include "mem_cuda.h"

namespace xccl {

namespace {

constexpr int kThreads = 256;

template <typename T, typename O, bool kSum>
__global__ void __launch_bounds__(kThreads)
reduce_multi_kernel(const T *__restrict__ a, const T *__restrict__ vecs, O *__restrict__ dst, int n_vectors,
                    size_t count, size_t stride_elems, int op, float scale, int do_scale, int vectorised)
{
    using Tr          = dev::Traits<T>;
    using A           = typename Tr::acc;
    constexpr int E   = dev::PackOf<T>::E;
    using InPack      = dev::Pack<T, E>;
    using OutPack     = dev::Pack<O, E>;
    const size_t tid  = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t nthr = (size_t)gridDim.x * blockDim.x;
    size_t       done = 0;

    if (vectorised) {
        const size_t npacks = count / E;
        for (size_t p = tid; p < npacks; p += nthr) {
            InPack x = reinterpret_cast<const InPack *>(a)[p];
            A      acc[E];
#pragma unroll
            for (int e = 0; e < E; e++) acc[e] = Tr::up(x.v[e]);
            int k = 0;
            for (; k + 4 <= n_vectors; k += 4) {
                InPack y[4];
#pragma unroll
                for (int u = 0; u < 4; u++) {
                    y[u] = reinterpret_cast<const InPack *>(vecs + (size_t)(k + u) * stride_elems)[p];
                }
#pragma unroll
                for (int u = 0; u < 4; u++) {
#pragma unroll
                    for (int e = 0; e < E; e++) acc[e] = dev::combine<T, kSum>(op, acc[e], Tr::up(y[u].v[e]));
                }
            }
            for (; k < n_vectors; k++) {
                InPack y = reinterpret_cast<const InPack *>(vecs + (size_t)k * stride_elems)[p];
#pragma unroll
                for (int e = 0; e < E; e++) acc[e] = dev::combine<T, kSum>(op, acc[e], Tr::up(y.v[e]));
            }
            OutPack out;
#pragma unroll
            for (int e = 0; e < E; e++) out.v[e] = dev::to_out<O>(dev::scaled(acc[e], scale, do_scale != 0));
            reinterpret_cast<OutPack *>(dst)[p] = out;
        }
        done = npacks * E;
    }
    for (size_t i = done + tid; i < count; i += nthr) {
        A acc = Tr::up(a[i]);
        for (int k = 0; k < n_vectors; k++) {
            acc = dev::combine<T, kSum>(op, acc, Tr::up(vecs[(size_t)k * stride_elems + i]));
        }
        dst[i] = dev::to_out<O>(dev::scaled(acc, scale, do_scale != 0));
    }
}

template <typename T, typename O>
xccl_status_t launch(const void *a, const void *vecs, void *dst, size_t n_vectors, size_t count, size_t stride_bytes,
                     xccl_op_t op, float scale, cudaStream_t stream)
{
    if (count == 0) return XCCL_OK;
    if (stride_bytes % sizeof(T) != 0) return XCCL_ERR_INVALID_PARAM;
    constexpr int E        = dev::PackOf<T>::E;
    const size_t  out_pack = sizeof(dev::Pack<O, E>) >= 16 ? 16 : sizeof(dev::Pack<O, E>);
    int vectorised = ((uintptr_t)a % 16 == 0) && ((uintptr_t)vecs % 16 == 0) && (stride_bytes % 16 == 0) &&
                     ((uintptr_t)dst % out_pack == 0);
    size_t work  = vectorised ? (count + E - 1) / E : count;
    size_t want  = (work + kThreads - 1) / kThreads;
    int    grid  = (int)(want < (size_t)(148 * 8) ? want : (size_t)(148 * 8));
    int    dosc  = (scale != 1.0f);
    size_t selem = stride_bytes / sizeof(T);
    if (op == XCCL_OP_SUM) {
        reduce_multi_kernel<T, O, true><<<grid, kThreads, 0, stream>>>((const T *)a, (const T *)vecs, (O *)dst,
                                                                       (int)n_vectors, count, selem, (int)op, scale,
                                                                       dosc, vectorised);
    } else {
        reduce_multi_kernel<T, O, false><<<grid, kThreads, 0, stream>>>((const T *)a, (const T *)vecs, (O *)dst,
                                                                        (int)n_vectors, count, selem, (int)op, scale,
                                                                        dosc, vectorised);
    }
    XCCL_CUDA_CHECK(cudaGetLastError());
    return XCCL_OK;
}

bool op_ok(xccl_dt_t dt, xccl_op_t op)
{
    bool arith = (op == XCCL_OP_MAX || op == XCCL_OP_MIN || op == XCCL_OP_SUM || op == XCCL_OP_PROD);
    bool logic = (op >= XCCL_OP_AND && op <= XCCL_OP_BXOR);
    bool is_f  = (dt == XCCL_DT_FLOAT16 || dt == XCCL_DT_FLOAT32 || dt == XCCL_DT_FLOAT64 || dt == XCCL_DT_BFLOAT16);
    return is_f ? arith : (arith || logic);
}

}  // namespace

xccl_status_t cuda_reduce_multi(const void *a, const void *vecs, void *dst, size_t n_vectors, size_t count,
                                size_t stride_bytes, xccl_dt_t dt, xccl_op_t op, float scale, xccl_dt_t out_dt,
                                void *stream)
{
    if (!op_ok(dt, op)) return XCCL_ERR_UNSUPPORTED;
    cudaStream_t s = (cudaStream_t)stream;
    return XCCL_DISPATCH_IO(dt, out_dt, return launch<T, O>(a, vecs, dst, n_vectors, count, stride_bytes, op, scale, s););
}

}  // namespace xccl
