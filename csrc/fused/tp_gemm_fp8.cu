// Block-scaled fp8 (e4m3) GEMM for sm_100a, host side:
//     C[m, n] = sum over 128-wide K blocks kb of  sa[m, kb] * sb[n / 128, kb] * (A8[m, kb-block] . B8[n, kb-block])
// with 1 x 128 activation scales (sa: [M, K/128] fp32) and 128 x 128 weight scales (sb: [rows/128, K/128]
// fp32), the recipe named by the fp8 configuration of the tensor-parallel MLP block. The kernel is the fp8
// instantiation of tp_gemm_kernel (tp_gemm.cu): same CTA pairs, tile order, lockstep and communication modes as the
// bf16 kernel. This file holds the byte tensor maps and the plain C entry point.
#include <cuda_bf16.h>

#include <algorithm>

#include "../cuda/cuda_common.h"
#include "gemm_fp8.h"
#include "sm100_ptx.cuh"
#include "tp_gemm.cuh"
#include "tp_device.cuh"

namespace xccl {
namespace tp {

namespace {
constexpr int kM8 = 128, kN8 = 128, kK8 = 128;  // rows of an A box, rows of a B box, bytes of K per box
}  // namespace

xccl_status_t make_tensor_map_u8(CUtensorMap *map, const void *base, uint64_t rows, uint64_t cols, uint32_t box_rows)
{
    XCCL_DRIVER_FN(cuTensorMapEncodeTiled);
    if (((uintptr_t)base & 15) != 0 || cols % 16 != 0) return XCCL_ERR_INVALID_PARAM;
    cuuint64_t dims[2]    = {cols, rows};
    cuuint64_t strides[1] = {cols};
    cuuint32_t box[2]     = {(cuuint32_t)kK8, box_rows};
    cuuint32_t estr[2]    = {1, 1};
    XCCL_CU_CHECK(cuTensorMapEncodeTiled(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void *>(base), dims, strides, box,
                                         estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                         CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE));
    return XCCL_OK;
}

}  // namespace tp
}  // namespace xccl

using namespace xccl;
using namespace xccl::tp;

extern "C" xccl_status_t xccl_gemm_fp8_blockscaled(const void *A8, const float *sa, const void *B8, const float *sb, void *C,
                                                   int M, int N, int K, void *stream)
{
    GemmParams p{};
    GemmLaunch l{};
    p.M = M; p.N = N; p.K = K;
    p.epilogue = EPI_STORE;
    p.comm     = COMM_NONE;
    p.tp_size  = 1;
    p.ldc      = N;
    p.C[0]     = (__nv_bfloat16 *)C;
    p.sg[0]    = const_cast<float *>(sa);
    p.sb0[0]   = sb;
    xccl_status_t st = make_tensor_map_u8(&l.tmA[0], A8, (uint64_t)M, (uint64_t)K, kM8);
    if (st != XCCL_OK) return st;
    st = make_tensor_map_u8(&l.tmB0[0], B8, (uint64_t)N, (uint64_t)K, kN8);
    if (st != XCCL_OK) return st;
    l.tmB1[0] = l.tmB0[0];
    return launch_gemm_fp8(p, l, (cudaStream_t)stream);
}
