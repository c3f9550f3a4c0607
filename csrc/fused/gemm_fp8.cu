// Block-scaled fp8 (e4m3) GEMM for sm_100a:  C[M,N] (bf16) = sum over 128-wide K blocks kb of
//     sa[m, kb] * sb[n / 128, kb] * (A8[m, kb-block] . B8[n, kb-block])
// with 1 x 128 activation scales (sa: [M, K/128] fp32) and 128 x 128 weight scales
// (sb: [N/128, K/128] fp32), the DeepSeek-style recipe named by the TP-MLP fp8 config.
//
// Same CTA anatomy as the bf16 kernel (TMA producer warp, single-thread tcgen05.mma issuer, four
// epilogue warps) with two differences: the tensor cores run kind::f8f6f4 on 128 x 128 x 128 stages
// whose fp32 partial product lands in a fresh tensor-memory buffer (two buffers alternate), and
// the epilogue warps promote every partial product into fp32 register accumulators with the two
// scales while the next K block is already being multiplied.
#include <cuda_bf16.h>

#include <algorithm>

#include "../cuda/cuda_common.h"
#include "gemm_fp8.h"
#include "sm100_ptx.cuh"
#include "tp_gemm.cuh"

namespace xccl {
namespace tp {

using namespace sm100;

namespace {

constexpr int      kM8 = 128, kN8 = 128, kK8 = 128, kStages8 = 6;
constexpr uint32_t kA8Bytes = kM8 * kK8, kB8Bytes = kN8 * kK8, kStage8Bytes = kA8Bytes + kB8Bytes;
constexpr uint32_t kRowBytes = 144, kEpi8Bytes = 4 * 32 * kRowBytes;
constexpr uint32_t kSmem8Bytes = kStages8 * kStage8Bytes + kEpi8Bytes + 256 + 1024;
constexpr uint32_t kTmemCols8 = 256;  // two 128-column partial-product buffers

struct Fp8Params {
    int          M, N, K, ldc;
    const float *sa, *sb;
    __nv_bfloat16 *C;
    uint32_t    *error;
    unsigned long long budget_ns;
};

__device__ __forceinline__ uint32_t pack2(float lo, float hi)
{
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t *>(&v);
}

__global__ void __launch_bounds__(kThreads, 1)
gemm_fp8_kernel(Fp8Params p, const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB)
{
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t       *smem_gen  = smem_raw + (smem_base - smem_u32(smem_raw));
    const uint32_t sA = smem_base, sB = smem_base + kStages8 * kA8Bytes;
    uint8_t       *epi_gen = smem_gen + kStages8 * kStage8Bytes;
    const uint32_t bars    = smem_base + kStages8 * kStage8Bytes + kEpi8Bytes;
    auto full_bar   = [&](int s) { return bars + 8u * s; };
    auto empty_bar  = [&](int s) { return bars + 8u * (kStages8 + s); };
    auto pfull_bar  = [&](int b) { return bars + 8u * (2 * kStages8 + b); };
    auto pempty_bar = [&](int b) { return bars + 8u * (2 * kStages8 + 2 + b); };
    volatile uint32_t *tmem_slot  = reinterpret_cast<volatile uint32_t *>(epi_gen + kEpi8Bytes + 8 * (2 * kStages8 + 4));
    volatile uint32_t *abort_slot = tmem_slot + 1;
    const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
    AbortFlag ab{abort_slot, p.error, p.budget_ns};

    if (threadIdx.x == 0) {
        *abort_slot = 0;
        for (int s = 0; s < kStages8; s++) {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), 1);
        }
        for (int b = 0; b < 2; b++) {
            mbar_init(pfull_bar(b), 1);
            mbar_init(pempty_bar(b), 4);
        }
        mbar_fence_init();
        tma_prefetch_desc(&tmA);
        tma_prefetch_desc(&tmB);
    }
    if (warp == 1) {
        tmem_alloc(smem_u32((const void *)tmem_slot), kTmemCols8);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    const int tiles_m = (p.M + kM8 - 1) / kM8, tiles_n = (p.N + kN8 - 1) / kN8;
    const int total   = tiles_m * tiles_n;
    const int kblocks = p.K / kK8;
    // groups of 16 row blocks share the same weight tiles while they are hot in L2
    auto tile_of = [&](int t, int &mb, int &nb) {
        const int group = 16 * tiles_n, g = t / group, within = t % group;
        const int gm = min(16, tiles_m - g * 16);
        mb = g * 16 + within % gm;
        nb = within / gm;
    };

    if (warp == 0) {
        if (elect_one()) {
            int      s = 0;
            uint32_t phase = 0;
            int      armed[kStages8];
            for (int i = 0; i < kStages8; i++) armed[i] = -1;
            bool ok = true;
            for (int t = blockIdx.x; t < total && ok; t += gridDim.x) {
                int mb, nb;
                tile_of(t, mb, nb);
                for (int kb = 0; kb < kblocks; kb++) {
                    if (!mbar_wait(empty_bar(s), phase ^ 1, ab, 0x12)) {
                        ok = false;
                        break;
                    }
                    mbar_arrive_expect_tx(full_bar(s), kStage8Bytes);
                    armed[s] = (int)phase;
                    tma_load_2d(sA + s * kA8Bytes, &tmA, kb * kK8, mb * kM8, full_bar(s));
                    tma_load_2d(sB + s * kB8Bytes, &tmB, kb * kK8, nb * kN8, full_bar(s));
                    if (++s == kStages8) {
                        s = 0;
                        phase ^= 1;
                    }
                }
            }
            if (!ok) {
                for (int i = 0; i < kStages8; i++) {
                    if (armed[i] < 0) continue;
                    for (int spin = 0; spin < (1 << 16); spin++) {
                        if (mbar_try_wait(full_bar(i), (uint32_t)armed[i])) break;
                    }
                }
            }
        }
    } else if (warp == 1) {
        if (elect_one()) {
            const uint32_t idesc = make_idesc(0, 0, kM8, kN8);  // e4m3 x e4m3 -> fp32
            int            s = 0, buf = 0;
            uint32_t       phase = 0, pphase = 0;
            bool           ok = true;
            for (int t = blockIdx.x; t < total && ok; t += gridDim.x) {
                for (int kb = 0; kb < kblocks; kb++) {
                    if (!mbar_wait(pempty_bar(buf), pphase ^ 1, ab, 0x13) || !mbar_wait(full_bar(s), phase, ab, 0x14)) {
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t d  = tmem_base + (uint32_t)buf * kN8;
                    const uint64_t da = make_desc_sw128(sA + s * kA8Bytes), db = make_desc_sw128(sB + s * kB8Bytes);
#pragma unroll
                    for (int k = 0; k < kK8 / 32; k++) {
                        // 32 fp8 values = 32 bytes further along K inside the 128-byte swizzle row
                        mma_f8(d, da + (uint64_t)(k * 2), db + (uint64_t)(k * 2), idesc, k != 0);
                    }
                    mma_commit(empty_bar(s));
                    mma_commit(pfull_bar(buf));
                    if (++s == kStages8) {
                        s = 0;
                        phase ^= 1;
                    }
                    buf ^= 1;
                    if (buf == 0) pphase ^= 1;
                }
            }
        }
    } else {
        const int quarter = warp % 4;
        uint8_t  *stage   = epi_gen + (warp - 2) * 32 * kRowBytes;
        int       buf = 0;
        uint32_t  pphase = 0;
        const int kb_stride = kblocks;  // sa is [M, K/128], sb is [N/128, K/128]
        bool      ok = true;
        for (int t = blockIdx.x; t < total && ok; t += gridDim.x) {
            int mb, nb;
            tile_of(t, mb, nb);
            const int  row    = mb * kM8 + quarter * 32 + lane;
            const bool row_ok = row < p.M;
            float      acc[kN8];
#pragma unroll
            for (int j = 0; j < kN8; j++) acc[j] = 0.0f;
            const float *sa_row = p.sa + (size_t)(row_ok ? row : 0) * kb_stride;
            const float *sb_row = p.sb + (size_t)nb * kb_stride;
            for (int kb = 0; kb < kblocks; kb++) {
                const float scale = (row_ok ? sa_row[kb] : 0.0f) * sb_row[kb];
                if (!mbar_wait(pfull_bar(buf), pphase, ab, 0x15)) {
                    ok = false;
                    break;
                }
                tc_fence_after();
                const uint32_t t_acc = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)buf * kN8;
#pragma unroll
                for (int c = 0; c < kN8 / 32; c++) {
                    uint32_t v[32];
                    tmem_ld_32x32(t_acc + (uint32_t)(c * 32), v);
                    tmem_ld_wait();
#pragma unroll
                    for (int j = 0; j < 32; j++) acc[c * 32 + j] = fmaf(scale, __uint_as_float(v[j]), acc[c * 32 + j]);
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(pempty_bar(buf));
                buf ^= 1;
                if (buf == 0) pphase ^= 1;
            }
            if (!ok) break;
            // write the tile: two passes of 64 columns through the transposing staging rows
#pragma unroll
            for (int oc = 0; oc < kN8; oc += 64) {
                uint4 *rowp = reinterpret_cast<uint4 *>(stage + lane * kRowBytes);
#pragma unroll
                for (int j = 0; j < 8; j++) {
                    rowp[j] = make_uint4(pack2(acc[oc + 8 * j], acc[oc + 8 * j + 1]), pack2(acc[oc + 8 * j + 2], acc[oc + 8 * j + 3]),
                                         pack2(acc[oc + 8 * j + 4], acc[oc + 8 * j + 5]), pack2(acc[oc + 8 * j + 6], acc[oc + 8 * j + 7]));
                }
                __syncwarp();
#pragma unroll
                for (int it = 0; it < 8; it++) {
                    const int r = it * 4 + lane / 8, chunk = lane % 8;
                    const int grow = mb * kM8 + quarter * 32 + r, gcol = nb * kN8 + oc + chunk * 8;
                    if (grow < p.M && gcol < p.N) {
                        uint4 v = *reinterpret_cast<const uint4 *>(stage + r * kRowBytes + chunk * 16);
                        *reinterpret_cast<uint4 *>(p.C + (size_t)grow * p.ldc + gcol) = v;
                    }
                }
                __syncwarp();
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, kTmemCols8);
    }
}

xccl_status_t make_map_u8(CUtensorMap *map, const void *base, uint64_t rows, uint64_t cols, uint32_t box_rows)
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

}  // namespace

}  // namespace tp
}  // namespace xccl

using namespace xccl;
using namespace xccl::tp;

extern "C" xccl_status_t xccl_gemm_fp8_blockscaled(const void *A8, const float *sa, const void *B8, const float *sb, void *C,
                                                   int M, int N, int K, void *stream)
{
    if (M <= 0 || N <= 0 || K <= 0 || K % kK8 != 0 || N % kN8 != 0) return XCCL_ERR_INVALID_PARAM;
    CUtensorMap   tmA, tmB;
    xccl_status_t st = make_map_u8(&tmA, A8, (uint64_t)M, (uint64_t)K, kM8);
    if (st != XCCL_OK) return st;
    st = make_map_u8(&tmB, B8, (uint64_t)N, (uint64_t)K, kN8);
    if (st != XCCL_OK) return st;
    Fp8Params p{};
    p.M = M; p.N = N; p.K = K; p.ldc = N;
    p.sa = sa; p.sb = sb;
    p.C         = (__nv_bfloat16 *)C;
    p.error     = error_word();
    p.budget_ns = 4000000000ull;
    static bool attr_set[64] = {false};
    int         dev = 0, sms = 0;
    XCCL_CUDA_CHECK(cudaGetDevice(&dev));
    XCCL_CUDA_CHECK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    if (!attr_set[dev]) {
        XCCL_CUDA_CHECK(cudaFuncSetAttribute(gemm_fp8_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmem8Bytes));
        attr_set[dev] = true;
    }
    gemm_fp8_kernel<<<sms, kThreads, kSmem8Bytes, (cudaStream_t)stream>>>(p, tmA, tmB);
    XCCL_CUDA_CHECK(cudaGetLastError());
    return XCCL_OK;
}
