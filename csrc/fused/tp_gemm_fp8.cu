// Block-scaled fp8 (e4m3) tensor-parallel GEMM for sm_100a:
//     C[m, n] = sum over 128-wide K blocks kb of  sa[m, kb] * sb[n / 128, kb] * (A8[m, kb-block] . B8[n, kb-block])
// with 1 x 128 activation scales (sa: [M, K/128] fp32) and 128 x 128 weight scales (sb: [rows/128, K/128]
// fp32), the recipe named by the fp8 configuration of the tensor-parallel MLP block.
//
// Same CTA anatomy and the same communication modes as the bf16 kernel (tp_gemm.cu): TMA producer warp,
// single-thread tcgen05.mma issuer, four epilogue warps; copy CTAs that pull remote fp8 rows AND their
// scales over NVLink in allgather mode; peer-store epilogue, arrival counters and an in-kernel reduce in
// reduce-scatter mode. Two differences in the math: the tensor cores run kind::f8f6f4 on 128 x 128 x 128
// stages whose fp32 partial product lands in a fresh tensor-memory buffer (two buffers alternate), and the
// epilogue warps promote every partial product into fp32 register accumulators with the two scales while
// the next K block is already being multiplied.
// SwiGLU tiles hold 64 "gate" columns and 64 "up" columns of the same 64 output columns.
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

constexpr int      kM8 = 128, kN8 = 128, kK8 = 128, kStages8 = 6;
constexpr uint32_t kA8Bytes = kM8 * kK8, kB8Bytes = kN8 * kK8, kStage8Bytes = kA8Bytes + kB8Bytes;
constexpr uint32_t kTmemCols8 = 256;  // two 128-column partial-product buffers
static_assert(kStages8 * kStage8Bytes == kStages * kStageBytes, "same shared-memory layout as the bf16 kernel");
static_assert(kM8 == kBM, "row blocks of both kernels are 128 rows: ready flags and arrival counters are shared");

__global__ void __launch_bounds__(kThreads, 1)
tp_gemm_fp8_kernel(GemmParams p, const __grid_constant__ GemmLaunch lp)
{
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t       *smem_gen  = smem_raw + (smem_base - smem_u32(smem_raw));
    const uint32_t sA = smem_base, sB = smem_base + kStages8 * kA8Bytes;
    uint8_t       *epi_gen = smem_gen + kStages8 * kStage8Bytes;
    const uint32_t bars    = smem_base + kStages8 * kStage8Bytes + kEpiBytes;
    auto full_bar   = [&](int s) { return bars + 8u * s; };
    auto empty_bar  = [&](int s) { return bars + 8u * (kStages8 + s); };
    auto pfull_bar  = [&](int b) { return bars + 8u * (2 * kStages8 + b); };
    auto pempty_bar = [&](int b) { return bars + 8u * (2 * kStages8 + 2 + b); };
    volatile uint32_t *tmem_slot  = reinterpret_cast<volatile uint32_t *>(epi_gen + kEpiBytes + 8 * (2 * kStages8 + 4));
    volatile uint32_t *abort_slot = tmem_slot + 1;
    const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
    const int local = blockIdx.y;
    const int rank  = p.rank_base + local;
    AbortFlag ab{abort_slot, p.error, p.budget_ns};

    if (threadIdx.x == 0) *abort_slot = 0;
    __syncthreads();

    // ---- copy CTAs (allgather mode): fp8 rows and their scales
    if ((int)blockIdx.x >= p.n_gemm_ctas) {
        copy_cta_loop(p, rank, local, blockIdx.x - p.n_gemm_ctas, gridDim.x - p.n_gemm_ctas, ab, smem_base, bars);
        return;
    }

    const CUtensorMap *tmA = &lp.tmA[local], *tmB0 = &lp.tmB0[local], *tmB1 = &lp.tmB1[local];
    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages8; s++) {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), 1);
        }
        for (int b = 0; b < 2; b++) {
            mbar_init(pfull_bar(b), 1);
            mbar_init(pempty_bar(b), 4);
        }
        mbar_fence_init();
        tma_prefetch_desc(tmA);
        tma_prefetch_desc(tmB0);
        if (p.epilogue == EPI_SWIGLU) tma_prefetch_desc(tmB1);
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

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer
        if (elect_one()) {
            int      s = 0;
            uint32_t phase = 0;
            int      armed[kStages8];
            for (int i = 0; i < kStages8; i++) armed[i] = -1;
            bool ok = true;
            for (int t = blockIdx.x; t < total && ok; t += p.n_gemm_ctas) {
                const Tile tl = tile_of(p, rank, t, tiles_m, tiles_n);
                if (p.comm == COMM_ALLGATHER_A && tl.shard != rank) {
                    // rows and scales of this block are being copied in by the copy CTAs of this kernel
                    const uint32_t n_copy = gridDim.x - p.n_gemm_ctas;
                    ok = wait_counter(p.ready[local] + tl.mb, p.seq * n_copy, false, ab, 0x11);
                    asm volatile("fence.proxy.async.global;" ::: "memory");
                    if (!ok) break;
                }
                for (int kb = 0; kb < kblocks; kb++) {
                    if (!mbar_wait(empty_bar(s), phase ^ 1, ab, 0x12)) {
                        ok = false;
                        break;
                    }
                    mbar_arrive_expect_tx(full_bar(s), kStage8Bytes);
                    armed[s] = (int)phase;
                    tma_load_2d(sA + s * kA8Bytes, tmA, kb * kK8, tl.mb * kM8, full_bar(s));
                    if (p.epilogue == EPI_SWIGLU) {
                        tma_load_2d(sB + s * kB8Bytes, tmB0, kb * kK8, tl.nb * (kN8 / 2), full_bar(s));
                        tma_load_2d(sB + s * kB8Bytes + kB8Bytes / 2, tmB1, kb * kK8, tl.nb * (kN8 / 2), full_bar(s));
                    } else {
                        tma_load_2d(sB + s * kB8Bytes, tmB0, kb * kK8, tl.nb * kN8, full_bar(s));
                    }
                    if (++s == kStages8) {
                        s = 0;
                        phase ^= 1;
                    }
                }
            }
            if (!ok) {
                // let the copies that are still in flight land before the CTA goes away
                for (int i = 0; i < kStages8; i++) {
                    if (armed[i] < 0) continue;
                    for (int spin = 0; spin < (1 << 16); spin++) {
                        if (mbar_try_wait(full_bar(i), (uint32_t)armed[i])) break;
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer
        if (elect_one()) {
            const uint32_t idesc = make_idesc(0, 0, kM8, kN8);  // e4m3 x e4m3 -> fp32
            int            s = 0, buf = 0;
            uint32_t       phase = 0, pphase = 0;
            bool           ok = true;
            for (int t = blockIdx.x; t < total && ok; t += p.n_gemm_ctas) {
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
        // ------------------------------------------------------------ epilogue warps: promotion + output
        const int quarter = warp % 4;
        uint8_t  *stage   = epi_gen + (warp - 2) * 32 * kStageRowBytes;
        int       buf = 0;
        uint32_t  pphase = 0;
        const int mbs = (p.comm == COMM_NONE) ? tiles_m : tiles_m / p.tp_size;
        bool      ok  = true;
        for (int t = blockIdx.x; t < total && ok; t += p.n_gemm_ctas) {
            const Tile tl     = tile_of(p, rank, t, tiles_m, tiles_n);
            const int  row    = tl.mb * kM8 + quarter * 32 + lane;
            const bool row_ok = row < p.M;
            float      acc[kN8];
#pragma unroll
            for (int j = 0; j < kN8; j++) acc[j] = 0.0f;
            const float *sa_row = p.sg[rank] + (size_t)(row_ok ? row : 0) * kblocks;
            // plain: one 128 x 128 weight block per tile; SwiGLU: 64 gate + 64 up columns, each inside one block
            const float *sb_lo = p.sb0[local] + (size_t)(p.epilogue == EPI_SWIGLU ? tl.nb / 2 : tl.nb) * kblocks;
            const float *sb_hi = (p.epilogue == EPI_SWIGLU) ? p.sb1[local] + (size_t)(tl.nb / 2) * kblocks : sb_lo;
            for (int kb = 0; kb < kblocks; kb++) {
                if (!mbar_wait(pfull_bar(buf), pphase, ab, 0x15)) {
                    ok = false;
                    break;
                }
                tc_fence_after();
                // the scales of gathered rows arrive with the rows: read them only now that the product of this
                // K block exists (its operands were released by the copy CTAs), and from L2, not a stale L1 line
                const float a_s = row_ok ? __ldcg(sa_row + kb) : 0.0f;
                const float s_lo = a_s * sb_lo[kb], s_hi = a_s * sb_hi[kb];
                const uint32_t t_acc = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)buf * kN8;
#pragma unroll
                for (int c = 0; c < kN8 / 32; c++) {
                    uint32_t v[32];
                    tmem_ld_32x32(t_acc + (uint32_t)(c * 32), v);
                    tmem_ld_wait();
                    const float sc = (c < 2) ? s_lo : s_hi;
#pragma unroll
                    for (int j = 0; j < 32; j++) acc[c * 32 + j] = fmaf(sc, __uint_as_float(v[j]), acc[c * 32 + j]);
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(pempty_bar(buf));
                buf ^= 1;
                if (buf == 0) pphase ^= 1;
            }
            if (!ok) break;
            // destination of this tile
            __nv_bfloat16 *out;
            size_t         ld;
            int            row0;
            if (p.comm == COMM_REDUCE_SCATTER_C) {
                const size_t shard_rows = (size_t)mbs * kM8;
                out  = p.part[tl.shard] + ((size_t)(p.seq & 1) * p.tp_size + rank) * shard_rows * (size_t)p.N;
                ld   = (size_t)p.N;
                row0 = (tl.mb - tl.shard * mbs) * kM8;
            } else {
                out  = p.C[local];
                ld   = (size_t)p.ldc;
                row0 = tl.mb * kM8;
            }
            const int rows_valid = ((p.comm == COMM_REDUCE_SCATTER_C) ? mbs * kM8 : p.M) - row0;
            const int out_cols   = (p.epilogue == EPI_SWIGLU) ? kN8 / 2 : kN8;
            const int n_out      = (p.epilogue == EPI_SWIGLU) ? p.N / 2 : p.N;
            if (p.epilogue == EPI_SWIGLU) {
#pragma unroll
                for (int j = 0; j < kN8 / 2; j++) acc[j] = silu(acc[j]) * acc[kN8 / 2 + j];
            }
            // 64 output columns at a time through the transposing staging rows
            for (int oc = 0; oc < out_cols; oc += 64) {
                uint4 *rowp = reinterpret_cast<uint4 *>(stage + lane * kStageRowBytes);
#pragma unroll
                for (int j = 0; j < 8; j++) {
                    // oc is 0 or 64: constant indices after unrolling both halves
                    if (oc == 0) {
                        rowp[j] = make_uint4(pack_bf16x2(acc[8 * j], acc[8 * j + 1]), pack_bf16x2(acc[8 * j + 2], acc[8 * j + 3]),
                                             pack_bf16x2(acc[8 * j + 4], acc[8 * j + 5]), pack_bf16x2(acc[8 * j + 6], acc[8 * j + 7]));
                    } else {
                        rowp[j] = make_uint4(pack_bf16x2(acc[64 + 8 * j], acc[64 + 8 * j + 1]), pack_bf16x2(acc[64 + 8 * j + 2], acc[64 + 8 * j + 3]),
                                             pack_bf16x2(acc[64 + 8 * j + 4], acc[64 + 8 * j + 5]), pack_bf16x2(acc[64 + 8 * j + 6], acc[64 + 8 * j + 7]));
                    }
                }
                __syncwarp();
                const int col0 = tl.nb * out_cols + oc;
#pragma unroll
                for (int it = 0; it < 8; it++) {
                    const int r = it * 4 + lane / 8, chunk = lane % 8;
                    const int grow = quarter * 32 + r, gcol = col0 + chunk * 8;
                    if (grow < rows_valid && gcol < n_out) {
                        uint4 v = *reinterpret_cast<const uint4 *>(stage + r * kStageRowBytes + chunk * 16);
                        *reinterpret_cast<uint4 *>(out + (size_t)(row0 + grow) * ld + gcol) = v;
                    }
                }
                __syncwarp();
            }
            if (p.comm == COMM_REDUCE_SCATTER_C) {
                // all four epilogue warps have stored their rows: tell the owner one more tile arrived
                asm volatile("bar.sync 1, 128;" ::: "memory");
                if (warp == 2 && lane == 0) {
                    __threadfence_system();
                    uint32_t *ctr = p.pad[tl.shard] + nvl::kPadCounterOff +
                                    ((p.seq & 1) * p.tp_size + rank) * 64 + (tl.mb - tl.shard * mbs);
                    nvl::red_release_sys_add(ctr, 1u);
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, kTmemCols8);
    }
    // ---- reduce-scatter: add up the partial tiles that every rank stored for my rows
    if (p.comm == COMM_REDUCE_SCATTER_C && *abort_slot == 0) rs_reduce_phase(p, rank, local, tiles_m, ab);
}

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

xccl_status_t launch_gemm_fp8(const GemmParams &p_in, const GemmLaunch &l, cudaStream_t stream)
{
    GemmParams p = p_in;
    if (p.M <= 0 || p.N <= 0 || p.K <= 0 || p.K % kK8 != 0 || p.N % kN8 != 0) return XCCL_ERR_INVALID_PARAM;
    if (p.comm != COMM_NONE) {
        int tiles_m = (p.M + kM8 - 1) / kM8;
        if (p.M % kM8 != 0 || tiles_m % p.tp_size != 0 || tiles_m / p.tp_size > 64) return XCCL_ERR_INVALID_PARAM;
    }
    p.a_bytes = 1;
    static bool attr_set[64] = {false};
    int         dev = 0, sms = 0;
    XCCL_CUDA_CHECK(cudaGetDevice(&dev));
    XCCL_CUDA_CHECK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    if (!attr_set[dev]) {
        XCCL_CUDA_CHECK(cudaFuncSetAttribute(tp_gemm_fp8_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBytes));
        attr_set[dev] = true;
    }
    int ctas = l.ctas > 0 ? l.ctas : sms / std::max(l.n_local, 1);
    if (p.n_gemm_ctas <= 0 || p.n_gemm_ctas > ctas) p.n_gemm_ctas = ctas;
    if (p.comm == COMM_ALLGATHER_A && p.tp_size > 1 && p.n_gemm_ctas == ctas) return XCCL_ERR_INVALID_PARAM;
    if (p.error == nullptr) p.error = error_word();
    if (p.budget_ns == 0) p.budget_ns = 4000000000ull;
    if (p.group_rows <= 0) p.group_rows = 16;
    for (int i = 0; i < kMaxTpRanks; i++) p.sync_ctr[i] = nullptr;
    cudaLaunchConfig_t cfg{};
    cfg.gridDim          = dim3((unsigned)ctas, (unsigned)l.n_local);
    cfg.blockDim         = dim3(kThreads);
    cfg.dynamicSmemBytes = kSmemBytes;
    cfg.stream           = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id              = cudaLaunchAttributeCooperative;
    attr[0].val.cooperative = l.cooperative ? 1 : 0;
    cfg.attrs               = attr;
    cfg.numAttrs            = 1;
    XCCL_CUDA_CHECK(cudaLaunchKernelEx(&cfg, tp_gemm_fp8_kernel, p, l));
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
