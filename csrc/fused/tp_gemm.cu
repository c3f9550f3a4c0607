// Tensor-parallel GEMM kernels for sm_100a (see tp_gemm.cuh for the operations).
//
// Default layout: CTA pairs. A cluster of two CTAs (256 threads each, 384 in fp8; one CTA per SM, persistent) owns an output tile
// of 256 x 256: tcgen05.mma.cta_group::2 (M256 N256 K16) is issued by CTA 0 of the pair and accumulates fp32 in the
// tensor memory of both CTAs. Each CTA stages its own 128 rows of A and HALF of the B tile per K block of 64, so a
// stage is 32 KB and the ring has six. When the shape or the device cannot place pairs, the same kernel runs as
// single CTAs on 128 x 256 tiles with a four-stage ring of 48 KB.
//   warp 0   one elected thread issues TMA tiled loads (128B swizzle) into the ring, guarded by full/empty
//            mbarriers; in pair mode the loads carry .cta_group::2 and both CTAs' bytes are counted on the barrier of
//            the CTA that issues the MMAs
//   warp 1   one elected thread (of CTA 0 in pair mode) issues the MMAs; tcgen05.commit releases the stage and, after
//            the last K block, hands the accumulator to the epilogue. Two accumulators (2 x 256 TMEM columns)
//            alternate so the epilogue of tile i overlaps the MMAs of tile i+1
//   warps 2-5  read their 32 TMEM lanes with tcgen05.ld, apply the epilogue (bf16 cast, silu(gate)*up, or the sum
//            with the peers' partial tiles in reduce-scatter mode), transpose through shared memory and write
//            128-byte row segments to local or peer memory
//   last two warps  allgather mode with copier warps: pull this CTA's share of the remote row blocks (idle otherwise)
// Tiles are walked in a shape-dependent order and the walkers are kept in soft lockstep so that CTAs sharing rows of A
// or B hit them in L2 together. No TMA load uses cluster multicast and no TMA load reads another GPU's memory:
// remote operands are first copied into local memory by the copy CTAs of this same kernel.
#include <algorithm>
#include <cstdio>
#include <cuda_bf16.h>
#include <cuda_fp8.h>

#include "../cuda/cuda_common.h"
#include "sm100_ptx.cuh"
#include "tp_gemm.cuh"
#include "tp_device.cuh"

namespace xccl {
namespace tp {
namespace {

// kFp8: block-scaled e4m3 operands (1 x 128 activation scales, 128 x 128 weight scales). A stage holds 128 bytes of
// K per row, which is 64 bf16 or 128 fp8 values, so both types share one shared-memory geometry. The tensor cores run
// kind::f8f6f4 and the product of ONE 128-wide K block lands in a fresh tensor-memory buffer (two alternate); eight
// promotion warps (two per TMEM lane quarter, 128 accumulator columns each) add it into fp32 registers with the two
// scales while the next K block is multiplied, and run the epilogue of the tile from those registers.
template <bool kPair, bool kFp8>
__global__ void __launch_bounds__(kFp8 ? kThreadsFp8 : kThreads, 1)
tp_gemm_kernel(GemmParams p, const __grid_constant__ GemmLaunch lp)
{
    constexpr int      kNS = kFp8 ? (kPair ? kStagesPair - 1 : kStages - 1) : (kPair ? kStagesPair : kStages);  // pipeline stages
    constexpr uint32_t kBB = kPair ? kBBytes / 2 : kBBytes;   // bytes of B per stage in this CTA
    constexpr uint32_t kSB = kABytes + kBB;                   // bytes per stage in this CTA
    constexpr int      kKE = kFp8 ? 2 * kBK : kBK;            // K elements per stage (128 bytes per row)
    constexpr int      kEpiWarps  = kFp8 ? 8 : 4;
    constexpr uint32_t kEpiBytesK = kEpiWarps * 32 * kStageRowBytes;
    // ring of stages, then the epilogue staging rows, then the barriers. The copy CTAs' ring (192 KB) must end
    // before the barriers in both layouts.
    constexpr uint32_t kRingBytes = kFp8 ? (uint32_t)(kStages * kStageBytes) - (kEpiBytesK - kEpiBytes) : (uint32_t)(kStages * kStageBytes);
    static_assert(kNS * kSB <= kRingBytes, "stages fit the ring");
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t       *smem_gen  = smem_raw + (smem_base - smem_u32(smem_raw));
    const uint32_t sA        = smem_base;
    const uint32_t sB        = smem_base + kNS * kABytes;
    uint8_t       *epi_gen   = smem_gen + kRingBytes;
    const uint32_t bars      = smem_base + kRingBytes + kEpiBytesK;
    auto full_bar       = [&](int s) { return bars + 8u * s; };
    auto empty_bar      = [&](int s) { return bars + 8u * (kNS + s); };
    auto tmem_full_bar  = [&](int a) { return bars + 8u * (2 * kNS + a); };
    auto tmem_empty_bar = [&](int a) { return bars + 8u * (2 * kNS + 2 + a); };
    volatile uint32_t *tmem_slot  = reinterpret_cast<volatile uint32_t *>(epi_gen + kEpiBytesK + 8 * (2 * kNS + 4));
    volatile uint32_t *abort_slot = tmem_slot + 1;

    const int warp  = threadIdx.x / 32, lane = threadIdx.x % 32;
    const int local = blockIdx.y;
    const int rank  = p.rank_base + local;
    AbortFlag ab{abort_slot, p.error, p.budget_ns};
    // pair mode: rank of this CTA in its cluster of two (0 issues the MMAs), tile walker per cluster
    const uint32_t cta_rank = kPair ? cluster_ctarank() : 0u;
    const int      unit     = kPair ? (int)blockIdx.x / 2 : (int)blockIdx.x;
    const int      n_units  = kPair ? p.n_gemm_ctas / 2 : p.n_gemm_ctas;

    if (threadIdx.x == 0) *abort_slot = 0;
    __syncthreads();

    constexpr int kCopierWarp0 = (kFp8 ? kThreadsFp8 : kThreads) / 32 - 2;  // the last two warps: copiers (allgather mode)

    // ---- copy CTAs (allgather mode) never touch the tensor cores
    if ((int)blockIdx.x >= p.n_gemm_ctas) {
        copy_cta_loop(p, rank, local, blockIdx.x - p.n_gemm_ctas, gridDim.x - p.n_gemm_ctas, ab, smem_base, bars);
        return;
    }

    const CUtensorMap *tmA = &lp.tmA[local], *tmB0 = &lp.tmB0[local], *tmB1 = &lp.tmB1[local];
    if (threadIdx.x == 0) {
        for (int s = 0; s < kNS; s++) {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), 1);
        }
        for (int a = 0; a < 2; a++) {
            mbar_init(tmem_full_bar(a), 1);
            mbar_init(tmem_empty_bar(a), (kPair ? 2 : 1) * kEpiWarps);  // epilogue warps of every CTA of the tile
        }
        mbar_fence_init();
        tma_prefetch_desc(tmA);
        tma_prefetch_desc(tmB0);
        if (p.epilogue == EPI_SWIGLU) tma_prefetch_desc(tmB1);
    }
    if (warp == 1) {
        if (kPair) {
            tmem_alloc_pair(smem_u32((const void *)tmem_slot), kTmemCols);
            tmem_relinquish_pair();
        } else {
            tmem_alloc(smem_u32((const void *)tmem_slot), kTmemCols);
            tmem_relinquish();
        }
    }
    tc_fence_before();
    __syncthreads();
    if (kPair) cluster_sync_all();  // the peer's barriers exist before anything is signalled across
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    const int tiles_m128 = (p.M + kBM - 1) / kBM;                        // 128-row blocks
    const int tiles_m    = kPair ? (tiles_m128 + 1) / 2 : tiles_m128;     // row blocks of a tile (256 rows in pair mode)
    const int tiles_n    = (p.N + kBN - 1) / kBN;
    const int total   = tiles_m * tiles_n;
    const int kblocks = (p.K + kKE - 1) / kKE;

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer
        if (elect_one()) {
            int      s = 0;
            uint32_t phase = 0;
            int      armed[kNS];
            for (int i = 0; i < kNS; i++) armed[i] = -1;
            bool ok = true;
            uint32_t *sync_ctr      = p.sync_ctr[local];
            const int sync_per_tile = p.sync_kblocks > 0 ? (kblocks + p.sync_kblocks - 1) / p.sync_kblocks : 1;
            int       wave          = 0;
            const uint64_t pol_last = l2_policy_evict_last(), pol_first = l2_policy_evict_first();
            const uint64_t pol_a = (p.l2_hint == 3) ? pol_first : pol_last;
            const uint64_t pol_b = (p.l2_hint == 2) ? pol_first : pol_last;
            auto load = [&](uint32_t dst, const CUtensorMap *map, int x, int y, uint32_t bar, uint64_t pol) {
                if (kPair) {
                    if (p.l2_hint != 0) tma_load_2d_pair_hint(dst, map, x, y, bar, pol);
                    else tma_load_2d_pair(dst, map, x, y, bar);
                } else {
                    if (p.l2_hint != 0) tma_load_2d_hint(dst, map, x, y, bar, pol);
                    else tma_load_2d(dst, map, x, y, bar);
                }
            };
            for (int t = unit; t < total && ok; t += n_units, wave++) {
                Tile tl = tile_of(p, rank, t, tiles_m, tiles_n);
                if (kPair) tl.mb = tl.mb * 2 + (int)cta_rank;  // this CTA's 128-row block
                if (p.comm == COMM_ALLGATHER_A && tl.shard != rank) {
                    // rows of this block are being copied in by the copy CTAs of this kernel
                    const uint32_t n_copy = p.copy_mode == 1 ? gridDim.x : gridDim.x - p.n_gemm_ctas;
                    ok = wait_counter(p.ready[local] + tl.mb, p.seq * n_copy, false, ab, 1);
                    asm volatile("fence.proxy.async.global;" ::: "memory");
                    if (!ok) break;
                } else if (p.in_ready[local] != nullptr && p.comm != COMM_REDUCE_SCATTER_C) {
                    // local rows that the copy engine is still bringing in from the host
                    const int shard_row0 = (p.comm == COMM_ALLGATHER_A) ? rank * (p.M / p.tp_size) : 0;
                    const int last_row   = min(tl.mb * kBM + kBM, p.M) - 1 - shard_row0;
                    ok = wait_counter(p.in_ready[local] + last_row / p.in_rows_per_flag, p.in_target, true, ab, 8);
                    asm volatile("fence.proxy.async.global;" ::: "memory");
                    if (!ok) break;
                }
                for (int kb = 0; kb < kblocks; kb++) {
                    if (sync_ctr != nullptr && (kb == 0 || (p.sync_kblocks > 0 && kb % p.sync_kblocks == 0))) {
                        const int point = wave * sync_per_tile + (p.sync_kblocks > 0 ? kb / p.sync_kblocks : 0);
                        if (point < p.sync_points) {
                            // walkers that have a tile in this wave
                            const uint32_t want = (uint32_t)min(n_units, total - wave * n_units);
                            if (cta_rank == 0) red_release_gpu_add(sync_ctr + point, 1u);
                            const unsigned long long t0 = now_ns();
                            while ((int32_t)(ld_acquire_gpu(sync_ctr + point) - want) < 0 &&
                                   now_ns() - t0 < p.sync_budget_ns) {}
                        }
                    }
                    if (!mbar_wait(empty_bar(s), phase ^ 1, ab, 2)) {
                        ok = false;
                        break;
                    }
                    if (kPair) {
                        // both CTAs' bytes are counted on the barrier of the CTA that issues the MMAs
                        const uint32_t fb = map_to_cta(full_bar(s), 0);
                        if (cta_rank == 0) {
                            mbar_arrive_expect_tx(full_bar(s), 2 * kSB);
                            armed[s] = (int)phase;
                        }
                        load(sA + s * kABytes, tmA, kb * kKE, tl.mb * kBM, fb, pol_a);
                        if (p.epilogue == EPI_SWIGLU) {
                            // columns 0..127 of the tile are "gate" (rank 0 stages them), 128..255 "up" (rank 1)
                            load(sB + s * kBB, cta_rank == 0 ? tmB0 : tmB1, kb * kKE, tl.nb * (kBN / 2), fb, pol_b);
                        } else {
                            load(sB + s * kBB, tmB0, kb * kKE, tl.nb * kBN + (int)cta_rank * (kBN / 2), fb, pol_b);
                        }
                    } else {
                        mbar_arrive_expect_tx(full_bar(s), kSB);
                        armed[s] = (int)phase;
                        load(sA + s * kABytes, tmA, kb * kKE, tl.mb * kBM, full_bar(s), pol_a);
                        if (p.epilogue == EPI_SWIGLU) {
                            load(sB + s * kBB, tmB0, kb * kKE, tl.nb * (kBN / 2), full_bar(s), pol_b);
                            load(sB + s * kBB + kBB / 2, tmB1, kb * kKE, tl.nb * (kBN / 2), full_bar(s), pol_b);
                        } else {
                            load(sB + s * kBB, tmB0, kb * kKE, tl.nb * kBN, full_bar(s), pol_b);
                            load(sB + s * kBB + kBB / 2, tmB0, kb * kKE, tl.nb * kBN + kBN / 2, full_bar(s), pol_b);
                        }
                    }
                    if (++s == kNS) {
                        s = 0;
                        phase ^= 1;
                    }
                }
            }
            if (!ok) {
                // let the copies that are still in flight land before the CTA goes away
                for (int i = 0; i < kNS; i++) {
                    if (armed[i] < 0) continue;
                    for (int spin = 0; spin < (1 << 16); spin++) {
                        if (mbar_try_wait(full_bar(i), (uint32_t)armed[i])) break;
                    }
                }
            }
        }
    } else if (warp >= kCopierWarp0) {
        // ------------------------------------------------------------ copier warps
        if (p.comm == COMM_ALLGATHER_A && p.copy_mode == 1 && p.tp_size > 1) {
            copier_warps_loop<kFp8 ? 8 : 32>(p, rank, local, (int)threadIdx.x - kCopierWarp0 * 32, ab);
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer
        if ((!kPair || cta_rank == 0) && elect_one()) {
            const uint32_t idesc = kFp8 ? make_idesc(0, 0, kPair ? 2 * kBM : kBM, kBN)   // e4m3 x e4m3 -> fp32
                                        : make_idesc(1, 1, kPair ? 2 * kBM : kBM, kBN);  // bf16 x bf16 -> fp32
            int            s = 0;
            uint32_t       phase = 0, acc_phase = 0;
            int            a = 0;
            bool           ok = true;
            // an MMA group's completion is announced to the barrier at the same offset in every CTA of the tile
            auto commit = [&](uint32_t bar) {
                if (kPair) {
                    mma_commit_pair(map_to_cta(bar, 0));
                    mma_commit_pair(map_to_cta(bar, 1));
                } else {
                    mma_commit(bar);
                }
            };
            for (int t = unit; kFp8 && t < total && ok; t += n_units) {
                // one product buffer per K block: the promotion warps empty it while the next block is multiplied
                for (int kb = 0; kb < kblocks; kb++) {
                    if (!mbar_wait(tmem_empty_bar(a), acc_phase ^ 1, ab, 3) || !mbar_wait(full_bar(s), phase, ab, 4)) {
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t d_tmem = tmem_base + (uint32_t)a * kBN;
                    const uint64_t da = make_desc_sw128(sA + s * kABytes);
                    const uint64_t db = make_desc_sw128(sB + s * kBB);
#pragma unroll
                    for (int k = 0; k < 4; k++) {
                        // 32 fp8 values = 32 bytes further along K inside the 128-byte swizzle row
                        if (kPair) {
                            mma_f8_pair(d_tmem, da + (uint64_t)(k * 2), db + (uint64_t)(k * 2), idesc, k != 0);
                        } else {
                            mma_f8(d_tmem, da + (uint64_t)(k * 2), db + (uint64_t)(k * 2), idesc, k != 0);
                        }
                    }
                    commit(empty_bar(s));
                    commit(tmem_full_bar(a));
                    if (++s == kNS) {
                        s = 0;
                        phase ^= 1;
                    }
                    a ^= 1;
                    if (a == 0) acc_phase ^= 1;
                }
            }
            for (int t = unit; !kFp8 && t < total && ok; t += n_units) {
                if (!mbar_wait(tmem_empty_bar(a), acc_phase ^ 1, ab, 3)) break;
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + (uint32_t)a * kBN;
                for (int kb = 0; kb < kblocks; kb++) {
                    if (!mbar_wait(full_bar(s), phase, ab, 4)) {
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    const uint64_t da = make_desc_sw128(sA + s * kABytes);
                    const uint64_t db = make_desc_sw128(sB + s * kBB);
#pragma unroll
                    for (int k = 0; k < kBK / 16; k++) {
                        // 16 bf16 = 32 bytes further along K inside the 128-byte swizzle row
                        if (kPair) {
                            mma_f16_pair(d_tmem, da + (uint64_t)(k * 2), db + (uint64_t)(k * 2), idesc, (kb | k) != 0);
                        } else {
                            mma_f16(d_tmem, da + (uint64_t)(k * 2), db + (uint64_t)(k * 2), idesc, (kb | k) != 0);
                        }
                    }
                    commit(empty_bar(s));
                    if (++s == kNS) {
                        s = 0;
                        phase ^= 1;
                    }
                }
                if (!ok) break;
                commit(tmem_full_bar(a));
                a ^= 1;
                if (a == 0) acc_phase ^= 1;
            }
        }
    } else if (kFp8) {
        // ------------------------------------------------------------ promotion + epilogue warps (fp8)
        const int      quarter = warp % 4;        // TMEM lanes this warp may read: 32*quarter ..
        const int      half    = (warp - 2) / 4;  // which 128 of the 256 accumulator columns
        uint8_t       *stage   = epi_gen + (warp - 2) * 32 * kStageRowBytes;
        uint32_t       acc_phase = 0;
        int            a = 0;
        const int      mbs   = (p.comm == COMM_NONE) ? tiles_m128 : tiles_m128 / p.tp_size;
        const bool     swi   = p.epilogue == EPI_SWIGLU;
        const int      n_out = swi ? p.N / 2 : p.N;
        // the two 64-column ranges of the accumulator this warp owns: plain tiles one weight block (128 columns),
        // SwiGLU tiles 64 "gate" columns and the 64 "up" columns of the same outputs
        const int      c0 = swi ? half * 64 : half * 128, c1 = swi ? kBN / 2 + half * 64 : half * 128 + 64;
        bool           ok = true;
        for (int t = unit; t < total && ok; t += n_units) {
            Tile tl = tile_of(p, rank, t, tiles_m, tiles_n);
            if (kPair) tl.mb = tl.mb * 2 + (int)cta_rank;
            const int  row    = tl.mb * kBM + quarter * 32 + lane;
            const bool row_ok = row < p.M;
            // running sums as pairs: the promotion is one packed fp32 FMA per two columns
            float2     acc2[64];
#pragma unroll
            for (int j = 0; j < 64; j++) acc2[j] = make_float2(0.0f, 0.0f);
            const float *sa_row = p.sg[rank] + (size_t)(row_ok ? row : 0) * kblocks;
            // weight scales: [rows / 128][K / 128]; a plain tile spans two weight blocks, a SwiGLU tile one of each matrix
            const int    wblk = (tl.nb * 2 + half) * 128 < p.N ? tl.nb * 2 + half : 0;  // a last tile may be half outside N
            const float *sb_0 = swi ? p.sb0[local] + (size_t)tl.nb * kblocks : p.sb0[local] + (size_t)wblk * kblocks;
            const float *sb_1 = swi ? p.sb1[local] + (size_t)tl.nb * kblocks : sb_0;
            // Scales are fetched one K block ahead: a load from L2 takes longer than the MMAs of a K block, and on the
            // critical path of every block it would bound the kernel. The weight scales can be read at any time. The
            // scales of gathered rows arrive with the rows, so the first one of a tile is read only when the product of
            // its first K block exists (the whole row block was released by the copiers before that), from L2, not from
            // a stale L1 line; from then on the next block's scale is requested while this block is added up.
            float w0_next = __ldg(sb_0), w1_next = __ldg(sb_1), a_next = 0.0f;
            for (int kb = 0; kb < kblocks; kb++) {
                if (!mbar_wait(tmem_full_bar(a), acc_phase, ab, 5)) {
                    ok = false;
                    break;
                }
                tc_fence_after();
                if (kb == 0) a_next = row_ok ? __ldcg(sa_row) : 0.0f;
                const float a_s = a_next, w0 = w0_next, w1 = w1_next;
                if (kb + 1 < kblocks) {
                    a_next  = row_ok ? __ldcg(sa_row + kb + 1) : 0.0f;
                    w0_next = __ldg(sb_0 + kb + 1);
                    w1_next = __ldg(sb_1 + kb + 1);
                }
                const float s0 = a_s * w0, s1 = a_s * w1;
                const uint32_t t_acc = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)a * kBN;
                // four batches of 32 columns: tcgen05.wait::ld waits for every load in flight, so a batch is "issue two
                // 16-column loads, wait once, add up"; as few waits per K block as the register budget allows (the 128
                // running sums leave room for 32 loaded values)
#pragma unroll
                for (int c = 0; c < 4; c++) {
                    uint32_t v[2][16];
                    const uint32_t col = (uint32_t)((c < 2 ? c0 : c1) + (c & 1) * 32);
                    tmem_ld_32x16(t_acc + col, v[0]);
                    tmem_ld_32x16(t_acc + col + 16, v[1]);
                    tmem_ld_wait();
                    const float  sc  = (c < 2) ? s0 : s1;
                    const float2 sc2 = make_float2(sc, sc);
#pragma unroll
                    for (int h2 = 0; h2 < 2; h2++) {
#pragma unroll
                        for (int j = 0; j < 8; j++) {
                            const float2 x = make_float2(__uint_as_float(v[h2][2 * j]), __uint_as_float(v[h2][2 * j + 1]));
                            acc2[c * 16 + h2 * 8 + j] = __ffma2_rn(sc2, x, acc2[c * 16 + h2 * 8 + j]);
                        }
                    }
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) {
                    if (kPair) {
                        mbar_arrive_cluster(map_to_cta(tmem_empty_bar(a), 0));
                    } else {
                        mbar_arrive(tmem_empty_bar(a));
                    }
                }
                a ^= 1;
                if (a == 0) acc_phase ^= 1;
            }
            if (!ok) break;
            // ---- epilogue of the tile from the registers
            float acc[128];
#pragma unroll
            for (int j = 0; j < 64; j++) {
                acc[2 * j]     = acc2[j].x;
                acc[2 * j + 1] = acc2[j].y;
            }
            __nv_bfloat16 *out;
            size_t         ld;
            int            row0;
            const bool     own_rs = (p.comm == COMM_REDUCE_SCATTER_C) && p.rs_fused != 0 && tl.shard == rank;
            const __nv_bfloat16 *rs_parts = nullptr;
            size_t               rs_slot  = 0;
            if (own_rs) {
                const size_t shard_rows = (size_t)mbs * kBM;
                rs_slot  = shard_rows * (size_t)p.N;
                rs_parts = p.part[rank] + (size_t)(p.seq & 1) * p.tp_size * rs_slot;
                out      = p.C[local];
                ld       = (size_t)p.ldc;
                row0     = (tl.mb - tl.shard * mbs) * kBM;
                int good = 1;
                if (lane < p.tp_size && lane != rank) {
                    const uint32_t *ctr = p.pad[rank] + nvl::kPadCounterOff + ((p.seq & 1) * p.tp_size + lane) * 64 +
                                          (tl.mb - tl.shard * mbs);
                    good = (p.rs_debug_local || wait_counter(ctr, p.rs_target, true, ab, 6)) ? 1 : 0;
                }
                if (!__all_sync(0xffffffffu, good)) break;
            } else if (p.comm == COMM_REDUCE_SCATTER_C) {
                const size_t shard_rows = (size_t)mbs * kBM;
                out  = p.part[p.rs_debug_local ? rank : tl.shard] + ((size_t)(p.seq & 1) * p.tp_size + rank) * shard_rows * (size_t)p.N;
                ld   = (size_t)p.N;
                row0 = (tl.mb - tl.shard * mbs) * kBM;
            } else {
                out  = p.C[local];
                ld   = (size_t)p.ldc;
                row0 = tl.mb * kBM;
            }
            const int rows_valid = ((p.comm == COMM_REDUCE_SCATTER_C) ? mbs * kBM : p.M) - row0;
            if (swi) {
#pragma unroll
                for (int j = 0; j < 64; j++) acc[j] = silu(acc[j]) * acc[64 + j];
            }
            // first output column of this warp's registers, and how many 64-column groups they hold
            const int col_base = swi ? tl.nb * (kBN / 2) + half * 64 : tl.nb * kBN + half * 128;
            const int groups   = swi ? 1 : 2;
            if (swi && p.out_fp8 != 0) {
                // the 128 outputs of this row in this tile are one 1 x 128 quantisation block of the next GEMM's
                // activations: amax over both halves (the partner warp holds the other 64), one scale, e4m3 bytes
                float amax = 0.0f;
#pragma unroll
                for (int j = 0; j < 64; j++) amax = fmaxf(amax, fabsf(acc[j]));
                float *xch = reinterpret_cast<float *>(stage);  // 32 floats of this warp's staging rows
                xch[lane]  = amax;
                asm volatile("bar.sync %0, 64;" ::"r"(2 + quarter) : "memory");
                const float *other = reinterpret_cast<const float *>(epi_gen + ((warp - 2) ^ 4) * 32 * kStageRowBytes);
                amax               = fmaxf(amax, other[lane]);
                asm volatile("bar.sync %0, 64;" ::"r"(2 + quarter) : "memory");
                const float sc = fmaxf(amax, 1e-12f) / 448.0f, inv = 1.0f / sc;
                uint8_t    *o8 = reinterpret_cast<uint8_t *>(p.C[local]);
                if (row_ok) {
                    if (half == 0) p.out_scale[local][(size_t)row * (size_t)(n_out / 128) + tl.nb] = sc;
                    uint4 *dstp = reinterpret_cast<uint4 *>(o8 + (size_t)row * (size_t)p.ldc + col_base);
#pragma unroll
                    for (int g4 = 0; g4 < 4; g4++) {
                        uint32_t w4[4];
#pragma unroll
                        for (int q = 0; q < 4; q++) {
                            const int j = g4 * 16 + q * 4;
                            w4[q] = (uint32_t)__nv_cvt_float_to_fp8(acc[j] * inv, __NV_SATFINITE, __NV_E4M3) |
                                    ((uint32_t)__nv_cvt_float_to_fp8(acc[j + 1] * inv, __NV_SATFINITE, __NV_E4M3) << 8) |
                                    ((uint32_t)__nv_cvt_float_to_fp8(acc[j + 2] * inv, __NV_SATFINITE, __NV_E4M3) << 16) |
                                    ((uint32_t)__nv_cvt_float_to_fp8(acc[j + 3] * inv, __NV_SATFINITE, __NV_E4M3) << 24);
                        }
                        dstp[g4] = make_uint4(w4[0], w4[1], w4[2], w4[3]);
                    }
                }
            } else {
                for (int g = 0; g < groups; g++) {
                    uint4 *rowp = reinterpret_cast<uint4 *>(stage + lane * kStageRowBytes);
#pragma unroll
                    for (int j = 0; j < 8; j++) {
                        // g is 0 or 1: constant indices after unrolling both branches
                        if (g == 0) {
                            rowp[j] = make_uint4(pack_bf16x2(acc[8 * j], acc[8 * j + 1]), pack_bf16x2(acc[8 * j + 2], acc[8 * j + 3]),
                                                 pack_bf16x2(acc[8 * j + 4], acc[8 * j + 5]), pack_bf16x2(acc[8 * j + 6], acc[8 * j + 7]));
                        } else {
                            rowp[j] = make_uint4(pack_bf16x2(acc[64 + 8 * j], acc[64 + 8 * j + 1]), pack_bf16x2(acc[64 + 8 * j + 2], acc[64 + 8 * j + 3]),
                                                 pack_bf16x2(acc[64 + 8 * j + 4], acc[64 + 8 * j + 5]), pack_bf16x2(acc[64 + 8 * j + 6], acc[64 + 8 * j + 7]));
                        }
                    }
                    __syncwarp();
                    const int col0 = col_base + g * 64;
#pragma unroll
                    for (int it = 0; it < 8; it++) {
                        const int r = it * 4 + lane / 8, chunk = lane % 8;
                        const int grow = quarter * 32 + r, gcol = col0 + chunk * 8;
                        if (grow < rows_valid && gcol < n_out) {
                            uint4 v = *reinterpret_cast<const uint4 *>(stage + r * kStageRowBytes + chunk * 16);
                            if (own_rs) {
                                // (registers are scarce next to the 128 running sums: two partials in flight at a time)
                                const size_t off = (size_t)(row0 + grow) * (size_t)p.N + gcol;
                                float        sum[8];
#pragma unroll
                                for (int e = 0; e < 8; e++) sum[e] = 0.0f;
                                for (int src = 0; src < p.tp_size; src += 2) {
                                    uint4 x0 = (src == rank) ? v : nvl::ld_nc16(rs_parts + (size_t)src * rs_slot + off);
                                    uint4 x1 = make_uint4(0, 0, 0, 0);
                                    if (src + 1 < p.tp_size) x1 = (src + 1 == rank) ? v : nvl::ld_nc16(rs_parts + (size_t)(src + 1) * rs_slot + off);
                                    const __nv_bfloat162 *h0 = reinterpret_cast<const __nv_bfloat162 *>(&x0);
                                    const __nv_bfloat162 *h1 = reinterpret_cast<const __nv_bfloat162 *>(&x1);
#pragma unroll
                                    for (int e = 0; e < 4; e++) {
                                        const float2 f0 = __bfloat1622float2(h0[e]), f1 = __bfloat1622float2(h1[e]);
                                        sum[2 * e] += f0.x;
                                        sum[2 * e + 1] += f0.y;
                                        sum[2 * e] += f1.x;
                                        sum[2 * e + 1] += f1.y;
                                    }
                                }
                                v = make_uint4(pack_bf16x2(sum[0], sum[1]), pack_bf16x2(sum[2], sum[3]),
                                               pack_bf16x2(sum[4], sum[5]), pack_bf16x2(sum[6], sum[7]));
                            }
                            *reinterpret_cast<uint4 *>(out + (size_t)(row0 + grow) * ld + gcol) = v;
                        }
                    }
                    __syncwarp();
                }
            }
            if (p.comm == COMM_REDUCE_SCATTER_C && !own_rs) {
                // all eight epilogue warps have stored their part of the rows: tell the owner one more tile arrived
                asm volatile("bar.sync 1, 256;" ::: "memory");
                if (warp == 2 && lane == 0) {
                    __threadfence_system();
                    uint32_t *ctr = p.pad[p.rs_debug_local ? rank : tl.shard] + nvl::kPadCounterOff +
                                    ((p.seq & 1) * p.tp_size + rank) * 64 + (tl.mb - tl.shard * mbs);
                    nvl::red_release_sys_add(ctr, 1u);
                }
            }
        }
    } else {
        // ------------------------------------------------------------ epilogue warps
        const int      quarter = warp % 4;  // TMEM lanes this warp may read: 32*quarter ..
        uint8_t       *stage   = epi_gen + (warp - 2) * 32 * kStageRowBytes;
        uint32_t       acc_phase = 0;
        int            a = 0;
        const int      mbs  = (p.comm == COMM_NONE) ? tiles_m128 : tiles_m128 / p.tp_size;
        const int      out_cols_per_tile = (p.epilogue == EPI_SWIGLU) ? kBN / 2 : kBN;
        const int      n_out = (p.epilogue == EPI_SWIGLU) ? p.N / 2 : p.N;
        for (int t = unit; t < total; t += n_units) {
            Tile tl = tile_of(p, rank, t, tiles_m, tiles_n);
            if (kPair) tl.mb = tl.mb * 2 + (int)cta_rank;
            if (!mbar_wait(tmem_full_bar(a), acc_phase, ab, 5)) break;
            tc_fence_after();
            const uint32_t t_acc = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)a * kBN;
            // destination of this tile
            __nv_bfloat16 *out;
            size_t         ld;
            int            row0;
            // reduce-scatter, tiles of my own rows (walked last): the partial tiles of the other ranks for these
            // rows are already in my partial buffer, so the epilogue adds them to the accumulator and writes the
            // final value - no pass over the partials after the last tile
            const bool     own_rs = (p.comm == COMM_REDUCE_SCATTER_C) && p.rs_fused != 0 && tl.shard == rank;
            const __nv_bfloat16 *rs_parts = nullptr;
            size_t               rs_slot  = 0;
            if (own_rs) {
                const size_t shard_rows = (size_t)mbs * kBM;
                rs_slot  = shard_rows * (size_t)p.N;
                rs_parts = p.part[rank] + (size_t)(p.seq & 1) * p.tp_size * rs_slot;
                out      = p.C[local];
                ld       = (size_t)p.ldc;
                row0     = (tl.mb - tl.shard * mbs) * kBM;
                // every other rank has sent all column tiles of this row block (bounded wait, one source per lane)
                int good = 1;
                if (lane < p.tp_size && lane != rank) {
                    const uint32_t *ctr = p.pad[rank] + nvl::kPadCounterOff + ((p.seq & 1) * p.tp_size + lane) * 64 +
                                          (tl.mb - tl.shard * mbs);
                    good = (p.rs_debug_local || wait_counter(ctr, p.rs_target, true, ab, 6)) ? 1 : 0;
                }
                if (!__all_sync(0xffffffffu, good)) break;
            } else if (p.comm == COMM_REDUCE_SCATTER_C) {
                // slot `rank` of the owner's partial buffer, parity by launch sequence
                const size_t shard_rows = (size_t)mbs * kBM;
                out  = p.part[p.rs_debug_local ? rank : tl.shard] + ((size_t)(p.seq & 1) * p.tp_size + rank) * shard_rows * (size_t)p.N;
                ld   = (size_t)p.N;
                row0 = (tl.mb - tl.shard * mbs) * kBM;
            } else {
                out  = p.C[local];
                ld   = (size_t)p.ldc;
                row0 = tl.mb * kBM;
            }
            const int rows_valid = ((p.comm == COMM_REDUCE_SCATTER_C) ? mbs * kBM : p.M) - row0;
            for (int oc = 0; oc < out_cols_per_tile; oc += 64) {
                // 64 output columns -> one 128-byte staging row per TMEM lane
#pragma unroll
                for (int h = 0; h < 2; h++) {
                    uint32_t g[32];
                    uint32_t packed[16];
                    tmem_ld_32x32(t_acc + (uint32_t)(oc + h * 32), g);
                    if (p.epilogue == EPI_SWIGLU) {
                        uint32_t u[32];
                        tmem_ld_32x32(t_acc + (uint32_t)(kBN / 2 + oc + h * 32), u);
                        tmem_ld_wait();
#pragma unroll
                        for (int j = 0; j < 16; j++) {
                            float g0 = __uint_as_float(g[2 * j]), g1 = __uint_as_float(g[2 * j + 1]);
                            float u0 = __uint_as_float(u[2 * j]), u1 = __uint_as_float(u[2 * j + 1]);
                            packed[j] = pack_bf16x2(silu(g0) * u0, silu(g1) * u1);
                        }
                    } else {
                        tmem_ld_wait();
#pragma unroll
                        for (int j = 0; j < 16; j++) {
                            packed[j] = pack_bf16x2(__uint_as_float(g[2 * j]), __uint_as_float(g[2 * j + 1]));
                        }
                    }
                    uint4 *row = reinterpret_cast<uint4 *>(stage + lane * kStageRowBytes + h * 64);
#pragma unroll
                    for (int j = 0; j < 4; j++) {
                        row[j] = make_uint4(packed[4 * j], packed[4 * j + 1], packed[4 * j + 2], packed[4 * j + 3]);
                    }
                }
                __syncwarp();
                const int col0 = tl.nb * out_cols_per_tile + oc;
#pragma unroll
                for (int it = 0; it < 8; it++) {
                    const int r = it * 4 + lane / 8, chunk = lane % 8;
                    const int grow = quarter * 32 + r, gcol = col0 + chunk * 8;
                    if (grow < rows_valid && gcol < n_out) {
                        uint4 v = *reinterpret_cast<const uint4 *>(stage + r * kStageRowBytes + chunk * 16);
                        if (own_rs) {
                            // sum of the tp partials in rank order, every one rounded to bf16 exactly as it would
                            // have travelled; all loads are issued before the first add
                            const size_t off = (size_t)(row0 + grow) * (size_t)p.N + gcol;
                            uint4        raw[kMaxTpRanks];
#pragma unroll
                            for (int src = 0; src < kMaxTpRanks; src++) {
                                if (src < p.tp_size && src != rank) raw[src] = nvl::ld_nc16(rs_parts + (size_t)src * rs_slot + off);
                            }
                            float acc[8];
#pragma unroll
                            for (int e = 0; e < 8; e++) acc[e] = 0.0f;
#pragma unroll
                            for (int src = 0; src < kMaxTpRanks; src++) {
                                if (src < p.tp_size) {
                                    const uint4           x = (src == rank) ? v : raw[src];
                                    const __nv_bfloat162 *h2 = reinterpret_cast<const __nv_bfloat162 *>(&x);
#pragma unroll
                                    for (int e = 0; e < 4; e++) {
                                        const float2 f = __bfloat1622float2(h2[e]);
                                        acc[2 * e] += f.x;
                                        acc[2 * e + 1] += f.y;
                                    }
                                }
                            }
                            v = make_uint4(pack_bf16x2(acc[0], acc[1]), pack_bf16x2(acc[2], acc[3]),
                                           pack_bf16x2(acc[4], acc[5]), pack_bf16x2(acc[6], acc[7]));
                        }
                        uint4 *dstp = reinterpret_cast<uint4 *>(out + (size_t)(row0 + grow) * ld + gcol);
                        if (p.st_stream) {
                            __stcs(dstp, v);
                        } else {
                            *dstp = v;
                        }
                    }
                }
                __syncwarp();
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) {
                if (kPair) {
                    mbar_arrive_cluster(map_to_cta(tmem_empty_bar(a), 0));
                } else {
                    mbar_arrive(tmem_empty_bar(a));
                }
            }
            if (p.comm == COMM_REDUCE_SCATTER_C && !own_rs) {
                // all four epilogue warps have stored their rows: tell the owner one more tile arrived
                asm volatile("bar.sync 1, 128;" ::: "memory");
                if (warp == 2 && lane == 0) {
                    __threadfence_system();
                    uint32_t *ctr = p.pad[p.rs_debug_local ? rank : tl.shard] + nvl::kPadCounterOff +
                                    ((p.seq & 1) * p.tp_size + rank) * 64 + (tl.mb - tl.shard * mbs);
                    nvl::red_release_sys_add(ctr, 1u);
                }
            }
            a ^= 1;
            if (a == 0) acc_phase ^= 1;
        }
    }

    tc_fence_before();
    __syncthreads();
    if (kPair) cluster_sync_all();  // nothing is signalled into a CTA that has gone, nor its tensor memory freed early
    if (warp == 1) {
        tc_fence_after();
        if (kPair) {
            tmem_dealloc_pair(tmem_base, kTmemCols);
        } else {
            tmem_dealloc(tmem_base, kTmemCols);
        }
    }

    // ---- reduce-scatter: add up the partial tiles that every rank stored for my rows
    // (only when the reduce is not fused into the epilogue of the local tiles)
    if (p.comm == COMM_REDUCE_SCATTER_C && p.rs_fused == 0 && *abort_slot == 0) rs_reduce_phase(p, rank, local, tiles_m128, ab);
}

}  // namespace

const OptTable &tp_options()
{
    static OptTable t = [] {
        OptTable o("TP_", {
            {"GEMM_PAIR", "y", "Run the GEMM kernels as CTA pairs (cta_group::2, 256 x 256 tiles) when the shape allows", OptType::BOOL},
            {"GEMM_GROUP", "0", "Row blocks of tiles walked together before moving along N (0: chosen from the shape)", OptType::UINT},
            {"GEMM_L2HINT", "0", "Cache hints of the operand loads: 0 none, 1 A and B evict_last, 2 A evict_last / B evict_first, 3 the reverse", OptType::UINT},
            {"GEMM_L2PROMO", "3", "L2 promotion of the tensor maps: 0 none, 1 64 B, 2 128 B, 3 256 B", OptType::UINT},
            {"GEMM_STCS", "n", "Mark output stores as streaming (evict first)", OptType::BOOL},
            {"GEMM_SYNC", "y", "Keep the tile walkers in soft lockstep (one counter per wave of tiles)", OptType::BOOL},
            {"GEMM_SYNC_KBLOCKS", "0", "Also synchronise every this many K blocks inside a tile (0: tile starts only)", OptType::UINT},
            {"GEMM_SYNC_NS", "30000", "Longest wait at a lockstep point in nanoseconds; running out is not an error", OptType::UINT},
            {"COPY_MODE", "-1", "allgather->GEMM: 1 = two copier warps in every CTA pull the remote shards, 0 = whole CTAs are set aside for it (COPY_CTAS), -1 = by team size (1 up to two ranks)", OptType::INT},
            {"COPY_CTAS", "0", "Copy mode 0: CTAs that pull the remote shards (0: 16)", OptType::UINT},
            {"RS_DEBUG_LOCAL", "n", "Diagnostic, wrong results: GEMM->reduce-scatter stores every partial tile into local memory and waits for nobody, to time the kernel without its NVLink traffic", OptType::BOOL},
            {"RS_FUSED", "y", "GEMM->reduce-scatter: add the peers' partial tiles in the epilogue of the local tiles instead of a reduce phase after the last tile", OptType::BOOL},
            {"H2D_CHUNK_ROWS", "256", "Rows per chunk of the overlapped host->device input copy", OptType::UINT},
            {"H2D_PHASES", "n", "Allgather with copy CTAs while every rank's input arrives from the host: ranks report their rows block by block and the tiles are walked row block by row block over all shards (set it on every rank alike). Measured on 4 GPUs: no gain over the default (3.07 against 2.94 ms per end-to-end step)", OptType::BOOL},
            {"H2D_RAMP", "y", "While the input rows arrive from the host, walk the local rows in groups of 1, 1, 2, 4, ... row blocks instead of full groups", OptType::BOOL},
        });
        o.read(nullptr, nullptr);
        return o;
    }();
    return t;
}

uint32_t *error_word()
{
    static uint32_t *word[64] = {nullptr};
    int              dev = 0;
    cudaGetDevice(&dev);
    if (word[dev] == nullptr) {
        if (cudaMalloc((void **)&word[dev], 4) != cudaSuccess) return nullptr;
        cudaMemset(word[dev], 0, 4);
    }
    return word[dev];
}

size_t gemm_smem_bytes() { return kSmemBytes; }

namespace {
constexpr int kSyncPoints = 8192;  // lockstep counters per local rank
uint32_t *sync_counters()
{
    static uint32_t *buf[64] = {nullptr};
    int              dev = 0;
    cudaGetDevice(&dev);
    if (buf[dev] == nullptr) {
        if (cudaMalloc((void **)&buf[dev], sizeof(uint32_t) * kSyncPoints * kMaxTpRanks) != cudaSuccess) return nullptr;
    }
    return buf[dev];
}
}  // namespace

xccl_status_t make_tensor_map_2d(CUtensorMap *map, const void *base, uint64_t rows, uint64_t cols, uint64_t ld,
                                 uint32_t box_rows)
{
    XCCL_DRIVER_FN(cuTensorMapEncodeTiled);
    if (((uintptr_t)base & 15) != 0 || (ld * 2) % 16 != 0) return XCCL_ERR_INVALID_PARAM;
    cuuint64_t dims[2]    = {cols, rows};
    cuuint64_t strides[1] = {ld * 2};
    cuuint32_t box[2]     = {(cuuint32_t)kBK, box_rows};
    cuuint32_t estr[2]    = {1, 1};
    const int promo = (int)std::max(0ll, std::min(3ll, tp_options().num("GEMM_L2PROMO")));
    const CUtensorMapL2promotion pr = promo == 0 ? CU_TENSOR_MAP_L2_PROMOTION_NONE
                                    : promo == 1 ? CU_TENSOR_MAP_L2_PROMOTION_L2_64B
                                    : promo == 2 ? CU_TENSOR_MAP_L2_PROMOTION_L2_128B
                                                 : CU_TENSOR_MAP_L2_PROMOTION_L2_256B;
    XCCL_CU_CHECK(cuTensorMapEncodeTiled(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void *>(base), dims,
                                         strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                         pr, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE));
    return XCCL_OK;
}

namespace {
xccl_status_t launch_gemm_impl(const GemmParams &p_in, const GemmLaunch &l, cudaStream_t stream, bool fp8);
}

xccl_status_t launch_gemm(const GemmParams &p_in, const GemmLaunch &l, cudaStream_t stream)
{
    return launch_gemm_impl(p_in, l, stream, false);
}

// Block-scaled fp8: K in whole 128-wide scale blocks, N in whole 128-column weight blocks.
xccl_status_t launch_gemm_fp8(const GemmParams &p_in, const GemmLaunch &l, cudaStream_t stream)
{
    GemmParams p = p_in;
    if (p.M <= 0 || p.N <= 0 || p.K <= 0 || p.K % 128 != 0 || p.N % 128 != 0) return XCCL_ERR_INVALID_PARAM;
    if (p.out_fp8 != 0 && p.epilogue != EPI_SWIGLU) return XCCL_ERR_INVALID_PARAM;
    p.a_bytes = 1;
    return launch_gemm_impl(p, l, stream, true);
}

namespace {
xccl_status_t launch_gemm_impl(const GemmParams &p_in, const GemmLaunch &l, cudaStream_t stream, bool fp8)
{
    GemmParams p = p_in;
    if (p.K % 8 != 0 || p.N % 8 != 0 || p.M <= 0 || p.N <= 0 || p.K <= 0) return XCCL_ERR_INVALID_PARAM;
    if (p.epilogue == EPI_SWIGLU && p.N % kBN != 0) return XCCL_ERR_INVALID_PARAM;  // gate/up halves of a tile
    if (p.comm != COMM_NONE) {
        int tiles_m = (p.M + kBM - 1) / kBM;
        if (p.M % kBM != 0 || tiles_m % p.tp_size != 0 || tiles_m / p.tp_size > 64) return XCCL_ERR_INVALID_PARAM;
    }
    static bool attr_set[64] = {false};
    int         dev = 0, sms = 0;
    XCCL_CUDA_CHECK(cudaGetDevice(&dev));
    XCCL_CUDA_CHECK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    if (!attr_set[dev]) {
        XCCL_CUDA_CHECK(cudaFuncSetAttribute(tp_gemm_kernel<false, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBytes));
        XCCL_CUDA_CHECK(cudaFuncSetAttribute(tp_gemm_kernel<true, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBytes));
        XCCL_CUDA_CHECK(cudaFuncSetAttribute(tp_gemm_kernel<false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBytes));
        XCCL_CUDA_CHECK(cudaFuncSetAttribute(tp_gemm_kernel<true, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBytes));
        attr_set[dev] = true;
    }
    int ctas = l.ctas > 0 ? l.ctas : sms / std::max(l.n_local, 1);
    if (p.n_gemm_ctas <= 0 || p.n_gemm_ctas > ctas) p.n_gemm_ctas = ctas;
    if (p.comm == COMM_ALLGATHER_A && p.tp_size > 1 && p.copy_mode == 0 && p.n_gemm_ctas == ctas) return XCCL_ERR_INVALID_PARAM;
    if (p.copy_mode == 1) p.n_gemm_ctas = ctas;
    if (p.error == nullptr) p.error = error_word();
    if (p.budget_ns == 0) p.budget_ns = 4000000000ull;

    // CTA pairs (clusters of two, one 256-row tile per pair) when the shape allows: an even number of
    // CTAs in each role and, with communication, row shards made of whole 256-row tiles.
    const OptTable &opt       = tp_options();
    const int       pair_env  = opt.flag("GEMM_PAIR") ? 1 : 0;
    const int       group_env = (int)opt.num("GEMM_GROUP");
    if (p.group_rows <= 0) p.group_rows = group_env;
    const int hint_env    = (int)std::max(0ll, std::min(3ll, opt.num("GEMM_L2HINT")));
    const int stcs_env    = opt.flag("GEMM_STCS") ? 1 : 0;
    const int sync_env    = opt.flag("GEMM_SYNC") ? 1 : 0;
    const int sync_kb_env = (int)opt.num("GEMM_SYNC_KBLOCKS");
    const int sync_ns_env = (int)opt.num("GEMM_SYNC_NS");
    for (int i = 0; i < kMaxTpRanks; i++) p.sync_ctr[i] = nullptr;
    p.sync_points = 0;
    // (not in reduce-scatter mode: there a walker may be held up by its stores to a peer or by a wait for the peers'
    // partial tiles, and every other walker would wait for it at the next lockstep point; measured on 8 GPUs,
    // 8192 x 8192 x 3584 per rank: 0.474 ms with lockstep, 0.401 ms without)
    if (sync_env == 1 && l.n_local <= kMaxTpRanks && p.comm != COMM_REDUCE_SCATTER_C) {
        uint32_t *ctr = sync_counters();
        // worth it only when a walker has several tiles: the drift builds up over tiles
        const int  tile_rows = 2 * kBM;
        const long tiles     = (long)((p.M + tile_rows - 1) / tile_rows) * ((p.N + kBN - 1) / kBN);
        const int  kblocks   = (p.K + (fp8 ? 2 * kBK : kBK) - 1) / (fp8 ? 2 * kBK : kBK);
        const int  per_tile  = sync_kb_env > 0 ? (kblocks + sync_kb_env - 1) / sync_kb_env : 1;
        const long waves     = (tiles + std::max(1, ctas / 2) - 1) / std::max(1, ctas / 2) * 2 + 2;  // single-CTA walkers: half-size tiles
        const long points    = std::min<long>(waves * per_tile, kSyncPoints);
        if (ctr != nullptr && tiles > ctas) {
            XCCL_CUDA_CHECK(cudaMemsetAsync(ctr, 0, sizeof(uint32_t) * kSyncPoints * (l.n_local - 1) + sizeof(uint32_t) * points, stream));
            for (int i = 0; i < l.n_local; i++) p.sync_ctr[i] = ctr + (size_t)i * kSyncPoints;
            p.sync_points    = (int)points;
            p.sync_kblocks   = sync_kb_env;
            p.sync_budget_ns = (unsigned)sync_ns_env;
        }
    }
    p.l2_hint   = hint_env;
    p.st_stream = (p.comm == COMM_REDUCE_SCATTER_C) ? 0 : stcs_env;  // partial tiles are read back at once
    static bool pair_refused[64] = {false};  // the device could not place the clusters: stay with single CTAs
    bool pair = pair_env == 1 && !pair_refused[dev];
    if (pair && p.comm != COMM_NONE && (p.M / p.tp_size) % (2 * kBM) != 0) pair = false;
    if (pair && ctas < 2) pair = false;

    // Row blocks walked together before moving along N. Short K: as many rows of A as stay in L2 next
    // to the streaming B (about 48 MiB); long K: the squarest arrangement of one wave of tiles, which
    // needs the fewest distinct rows of A and B from DRAM.
    auto auto_group = [&](int tile_rows, int wave_rows) {
        if (p.group_rows > 0) return p.group_rows;
        long rows = (48l << 20) / ((long)p.K * 2);
        rows      = std::max<long>(wave_rows, std::min<long>(rows, 4096));
        return (int)std::max<long>(1, (rows + tile_rows / 2) / tile_rows);
    };
    const int group_single = auto_group(kBM, 12 * kBM), group_pair = auto_group(2 * kBM, 8 * 2 * kBM);
    p.group_rows           = group_single;

    cudaLaunchConfig_t cfg{};
    cfg.blockDim         = dim3(fp8 ? kThreadsFp8 : kThreads);
    cfg.dynamicSmemBytes = kSmemBytes;
    cfg.stream           = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id              = cudaLaunchAttributeCooperative;
    attr[0].val.cooperative = l.cooperative ? 1 : 0;
    cfg.attrs               = attr;
    cfg.numAttrs            = 1;
    if (pair) {
        GemmParams pp     = p;
        int        pctas  = ctas & ~1;
        int        n_copy = ctas - p.n_gemm_ctas;
        n_copy            = (n_copy + 1) & ~1;
        pp.n_gemm_ctas    = pctas - n_copy;
        pp.group_rows     = group_pair;
        attr[1].id               = cudaLaunchAttributeClusterDimension;
        attr[1].val.clusterDim.x = 2;
        attr[1].val.clusterDim.y = 1;
        attr[1].val.clusterDim.z = 1;
        cfg.numAttrs             = 2;
        cfg.gridDim              = dim3((unsigned)pctas, (unsigned)l.n_local);
        // every CTA of the grid must be resident at once: roles wait for one another
        // (a property of the device, the kernel and its launch shape, none of which changes: asked once per device)
        static int  clusters_fit[64][2] = {};
        int         max_clusters        = clusters_fit[dev][fp8 ? 1 : 0];
        cudaError_t oe                  = cudaSuccess;
        if (max_clusters == 0) {
            oe = fp8 ? cudaOccupancyMaxActiveClusters(&max_clusters, tp_gemm_kernel<true, true>, &cfg)
                     : cudaOccupancyMaxActiveClusters(&max_clusters, tp_gemm_kernel<true, false>, &cfg);
            if (oe == cudaSuccess) clusters_fit[dev][fp8 ? 1 : 0] = max_clusters;
        }
        if (oe == cudaSuccess && pp.n_gemm_ctas >= 2 && max_clusters * 2 >= pctas * l.n_local) {
            cudaError_t le = fp8 ? cudaLaunchKernelEx(&cfg, tp_gemm_kernel<true, true>, pp, l)
                                 : cudaLaunchKernelEx(&cfg, tp_gemm_kernel<true, false>, pp, l);
            if (le == cudaSuccess) return XCCL_OK;
            (void)cudaGetLastError();
            xccl_warn("tp gemm: launch with CTA pairs refused (%s); using single CTAs", cudaGetErrorString(le));
        } else {
            (void)cudaGetLastError();
            xccl_warn("tp gemm: %d clusters of two fit, %d CTAs wanted; using single CTAs", max_clusters, pctas * l.n_local);
        }
        pair_refused[dev] = true;
        cfg.numAttrs      = 1;
    }
    cfg.gridDim = dim3((unsigned)ctas, (unsigned)l.n_local);
    if (fp8) {
        XCCL_CUDA_CHECK(cudaLaunchKernelEx(&cfg, tp_gemm_kernel<false, true>, p, l));
    } else {
        XCCL_CUDA_CHECK(cudaLaunchKernelEx(&cfg, tp_gemm_kernel<false, false>, p, l));
    }
    return XCCL_OK;
}
}  // namespace

}  // namespace tp
}  // namespace xccl

using namespace xccl;
using namespace xccl::tp;

extern "C" {

xccl_status_t xccl_gemm_bf16(const void *A, const void *B, void *C, int M, int N, int K, void *stream)
{
    GemmParams p{};
    GemmLaunch l{};
    p.M = M; p.N = N; p.K = K;
    p.epilogue = EPI_STORE;
    p.comm     = COMM_NONE;
    p.tp_size  = 1;
    p.ldc      = N;
    p.C[0]     = (__nv_bfloat16 *)C;
    xccl_status_t st = make_tensor_map_2d(&l.tmA[0], A, (uint64_t)M, (uint64_t)K, (uint64_t)K, kBM);
    if (st != XCCL_OK) return st;
    st = make_tensor_map_2d(&l.tmB0[0], B, (uint64_t)N, (uint64_t)K, (uint64_t)K, kBN / 2);
    if (st != XCCL_OK) return st;
    l.tmB1[0] = l.tmB0[0];
    return launch_gemm(p, l, (cudaStream_t)stream);
}

xccl_status_t xccl_gemm_swiglu_bf16(const void *A, const void *Wg, const void *Wu, void *H, int M, int F, int K,
                                    void *stream)
{
    GemmParams p{};
    GemmLaunch l{};
    p.M = M; p.N = 2 * F; p.K = K;
    p.epilogue = EPI_SWIGLU;
    p.comm     = COMM_NONE;
    p.tp_size  = 1;
    p.ldc      = F;
    p.C[0]     = (__nv_bfloat16 *)H;
    if (F % (kBN / 2) != 0) return XCCL_ERR_INVALID_PARAM;
    xccl_status_t st = make_tensor_map_2d(&l.tmA[0], A, (uint64_t)M, (uint64_t)K, (uint64_t)K, kBM);
    if (st != XCCL_OK) return st;
    st = make_tensor_map_2d(&l.tmB0[0], Wg, (uint64_t)F, (uint64_t)K, (uint64_t)K, kBN / 2);
    if (st != XCCL_OK) return st;
    st = make_tensor_map_2d(&l.tmB1[0], Wu, (uint64_t)F, (uint64_t)K, (uint64_t)K, kBN / 2);
    if (st != XCCL_OK) return st;
    return launch_gemm(p, l, (cudaStream_t)stream);
}

// Host-side view of the tile order (tests): writes (row block, column block, shard) of tile t = 0 .. tiles-1 as
// rank `rank` walks them and returns the number of tiles, or -1 when `max` is too small.
int xccl_tp_tile_order_ramp(int tiles_m, int tiles_n, int tp, int rank, int comm, int group_rows, int ramp, int *mb,
                            int *nb, int *shard, int max);

int xccl_tp_tile_order(int tiles_m, int tiles_n, int tp, int rank, int comm, int group_rows, int *mb, int *nb, int *shard,
                       int max)
{
    return xccl_tp_tile_order_ramp(tiles_m, tiles_n, tp, rank, comm, group_rows, 0, mb, nb, shard, max);
}

// ramp = 1: the order used while the local rows are still arriving from the host (GemmParams::group_ramp)
int xccl_tp_tile_order_ramp(int tiles_m, int tiles_n, int tp, int rank, int comm, int group_rows, int ramp, int *mb,
                            int *nb, int *shard, int max)
{
    GemmParams p{};
    p.comm       = comm;
    p.tp_size    = tp;
    p.group_rows = group_rows;
    p.group_ramp = ramp;
    const int total = tiles_m * tiles_n;
    if (total > max) return -1;
    for (int t = 0; t < total; t++) {
        const Tile tl = tile_of(p, rank, t, tiles_m, tiles_n);
        mb[t] = tl.mb;
        nb[t] = tl.nb;
        shard[t] = tl.shard;
    }
    return total;
}

void xccl_tp_config_print(FILE *stream)
{
    if (stream != nullptr) xccl::tp::tp_options().print(stream, "fused tensor-parallel kernels", XCCL_CONFIG_PRINT_CONFIG | XCCL_CONFIG_PRINT_DOC | XCCL_CONFIG_PRINT_HEADER);
}

uint32_t xccl_gemm_last_error(void)
{
    uint32_t *w = xccl::tp::error_word();
    uint32_t  v = 0;
    if (w == nullptr) return 0xffffffffu;
    cudaMemcpy(&v, w, 4, cudaMemcpyDeviceToHost);
    if (v != 0) cudaMemset(w, 0, 4);
    return v;
}

}  // extern "C"
