// Device code shared by the tensor-parallel GEMM kernels (bf16 in tp_gemm.cu, block-scaled fp8 in
// tp_gemm_fp8.cu): tile order per communication mode, bounded counter waits, the copy CTAs of the
// allgather mode and the reduce phase of the reduce-scatter mode. Included inside a translation unit
// (everything lives in an unnamed namespace).
#pragma once
#include <cuda_bf16.h>

#include "sm100_ptx.cuh"
#include "tp_gemm.cuh"

namespace xccl {
namespace tp {

using namespace sm100;

namespace {

constexpr uint32_t kABytes     = kBM * kBK * 2;          // 16 KB
constexpr uint32_t kBBytes     = kBN * kBK * 2;          // 32 KB
constexpr uint32_t kStageBytes = kABytes + kBBytes;
constexpr uint32_t kStageRowBytes = 144;                 // 128 B of payload + 16 B pad: conflict-free transposes
constexpr uint32_t kEpiBytes   = 4 * 32 * kStageRowBytes;
constexpr uint32_t kTmemCols   = 512;
constexpr uint32_t kSmemBytes  = kStages * kStageBytes + kEpiBytes + 256 + 1024;  // + barriers + alignment slack
// CTA-pair mode (cta_group::2): a cluster of two CTAs owns a 256 x 256 tile; each CTA stages its
// 128 rows of A and HALF of the B tile, so a stage is 32 KB and six of them fit in the same ring.
constexpr int      kStagesPair = 6;
static_assert(kStagesPair * (kABytes + kBBytes / 2) == kStages * kStageBytes, "both modes share one shared-memory layout");

struct Tile {
    int mb, nb, shard;
};

// Order in which a rank walks its output tiles.
//  COMM_NONE            groups of group_rows row blocks x all column blocks (L2 reuse of A and B)
//  COMM_ALLGATHER_A     row shard by row shard, starting with the local one (its A is already here)
//  COMM_REDUCE_SCATTER  row shard by row shard, starting with the next rank's and ending with the
//                       local one, so remote partial tiles leave early and local ones need no wire
// Position t in a band of `mbs` row blocks x tiles_n column blocks that is walked in groups of row blocks (all column
// blocks of a group before the next group) whose heights ramp up 1, 1, 2, 4, ... to `gr`. Used while the band's rows
// are still arriving from the host: the first wave of tiles then needs the first rows only, and later groups are
// reached after their rows have landed (the copy delivers rows faster than the tiles consume them).
__host__ __device__ __forceinline__ void ramp_pos(int t, int mbs, int tiles_n, int gr, int *mb, int *nb)
{
    int start = 0, h = 1, i = 0;
    for (;;) {
        const int gm  = min(min(h, gr), mbs - start);
        const int cnt = gm * tiles_n;
        if (t < cnt || start + gm >= mbs) {
            *mb = start + t % gm;
            *nb = t / gm;
            return;
        }
        t -= cnt;
        start += gm;
        h = (i++ == 0) ? 1 : min(h * 2, gr);  // capped: heights stay at gr once they reach it
    }
}

__host__ __device__ __forceinline__ Tile tile_of(const GemmParams &p, int rank, int t, int tiles_m, int tiles_n)
{
    Tile tl;
    if (p.comm == COMM_NONE) {
        const int gr    = p.group_rows > 0 ? p.group_rows : 16;
        if (p.group_ramp) {
            ramp_pos(t, tiles_m, tiles_n, gr, &tl.mb, &tl.nb);
            tl.shard = 0;
            return tl;
        }
        const int group = gr * tiles_n;
        const int g = t / group, within = t % group;
        const int gm = min(gr, tiles_m - g * gr);
        tl.mb    = g * gr + within % gm;
        tl.nb    = within / gm;
        tl.shard = 0;
        return tl;
    }
    const int mbs   = tiles_m / p.tp_size;
    const int per   = mbs * tiles_n;
    const int idx   = t / per, within = t % per;
    if (p.comm == COMM_ALLGATHER_A && p.group_ramp == 2) {
        // every rank's rows are still arriving: row block c of every shard, local shard first, all column blocks
        const int per_phase = tiles_n * p.tp_size;
        const int c = t / per_phase, rem = t % per_phase;
        tl.nb    = rem / p.tp_size;
        tl.shard = (rank + rem % p.tp_size) % p.tp_size;
        tl.mb    = tl.shard * mbs + c;
        return tl;
    }
    const int first = (p.comm == COMM_ALLGATHER_A) ? 0 : 1;
    tl.shard = (rank + first + idx) % p.tp_size;
    // inside a shard: sub-groups of group_rows row blocks x all column blocks
    const int gr  = (p.group_rows > 0 && p.group_rows < mbs) ? p.group_rows : mbs;
    if (p.group_ramp && idx == 0 && p.comm == COMM_ALLGATHER_A) {  // the local shard, whose rows may still be arriving
        ramp_pos(within, mbs, tiles_n, gr, &tl.mb, &tl.nb);
        tl.mb += tl.shard * mbs;
        return tl;
    }
    const int sub = within / (gr * tiles_n), rem = within % (gr * tiles_n);
    const int gm  = min(gr, mbs - sub * gr);
    tl.mb = tl.shard * mbs + sub * gr + rem % gm;
    tl.nb = rem / gm;
    return tl;
}

__device__ __forceinline__ uint32_t ld_acquire_gpu(const uint32_t *p)
{
    uint32_t v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void red_release_gpu_add(uint32_t *p, uint32_t v)
{
    asm volatile("red.release.gpu.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// Bounded wait for a counter to reach `target` (wrap-safe); sys = counter written by another GPU.
__device__ __forceinline__ bool wait_counter(const uint32_t *ctr, uint32_t target, bool sys, const AbortFlag &ab,
                                             uint32_t where)
{
    const unsigned long long t0 = now_ns();
    for (;;) {
#pragma unroll 1
        for (int i = 0; i < 64; i++) {
            uint32_t v = sys ? nvl::ld_acquire_sys(ctr) : ld_acquire_gpu(ctr);
            if ((int32_t)(v - target) >= 0) return true;
        }
        if (*ab.smem != 0) return false;
        if (now_ns() - t0 > ab.budget_ns) {
            *ab.smem = 1;
            atomicCAS(ab.global, 0u, 0x200u | where);
            return false;
        }
    }
}

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi)
{
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t *>(&v);
}
__device__ __forceinline__ float silu(float x) { return x / (1.0f + __expf(-x)); }

// Copy CTAs of the allgather mode: pull the remote row shards into the local gathered buffer,
// one 128-row block at a time, and count each finished slice into ready[block].
// One thread drives a ring of kCopySlots shared-memory slots with untiled bulk copies: the load of
// chunk i (peer memory -> slot) is issued kCopyAhead chunks before its store (slot -> local buffer),
// so every copy CTA keeps kCopyAhead * kCopyChunk bytes in flight on the wire without holding them
// in registers.
constexpr int      kProgressSlot = 1200;  // pad counter words [1200, 1200 + ranks): blocks of each rank's shard that have landed
constexpr int      kCopySlots = 12;
constexpr int      kCopyAhead = 8;
constexpr int      kCopyLag   = 2;       // a block is announced once the stores of 2 later chunks were issued
constexpr uint32_t kCopyChunk = 16384;
static_assert(kCopySlots * kCopyChunk <= kStages * kStageBytes, "the copy ring reuses the pipeline stages");
static_assert(kCopySlots <= 2 * kStages + 4, "one mbarrier per slot in the barrier area");

__device__ void copy_cta_loop(const GemmParams &p, int rank, int local, int copy_idx, int n_copy, const AbortFlag &ab,
                              uint32_t ring, uint32_t bars)
{
    const int    tiles_m = (p.M + kBM - 1) / kBM;
    const int    mbs     = tiles_m / p.tp_size;
    const int    a_bytes   = p.a_bytes > 0 ? p.a_bytes : 2;
    const size_t blk_bytes = (size_t)kBM * p.K * a_bytes;
    const size_t blk_packs = blk_bytes / 16;  // 16-byte packs in one row block
    const size_t per   = (blk_packs + n_copy - 1) / n_copy;
    const size_t lo    = min((size_t)copy_idx * per, blk_packs) * 16, hi = min(((size_t)copy_idx + 1) * per, blk_packs) * 16;
    const int    cpb_x = (int)((hi - lo + kCopyChunk - 1) / kCopyChunk);  // chunks of this CTA per row block
    // fp8 activations travel with their 1 x 128 scales: [kBM, K / 128] fp32 per row block
    const size_t sblk_bytes = (a_bytes == 1) ? (size_t)kBM * (p.K / 128) * 4 : 0;
    const size_t sper  = (sblk_bytes / 16 + n_copy - 1) / n_copy;
    const size_t slo   = min((size_t)copy_idx * sper, sblk_bytes / 16) * 16, shi = min(((size_t)copy_idx + 1) * sper, sblk_bytes / 16) * 16;
    const int    cpb_s = (int)((shi - slo + kCopyChunk - 1) / kCopyChunk);
    const int    cpb   = cpb_x + cpb_s;
    if (threadIdx.x == 0) {
        for (int s = 0; s < kCopySlots; s++) mbar_init(bars + 8u * s, 1);
        mbar_fence_init();
    }
    // Two ways of telling the peers that this rank's shard may be read.
    //  whole (default): the shard is complete before this CTA joins the opening barrier below; where it is still
    //    arriving from the host, thread 0 waits for all of its chunks first.
    //  by block (group_ramp == 2, the same on every rank of the launch): a word per source rank in every reader's
    //    pad holds (sequence number of this launch << 8) | 128-row blocks that have landed. A shard that was
    //    complete when the kernel started is reported whole at once; one that is still arriving is reported block by
    //    block as its chunks land. Written by one thread of copy CTA 0 (beside thread 0's copy ring), read by every
    //    copy CTA before it pulls a block.
    const bool     by_block  = p.group_ramp == 2;
    const uint32_t prog_base = p.seq << 8;
    if (!by_block) {
        if (p.in_ready[local] != nullptr && threadIdx.x == 0) {
            const int chunks = (p.M / p.tp_size + p.in_rows_per_flag - 1) / p.in_rows_per_flag;
            for (int c = 0; c < chunks; c++) {
                if (!wait_counter(p.in_ready[local] + c, p.in_target, true, ab, 9)) break;
            }
        }
    } else if (copy_idx == 0 && threadIdx.x == 32) {
        auto publish = [&](uint32_t blocks) {
            for (int q = 0; q < p.tp_size; q++) {
                if (q != rank) nvl::st_release_sys(p.pad[q] + nvl::kPadCounterOff + kProgressSlot + rank, prog_base | blocks);
            }
        };
        if (p.in_ready[local] == nullptr) {
            publish((uint32_t)mbs);
        } else {
            const int rows   = p.M / p.tp_size;
            const int chunks = (rows + p.in_rows_per_flag - 1) / p.in_rows_per_flag;
            uint32_t  told   = 0;
            for (int c = 0; c < chunks; c++) {
                if (!wait_counter(p.in_ready[local] + c, p.in_target, true, ab, 9)) break;
                const uint32_t landed = (uint32_t)(min(rows, (c + 1) * p.in_rows_per_flag) / kBM);
                if (landed > told) publish(told = landed);
            }
        }
    }
    // every peer has entered this launch (its gathered buffer is no longer read by its previous kernels' tiles)
    uint32_t *epoch_slot = p.pad[rank] + nvl::kPadEpochOff + copy_idx;
    uint32_t  epoch      = *epoch_slot + 1;
    __syncthreads();
    int bad = 0;
    if ((int)threadIdx.x < p.tp_size) {
        const int q = threadIdx.x;
        nvl::st_release_sys(p.pad[q] + (size_t)copy_idx * nvl::kMaxRanks + rank, epoch);
        if (!nvl::wait_flag(p.pad[rank] + (size_t)copy_idx * nvl::kMaxRanks + q, epoch, ab.budget_ns)) bad = 1;
    }
    if (__syncthreads_or(bad)) {
        if (threadIdx.x == 0) {
            *ab.smem = 1;
            atomicCAS(ab.global, 0u, 0x300u);
        }
        return;
    }
    if (threadIdx.x == 0) {
        const int n_blocks = (p.tp_size - 1) * mbs;
        auto block_of = [&](int b) {  // b-th remote row block in the order this rank pulls them
            if (by_block) {           // row block c of every remote shard, then c + 1: the order of the tile walk
                const int c = b / (p.tp_size - 1), shard = (rank + 1 + b % (p.tp_size - 1)) % p.tp_size;
                return shard * mbs + c;
            }
            const int shard = (rank + 1 + b / mbs) % p.tp_size;
            return shard * mbs + b % mbs;
        };
        // blocks of each shard known to have landed at their owner
        uint32_t        landed[kMaxTpRanks] = {0};
        const uint32_t *progress = p.pad[rank] + nvl::kPadCounterOff + kProgressSlot;
        auto wait_landed = [&](int blk) {
            if (!by_block) return true;  // the opening barrier has said it for the whole shard
            const int      shard = blk / mbs;
            const uint32_t need  = (uint32_t)(blk % mbs) + 1u;
            if (landed[shard] >= need) return true;
            if (!wait_counter(progress + shard, prog_base | need, true, ab, 10)) return false;
            landed[shard] = nvl::ld_acquire_sys(progress + shard) - prog_base;  // at least `need`; a later launch's value is larger still
            return true;
        };
        auto announce = [&](int b) {
            asm volatile("fence.proxy.async.global;" ::: "memory");
            __threadfence();
            red_release_gpu_add(p.ready[local] + block_of(b), 1u);
        };
        if (cpb == 0) {
            for (int b = 0; b < n_blocks; b++) {
                if (!wait_landed(block_of(b))) break;
                announce(b);
            }
        } else {
            const int total = n_blocks * cpb;
            // chunk g of this CTA: where it comes from in rank `shard`'s buffers and where it goes in mine
            auto span = [&](int g, const char *&src, char *&dst, uint32_t &bytes) {
                const int b = g / cpb, c = g % cpb;
                const int blk = block_of(b), shard = blk / mbs;
                if (c < cpb_x) {
                    const size_t in  = lo + (size_t)c * kCopyChunk;
                    const size_t off = (size_t)blk * blk_bytes + in;
                    src   = reinterpret_cast<const char *>(p.xg[shard]) + off;
                    dst   = reinterpret_cast<char *>(p.xg[rank]) + off;
                    bytes = (uint32_t)min((size_t)kCopyChunk, hi - in);
                } else {
                    const size_t in  = slo + (size_t)(c - cpb_x) * kCopyChunk;
                    const size_t off = (size_t)blk * sblk_bytes + in;
                    src   = reinterpret_cast<const char *>(p.sg[shard]) + off;
                    dst   = reinterpret_cast<char *>(p.sg[rank]) + off;
                    bytes = (uint32_t)min((size_t)kCopyChunk, shi - in);
                }
            };
            bool ok = true;
            int  loads_issued = 0, stores_issued = 0;
            for (int i = 0; i < total + kCopyAhead && ok; i++) {
                if (i < total) {
                    if (i % cpb == 0 && !wait_landed(block_of(i / cpb))) {  // first chunk of a block: its rows are at the owner
                        ok = false;
                        break;
                    }
                    // the slot's previous store (chunk i - kCopySlots) must have left shared memory
                    if (i >= kCopySlots) bulk_wait_read<kCopySlots - 1 - kCopyAhead>();
                    const char *src;
                    char       *dst;
                    uint32_t    bytes;
                    span(i, src, dst, bytes);
                    const uint32_t bar = bars + 8u * (i % kCopySlots);
                    mbar_arrive_expect_tx(bar, bytes);
                    bulk_load(ring + (i % kCopySlots) * kCopyChunk, src, bytes, bar);
                    loads_issued = i + 1;
                }
                const int j = i - kCopyAhead;
                if (j >= 0) {
                    if (!mbar_wait(bars + 8u * (j % kCopySlots), (uint32_t)(j / kCopySlots) & 1u, ab, 7)) {
                        ok = false;
                        break;
                    }
                    const char *src;
                    char       *dst;
                    uint32_t    bytes;
                    span(j, src, dst, bytes);
                    bulk_store(dst, ring + (j % kCopySlots) * kCopyChunk, bytes);
                    bulk_commit();
                    stores_issued = j + 1;
                    const int done = j - kCopyLag;
                    if (done >= 0 && done % cpb == cpb - 1) {
                        bulk_wait<kCopyLag>();
                        announce(done / cpb);
                    }
                }
            }
            if (ok) {
                bulk_wait<0>();
                for (int done = max(total - kCopyLag, 0); done < total; done++)
                    if (done % cpb == cpb - 1) announce(done / cpb);
            } else {
                // leave no copy in flight into this CTA's shared memory: bounded second wait per slot
                for (int j = stores_issued; j < loads_issued; j++) {
                    const unsigned long long t0 = now_ns();
                    while (!mbar_try_wait(bars + 8u * (j % kCopySlots), (uint32_t)(j / kCopySlots) & 1u) &&
                           now_ns() - t0 < ab.budget_ns) {}
                }
                bulk_wait<0>();
            }
        }
    }
    __syncthreads();
    // closing barrier: nobody overwrites a shard that a peer may still be reading
    epoch++;
    __syncthreads();
    bad = 0;
    if ((int)threadIdx.x < p.tp_size) {
        const int q = threadIdx.x;
        nvl::st_release_sys(p.pad[q] + (size_t)copy_idx * nvl::kMaxRanks + rank, epoch);
        if (!nvl::wait_flag(p.pad[rank] + (size_t)copy_idx * nvl::kMaxRanks + q, epoch, ab.budget_ns)) bad = 1;
    }
    if (__syncthreads_or(bad) && threadIdx.x == 0) {
        *ab.smem = 1;
        atomicCAS(ab.global, 0u, 0x301u);
    }
    if (threadIdx.x == 0) *epoch_slot = epoch;
}

// Copier warps of the allgather mode (copy_mode 1): instead of setting whole CTAs aside for the copy, the last two
// warps of EVERY CTA pull this CTA's share of each remote row block with plain 16-byte loads from the peer and
// stores into the local gathered buffer. One SM sustains only a few tens of GB/s of remote loads, whatever engine
// issues them, so the copy is spread over all SMs, where it needs about 1.5 GB/s from each and costs no tensor
// throughput. CTA 0's copiers also run the two cross-rank barriers (peers have published their shards / everybody
// has finished reading) and release the other CTAs through a counter in local memory.
constexpr int kCopierThreads = 64;
constexpr int kGoSlot = 1100, kDoneSlot = 1101;  // words of the pad's counter area (the reduce-scatter counters end at 1024)

template <int kU>   // 16-byte loads a thread keeps in flight (as many as the kernel's register budget allows)
__device__ void copier_warps_loop(const GemmParams &p, int rank, int local, int tid, const AbortFlag &ab)
{
    const int    n_cta   = gridDim.x;
    const int    me      = blockIdx.x;
    const int    tiles_m = (p.M + kBM - 1) / kBM;
    const int    mbs     = tiles_m / p.tp_size;
    const int    a_bytes = p.a_bytes > 0 ? p.a_bytes : 2;
    const size_t blk_bytes  = (size_t)kBM * p.K * a_bytes;
    const size_t blk_packs  = blk_bytes / 16;
    const size_t per  = (blk_packs + n_cta - 1) / n_cta;
    const size_t lo   = min((size_t)me * per, blk_packs), hi = min(lo + per, blk_packs);
    const size_t sblk_bytes = (a_bytes == 1) ? (size_t)kBM * (p.K / 128) * 4 : 0;
    const size_t sblk_packs = sblk_bytes / 16;
    const size_t sper = (sblk_packs + n_cta - 1) / n_cta;
    const size_t slo  = min((size_t)me * sper, sblk_packs), shi = min(slo + sper, sblk_packs);
    uint32_t    *go   = p.pad[rank] + nvl::kPadCounterOff + kGoSlot;
    uint32_t    *done = p.pad[rank] + nvl::kPadCounterOff + kDoneSlot;
    auto sync_copiers = [] { asm volatile("bar.sync 6, 64;" ::: "memory"); };
    bool ok = true;

    if (me == 0) {
        // my own shard may still be arriving from the host: the peers are told to read it only when all of it is here
        if (tid == 0 && p.in_ready[local] != nullptr) {
            const int chunks = (p.M / p.tp_size + p.in_rows_per_flag - 1) / p.in_rows_per_flag;
            for (int c = 0; c < chunks; c++) {
                if (!wait_counter(p.in_ready[local] + c, p.in_target, true, ab, 9)) break;
            }
        }
        sync_copiers();
        // opening barrier among the ranks (flag row 0 of the pads)
        uint32_t *epoch_slot = p.pad[rank] + nvl::kPadEpochOff;
        const uint32_t epoch = *epoch_slot + 1;
        int bad = 0;
        if (tid < p.tp_size) {
            nvl::st_release_sys(p.pad[tid] + rank, epoch);
            if (!nvl::wait_flag(p.pad[rank] + tid, epoch, ab.budget_ns)) bad = 1;
        }
        if (bad) {
            *ab.smem = 1;
            atomicCAS(ab.global, 0u, 0x300u);
        }
        sync_copiers();
        if (tid == 0) {
            *epoch_slot = epoch;
            red_release_gpu_add(go, 1u);   // go counts launches: seq
        }
    }
    if (tid == 0) ok = wait_counter(go, p.seq, false, ab, 0xa);
    sync_copiers();
    ok = (*ab.smem == 0);

    // The remote row blocks in the order the tile walk needs them; this CTA copies packs [lo, hi) of each. All of it is
    // one sequence of items (block, pack) walked in batches of kCopierThreads x kU, whatever block an item belongs to:
    // NVLink round trips under load take several microseconds, so what counts is how many bytes an SM keeps in flight
    // (kU x 16 bytes per thread), not the block boundaries. A block is announced when the batch holding its last item
    // has been stored.
    const int n_blocks = (p.tp_size - 1) * mbs;
    auto blk_of = [&](int b) { return ((rank + 1 + b / mbs) % p.tp_size) * mbs + b % mbs; };
    auto copy_all = [&](size_t first, uint32_t cnt, size_t bytes_per_blk, bool scales, bool announce_blocks) {
        const uint32_t total = (uint32_t)n_blocks * cnt;
        int            announced = 0;
        for (uint32_t j0 = 0; j0 < total && ok; j0 += kCopierThreads * kU) {
            uint4 v[kU];
#pragma unroll
            for (int u = 0; u < kU; u++) {
                const uint32_t j = j0 + (uint32_t)u * kCopierThreads + (uint32_t)tid;
                if (j < total) {
                    const uint32_t b = j / cnt, i = j - b * cnt;
                    const int      blk = blk_of((int)b);
                    const char    *src = reinterpret_cast<const char *>(scales ? (const void *)p.sg[blk / mbs] : (const void *)p.xg[blk / mbs]);
                    v[u] = nvl::ld_nc16(src + (size_t)blk * bytes_per_blk + (first + i) * 16);
                }
            }
#pragma unroll
            for (int u = 0; u < kU; u++) {
                const uint32_t j = j0 + (uint32_t)u * kCopierThreads + (uint32_t)tid;
                if (j < total) {
                    const uint32_t b = j / cnt, i = j - b * cnt;
                    const int      blk = blk_of((int)b);
                    char          *dst = reinterpret_cast<char *>(scales ? (void *)p.sg[rank] : (void *)p.xg[rank]);
                    *reinterpret_cast<uint4 *>(dst + (size_t)blk * bytes_per_blk + (first + i) * 16) = v[u];
                }
            }
            sync_copiers();
            ok = (*ab.smem == 0);
            if (announce_blocks && tid == 0) {
                const uint32_t stored = min(j0 + (uint32_t)(kCopierThreads * kU), total);
                if ((uint32_t)(announced + 1) * cnt <= stored) {
                    // the TMA unit (async proxy) of any CTA of this rank reads these rows next
                    asm volatile("fence.proxy.async.global;" ::: "memory");
                    __threadfence();
                    while ((uint32_t)(announced + 1) * cnt <= stored) {
                        red_release_gpu_add(p.ready[local] + blk_of(announced), 1u);
                        announced++;
                    }
                }
            }
        }
    };
    if (ok && shi > slo) copy_all(slo, (uint32_t)(shi - slo), sblk_bytes, true, false);   // scales first: covered by the data's fence
    if (ok && hi > lo) {
        copy_all(lo, (uint32_t)(hi - lo), blk_bytes, false, true);
    } else if (ok) {
        sync_copiers();
        if (tid == 0) {
            asm volatile("fence.proxy.async.global;" ::: "memory");
            __threadfence();
            for (int bb = 0; bb < n_blocks; bb++) red_release_gpu_add(p.ready[local] + blk_of(bb), 1u);
        }
    }
    // closing: nobody overwrites a shard that a peer may still be reading
    sync_copiers();
    if (tid == 0) red_release_gpu_add(done, 1u);
    if (me == 0) {
        if (tid == 0) wait_counter(done, p.seq * (uint32_t)n_cta, false, ab, 0xb);
        sync_copiers();
        uint32_t *epoch_slot = p.pad[rank] + nvl::kPadEpochOff;
        const uint32_t epoch = *epoch_slot + 1;
        int bad = 0;
        if (tid < p.tp_size) {
            nvl::st_release_sys(p.pad[tid] + rank, epoch);
            if (!nvl::wait_flag(p.pad[rank] + tid, epoch, ab.budget_ns)) bad = 1;
        }
        if (bad) {
            *ab.smem = 1;
            atomicCAS(ab.global, 0u, 0x301u);
        }
        sync_copiers();
        if (tid == 0) *epoch_slot = epoch;
    }
}

// Reduce phase of GEMM -> reduce-scatter: every rank has stored its partial tiles for MY rows into my
// partial buffer (slot = source rank, parity = launch sequence) and counted them into my arrival
// counters; when a 128-row block has arrived from every rank, add the partials up in fp32 and write
// the bf16 result. Work items are 128 rows x 256 columns, shared out among the GEMM CTAs.
__device__ void rs_reduce_phase(const GemmParams &p, int rank, int local, int tiles_m128, const AbortFlag &ab)
{
    const int    mbs        = tiles_m128 / p.tp_size;
    const size_t shard_rows = (size_t)mbs * kBM;
    const size_t slot_elems = shard_rows * (size_t)p.N;
    const __nv_bfloat16 *mine = p.part[rank] + (size_t)(p.seq & 1) * p.tp_size * slot_elems;
    const uint32_t *ctr_base  = p.pad[rank] + nvl::kPadCounterOff + (p.seq & 1) * p.tp_size * 64;
    const int chunks_n = (p.N + kBN - 1) / kBN;
    const int items = mbs * chunks_n;
    __shared__ int item_ok;
    for (int it = blockIdx.x; it < items; it += p.n_gemm_ctas) {
        const int mb_in = it % mbs, nb = it / mbs;
        if (threadIdx.x == 0) {
            int good = 1;
            for (int src = 0; src < p.tp_size && good; src++) {
                // rs_target = tiles that rank `src` has sent for this row block over all launches
                // of this parity, this one included (the host keeps the running total)
                good = wait_counter(ctr_base + src * 64 + mb_in, p.rs_target, true, ab, 6) ? 1 : 0;
            }
            item_ok = good;
        }
        __syncthreads();
        if (!item_ok) break;
        // 128 rows x 256 columns: 32 packs of 8 bf16 per row
        for (int k = threadIdx.x; k < kBM * (kBN / 8); k += blockDim.x) {
            const int    r = k / (kBN / 8), cpk = k % (kBN / 8);
            const size_t row = (size_t)mb_in * kBM + r;
            const int    col = nb * kBN + cpk * 8;
            if (col >= p.N) continue;
            float acc[8];
#pragma unroll
            for (int e = 0; e < 8; e++) acc[e] = 0.0f;
            // all partials of this pack are requested before the first one is used
            uint4 raw[kMaxTpRanks];
#pragma unroll
            for (int src = 0; src < kMaxTpRanks; src++) {
                if (src < p.tp_size) raw[src] = nvl::ld_nc16(mine + (size_t)src * slot_elems + row * (size_t)p.N + col);
            }
#pragma unroll
            for (int src = 0; src < kMaxTpRanks; src++) {
                if (src < p.tp_size) {
                    const __nv_bfloat162 *h = reinterpret_cast<const __nv_bfloat162 *>(&raw[src]);
#pragma unroll
                    for (int e = 0; e < 4; e++) {
                        float2 f = __bfloat1622float2(h[e]);
                        acc[2 * e] += f.x;
                        acc[2 * e + 1] += f.y;
                    }
                }
            }
            uint4 o = make_uint4(pack_bf16x2(acc[0], acc[1]), pack_bf16x2(acc[2], acc[3]),
                                 pack_bf16x2(acc[4], acc[5]), pack_bf16x2(acc[6], acc[7]));
            *reinterpret_cast<uint4 *>(p.C[local] + row * (size_t)p.ldc + col) = o;
        }
        __syncthreads();
    }
}

}  // namespace
}  // namespace tp
}  // namespace xccl
