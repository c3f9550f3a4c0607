// Device-side vocabulary of the NVLink team: the world description every kernel receives,
// system-scope loads/stores, the bounded cross-GPU block barrier and multimem (NVLS) wrappers.
//
// Memory model. Each rank owns a "signal pad" and a "workspace" that all ranks have mapped.
// Block b of rank r synchronises ONLY with block b of every other rank: work is partitioned so
// that whatever block b of a rank reads was produced by block b of its peers, so no grid-wide
// synchronisation is needed and blocks pipeline independently.
// A barrier is: bar.sync; thread p stores the new epoch into peer p's pad slot
// [block][my rank] with release.sys and then polls its own slot [block][p] with acquire.sys;
// bar.sync. Epochs only grow, so flags are never reset. Every poll loop has a time budget
// read from %globaltimer; when it runs out the kernel records {code, rank, peer, epoch} in the
// rank's status words, skips the rest of its work and returns normally.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace xccl {
namespace nvl {

constexpr int kMaxRanks  = 16;
constexpr int kMaxBlocks = 128;

// layout of a signal pad, in 32-bit words
constexpr int kPadFlagWords   = kMaxBlocks * kMaxRanks;   // barrier flags [block][source rank]
constexpr int kPadEpochOff    = kPadFlagWords;            // per-block epoch counters, owner-private
constexpr int kPadCounterOff  = kPadEpochOff + kMaxBlocks;   // general counters for fused kernels
constexpr int kPadCounterWords = 2048;
constexpr int kPadWords       = kPadCounterOff + kPadCounterWords;
constexpr size_t kPadBytes    = ((size_t)kPadWords * 4 + 4095) & ~(size_t)4095;

enum StatusCode : uint32_t { NVL_OK = 0, NVL_TIMEOUT = 1, NVL_BAD_ARG = 2 };

struct World {
    int       size;        // team size
    int       rank_base;   // team rank served by blockIdx.y == 0 (0 when all ranks are emulated)
    int       n_local;     // ranks served by this launch (gridDim.y): 1, or `size` when emulated
    int       reserved;
    char     *ws[kMaxRanks];      // workspaces as mapped in this process
    uint32_t *pad[kMaxRanks];     // signal pads as mapped in this process
    uint32_t *status[kMaxRanks];  // 4 words per LOCAL rank (index blockIdx.y): code, rank, peer, epoch
    char     *mc_ws;              // multicast (NVLS) view of the workspaces, or nullptr
    size_t    ws_bytes;           // bytes of one workspace (two halves of ws_bytes / 2)
    unsigned long long wait_budget_ns;
    size_t    mc_bcast_cap;       // multicast bcast: packs per chunk (0 = a whole workspace half), so that copying chunk k
                                  // out overlaps the root's push of chunk k+1
};

__device__ __forceinline__ void st_release_sys(uint32_t *p, uint32_t v)
{
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t *p)
{
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ uint32_t ld_relaxed_sys(const uint32_t *p)
{
    uint32_t v;
    asm volatile("ld.relaxed.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void red_release_sys_add(uint32_t *p, uint32_t v)
{
    asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned long long global_ns()
{
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

// 16-byte accesses that bypass L1 (peer memory must not be served from a stale L1 line)
__device__ __forceinline__ uint4 ld_nc16(const void *p)
{
    uint4 v;
    asm volatile("ld.relaxed.sys.global.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p)
                 : "memory");
    return v;
}
__device__ __forceinline__ void st_16(void *p, uint4 v)
{
    asm volatile("st.relaxed.sys.global.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
                 : "memory");
}

// Per-kernel view of "who am I".
struct Self {
    int      rank;    // team rank
    int      local;   // blockIdx.y
    uint32_t epoch;   // last epoch used by this block
    bool     failed;
};

__device__ __forceinline__ Self self_begin(const World &w)
{
    Self s;
    s.local  = blockIdx.y;
    s.rank   = w.rank_base + blockIdx.y;
    s.epoch  = w.pad[s.rank][kPadEpochOff + blockIdx.x];
    s.failed = false;
    return s;
}

// Must be reached by every thread of the block.
__device__ __forceinline__ void self_end(const World &w, const Self &s)
{
    __syncthreads();
    if (threadIdx.x == 0) {
        w.pad[s.rank][kPadEpochOff + blockIdx.x] = s.epoch;
    }
}

__device__ __forceinline__ void record_failure(const World &w, const Self &s, uint32_t code, int peer, uint32_t epoch)
{
    uint32_t *st = w.status[s.local];
    if (atomicCAS(st, 0u, code) == 0u) {
        st[1] = (uint32_t)s.rank;
        st[2] = (uint32_t)peer;
        st[3] = epoch;
        __threadfence_system();
    }
}

// Bounded wait until *flag has reached `epoch` (wrap-safe). Returns false on timeout.
__device__ __forceinline__ bool wait_flag(const uint32_t *flag, uint32_t epoch, unsigned long long budget_ns)
{
    if ((int32_t)(ld_acquire_sys(flag) - epoch) >= 0) return true;
    const unsigned long long t0 = global_ns();
    for (;;) {
#pragma unroll 1
        for (int i = 0; i < 64; i++) {
            if ((int32_t)(ld_acquire_sys(flag) - epoch) >= 0) return true;
        }
        if (global_ns() - t0 > budget_ns) return false;
    }
}

// Cross-rank barrier among the blocks with this blockIdx.x. All threads of the block call it.
// After a failure every later barrier is skipped, so a failed kernel drains quickly.
__device__ __forceinline__ void block_barrier(const World &w, Self &s)
{
    s.epoch++;
    if (s.failed) return;
    __syncthreads();
    int bad = 0;
    if ((int)threadIdx.x < w.size) {
        const int p = threadIdx.x;
        st_release_sys(w.pad[p] + (size_t)blockIdx.x * kMaxRanks + s.rank, s.epoch);
        if (!wait_flag(w.pad[s.rank] + (size_t)blockIdx.x * kMaxRanks + p, s.epoch, w.wait_budget_ns)) {
            record_failure(w, s, NVL_TIMEOUT, p, s.epoch);
            bad = 1;
        }
    }
    s.failed = __syncthreads_or(bad) != 0;
}

// One-directional pieces of the barrier, for fan-in / fan-out and producer-consumer kernels.
__device__ __forceinline__ void signal_rank(const World &w, const Self &s, int peer, uint32_t epoch)
{
    st_release_sys(w.pad[peer] + (size_t)blockIdx.x * kMaxRanks + s.rank, epoch);
}
__device__ __forceinline__ bool wait_rank(const World &w, const Self &s, int peer, uint32_t epoch)
{
    return wait_flag(w.pad[s.rank] + (size_t)blockIdx.x * kMaxRanks + peer, epoch, w.wait_budget_ns);
}

// ------------------------------------------------------------------ NVLS (multimem)
// Addresses are in the multicast mapping: a load-reduce returns the combination of the same
// offset in every rank's memory, computed in the switch; a store writes every rank's copy.

__device__ __forceinline__ uint4 mm_ld_reduce_add_f32x4(const void *mc)
{
    uint4 v;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(mc)
                 : "memory");
    return v;
}
__device__ __forceinline__ uint4 mm_ld_reduce_add_bf16x8(const void *mc)
{
    uint4 v;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(mc)
                 : "memory");
    return v;
}
__device__ __forceinline__ uint4 mm_ld_reduce_add_f16x8(const void *mc)
{
    uint4 v;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.f16x2 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(mc)
                 : "memory");
    return v;
}
__device__ __forceinline__ void mm_st_16(void *mc, uint4 v)
{
    asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(mc), "r"(v.x), "r"(v.y), "r"(v.z),
                 "r"(v.w)
                 : "memory");
}

}  // namespace nvl
}  // namespace xccl
