// MoE expert dispatch / combine fused with the all-to-all (extension; the reference only has
// alltoallv call sites: src/team_lib/nccl/xccl_nccl_collective.c:125-163).
//
// dispatch (ONE kernel): count tokens per expert, exchange the counts with every rank through
//   peer memory, turn them into receive offsets, and copy every routed token row straight into its
//   slot of the destination rank's receive buffer - rows arrive grouped by (local expert, source
//   rank), ready for a grouped GEMM. No host round trip, no intermediate permuted copy.
// combine (ONE kernel): every token pulls its top-k expert outputs from the owners' buffers and
//   adds them up with its gate weights in fp32.
// Ranks are real (one process per GPU) or emulated (blockIdx.y = rank in one cooperative launch).
// Waits on peers are bounded; a timeout sets the workspace's error word and the kernel drains.
#include <cooperative_groups.h>
#include <cuda_bf16.h>

#include <algorithm>
#include <cstring>
#include <vector>

#include "../core/core.h"
#include "../cuda/cuda_common.h"
#include "../tl/nvlink/nvl_device.cuh"
#include "../tl/nvlink/nvl_shm.h"
#include "moe.h"

namespace cg = cooperative_groups;

namespace xccl {
namespace moe {

constexpr int kMaxRanks   = 8;
constexpr int kMaxExperts = 1024;

struct MoeParams {
    int T, H, E, K, tp, rank_base, n_local;
    int cap_rows;
    unsigned long long budget_ns;
    // per TEAM rank (as mapped here)
    uint32_t      *pad[kMaxRanks];
    uint32_t      *cnt[kMaxRanks];    // [tp][E_local] tokens from each source for each local expert
    uint32_t      *base[kMaxRanks];   // [E_local][tp] first row of (local expert, source)
    __nv_bfloat16 *recv[kMaxRanks];   // [cap_rows][H]
    __nv_bfloat16 *yout[kMaxRanks];   // [cap_rows][H] expert outputs, same row numbering
    int32_t       *rsrc[kMaxRanks];   // [cap_rows] source rank * T + token
    // per LOCAL rank
    uint32_t *local_cnt[kMaxRanks];   // [E] my tokens per global expert
    uint32_t *send_base[kMaxRanks];   // [E] first row at the destination for my tokens of expert e
    uint32_t *pos[kMaxRanks];         // [T*K] position among my tokens of the same expert
    uint32_t *slot[kMaxRanks];        // [T*K] row at the destination (kept for combine)
    uint32_t *expert_rows[kMaxRanks]; // [E_local + 1] rows per local expert, total last
    uint32_t *error[kMaxRanks];
    const __nv_bfloat16 *x[kMaxRanks];
    const int32_t       *ids[kMaxRanks];
    const float         *w[kMaxRanks];
    __nv_bfloat16       *out[kMaxRanks];
};

namespace {

// Barrier among block 0 of every rank (flags row 0 of the pads), bounded.
__device__ bool cross_rank_barrier_block0(const MoeParams &p, int rank, uint32_t &epoch)
{
    epoch++;
    __syncthreads();
    int bad = 0;
    if ((int)threadIdx.x < p.tp) {
        const int q = threadIdx.x;
        nvl::st_release_sys(p.pad[q] + rank, epoch);
        if (!nvl::wait_flag(p.pad[rank] + q, epoch, p.budget_ns)) bad = 1;
    }
    return __syncthreads_or(bad) == 0;
}

__global__ void __launch_bounds__(512) moe_dispatch_kernel(MoeParams p)
{
    cg::grid_group grid  = cg::this_grid();
    const int      local = blockIdx.y, rank = p.rank_base + local;
    const int      EL    = p.E / p.tp;
    const int      nent  = p.T * p.K;
    const size_t   tid   = (size_t)blockIdx.x * blockDim.x + threadIdx.x, nthr = (size_t)gridDim.x * blockDim.x;
    uint32_t      *lcnt  = p.local_cnt[local];
    const int32_t *ids   = p.ids[local];
    __shared__ uint32_t s_epoch;
    __shared__ int      s_ok;

    // 0. clear my per-expert counters
    for (size_t e = tid; e < (size_t)p.E; e += nthr) lcnt[e] = 0;
    grid.sync();
    // 1. position of every routed entry among my entries of the same expert
    for (size_t i = tid; i < (size_t)nent; i += nthr) {
        int e = ids[i];
        p.pos[local][i] = (e >= 0 && e < p.E) ? atomicAdd(&lcnt[e], 1u) : 0u;
    }
    grid.sync();
    // 2. block 0: publish my counts to the owners, agree, build my receive offsets, publish them
    if (blockIdx.x == 0) {
        if (threadIdx.x == 0) s_epoch = p.pad[rank][nvl::kPadEpochOff];
        __syncthreads();
        uint32_t epoch = s_epoch;
        for (int e = threadIdx.x; e < p.E; e += blockDim.x) {
            const int d = e / EL, le = e % EL;
            nvl::st_release_sys(p.cnt[d] + (size_t)rank * EL + le, lcnt[e]);
        }
        bool ok = cross_rank_barrier_block0(p, rank, epoch);
        if (ok && threadIdx.x == 0) {
            // rows grouped by local expert, then by source rank
            uint32_t row = 0;
            for (int le = 0; le < EL; le++) {
                uint32_t start = row;
                for (int s = 0; s < p.tp; s++) {
                    p.base[rank][le * p.tp + s] = row;
                    row += nvl::ld_relaxed_sys(p.cnt[rank] + (size_t)s * EL + le);
                }
                p.expert_rows[local][le] = row - start;
            }
            p.expert_rows[local][EL] = row;
            if (row > (uint32_t)p.cap_rows) atomicExch(p.error[local], 0x400u);  // receive buffer too small
            __threadfence_system();
        }
        ok = ok && cross_rank_barrier_block0(p, rank, epoch);
        if (ok) {
            for (int e = threadIdx.x; e < p.E; e += blockDim.x) {
                const int d = e / EL, le = e % EL;
                p.send_base[local][e] = nvl::ld_relaxed_sys(p.base[d] + le * p.tp + rank);
            }
        }
        if (threadIdx.x == 0) {
            p.pad[rank][nvl::kPadEpochOff] = epoch;
            if (!ok) atomicExch(p.error[local], 0x401u);
            __threadfence();
        }
    }
    grid.sync();
    if (threadIdx.x == 0) s_ok = (*(volatile uint32_t *)p.error[local] == 0);
    __syncthreads();
    // 3. every routed row goes straight to its slot at the owner: one warp per entry
    if (s_ok) {
        const int    lane = threadIdx.x % 32;
        const size_t warp = tid / 32, nwarps = nthr / 32;
        const int    packs = p.H * 2 / 16;
        for (size_t i = warp; i < (size_t)nent; i += nwarps) {
            const int e = ids[i];
            if (e < 0 || e >= p.E) continue;
            const int      d   = e / EL, t = (int)(i / p.K);
            const uint32_t row = p.send_base[local][e] + p.pos[local][i];
            if (lane == 0) {
                p.slot[local][i] = row;
                p.rsrc[d][row]   = rank * p.T + t;
            }
            const uint4 *src = reinterpret_cast<const uint4 *>(p.x[local] + (size_t)t * p.H);
            uint4       *dst = reinterpret_cast<uint4 *>(p.recv[d] + (size_t)row * p.H);
            for (int k = lane; k < packs; k += 32) nvl::st_16(dst + k, src[k]);
        }
    }
    __threadfence_system();
    grid.sync();
    // 4. everything has landed everywhere before anyone returns
    if (blockIdx.x == 0 && s_ok) {
        uint32_t epoch = p.pad[rank][nvl::kPadEpochOff];
        __syncthreads();
        bool ok = cross_rank_barrier_block0(p, rank, epoch);
        if (threadIdx.x == 0) {
            p.pad[rank][nvl::kPadEpochOff] = epoch;
            if (!ok) atomicExch(p.error[local], 0x402u);
        }
    }
}

__global__ void __launch_bounds__(512) moe_combine_kernel(MoeParams p)
{
    cg::grid_group grid  = cg::this_grid();
    const int      local = blockIdx.y, rank = p.rank_base + local;
    const int      EL    = p.E / p.tp;
    __shared__ int s_ok;
    // the experts' outputs must be complete on every rank before anyone pulls
    if (blockIdx.x == 0) {
        uint32_t epoch = p.pad[rank][nvl::kPadEpochOff];
        __syncthreads();
        bool ok = cross_rank_barrier_block0(p, rank, epoch);
        if (threadIdx.x == 0) {
            p.pad[rank][nvl::kPadEpochOff] = epoch;
            if (!ok) atomicExch(p.error[local], 0x403u);
            __threadfence();
        }
    }
    grid.sync();
    if (threadIdx.x == 0) s_ok = (*(volatile uint32_t *)p.error[local] == 0);
    __syncthreads();
    if (s_ok) {
        const size_t tid  = (size_t)blockIdx.x * blockDim.x + threadIdx.x, nthr = (size_t)gridDim.x * blockDim.x;
        const int    lane = threadIdx.x % 32;
        const size_t warp = tid / 32, nwarps = nthr / 32;
        const int    packs = p.H * 2 / 16;
        for (size_t t = warp; t < (size_t)p.T; t += nwarps) {
            // routing entries of this token, eight at a time: lane k holds entry k, the warp shares them
            // (with more than eight entries the running sum passes through bf16 between groups)
            for (int kb = 0; kb < p.K; kb += 8) {
                const int kn = min(8, p.K - kb);
                const uint4 *my_row = nullptr;
                float        my_g   = 0.0f;
                if (lane < kn) {
                    const size_t i = t * p.K + kb + lane;
                    const int    e = p.ids[local][i];
                    if (e >= 0 && e < p.E) {
                        my_g   = p.w[local][i];
                        my_row = reinterpret_cast<const uint4 *>(p.yout[e / EL] + (size_t)p.slot[local][i] * p.H);
                    }
                }
                const uint4 *rows[8];
                float        gs[8];
#pragma unroll
                for (int k = 0; k < 8; k++) {
                    rows[k] = reinterpret_cast<const uint4 *>(__shfl_sync(0xffffffffu, (unsigned long long)my_row, k));
                    gs[k]   = __shfl_sync(0xffffffffu, my_g, k);
                }
                for (int k0 = lane; k0 < packs; k0 += 32) {
                    // all expert rows of the pack are requested before the first one is used
                    uint4 raw[8];
#pragma unroll
                    for (int k = 0; k < 8; k++) raw[k] = rows[k] ? nvl::ld_nc16(rows[k] + k0) : make_uint4(0, 0, 0, 0);
                    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
                    uint4 *dst = reinterpret_cast<uint4 *>(p.out[local] + t * p.H) + k0;
                    if (kb > 0) {
                        const uint4 prev = *dst;
                        const __nv_bfloat162 *ph = reinterpret_cast<const __nv_bfloat162 *>(&prev);
#pragma unroll
                        for (int j = 0; j < 4; j++) {
                            float2 f = __bfloat1622float2(ph[j]);
                            acc[2 * j] = f.x;
                            acc[2 * j + 1] = f.y;
                        }
                    }
#pragma unroll
                    for (int k = 0; k < 8; k++) {
                        const __nv_bfloat162 *h = reinterpret_cast<const __nv_bfloat162 *>(&raw[k]);
#pragma unroll
                        for (int j = 0; j < 4; j++) {
                            float2 f = __bfloat1622float2(h[j]);
                            acc[2 * j] += gs[k] * f.x;
                            acc[2 * j + 1] += gs[k] * f.y;
                        }
                    }
                    uint4 o;
                    __nv_bfloat162 *oh = reinterpret_cast<__nv_bfloat162 *>(&o);
#pragma unroll
                    for (int j = 0; j < 4; j++) oh[j] = __floats2bfloat162_rn(acc[2 * j], acc[2 * j + 1]);
                    *dst = o;
                }
            }
        }
    }
    grid.sync();
    // nobody's buffer is reused while a peer may still be reading it
    if (blockIdx.x == 0 && s_ok) {
        uint32_t epoch = p.pad[rank][nvl::kPadEpochOff];
        __syncthreads();
        bool ok = cross_rank_barrier_block0(p, rank, epoch);
        if (threadIdx.x == 0) {
            p.pad[rank][nvl::kPadEpochOff] = epoch;
            if (!ok) atomicExch(p.error[local], 0x404u);
        }
    }
}

size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

}  // namespace

struct MoeWorkspace {
    MoeParams             p{};
    bool                  emulated = false;
    nvl::SymmetricRegion *region   = nullptr;
    std::vector<void *>   allocs;
    char                 *sym[kMaxRanks] = {nullptr};
    size_t                off_cnt = 0, off_base = 0, off_rsrc = 0, off_recv = 0, off_yout = 0, total = 0;
    int                   blocks = 0;
};

}  // namespace moe
}  // namespace xccl

using namespace xccl;
using namespace xccl::moe;

extern "C" {

xccl_status_t xccl_moe_ws_create(const xccl_oob_collectives_t *oob, int emu_ranks, int T, int H, int E, int K,
                                 int cap_rows, xccl_moe_ws_h *out)
{
    if (out == nullptr || T <= 0 || H <= 0 || (H * 2) % 16 != 0 || E <= 0 || E > kMaxExperts || K <= 0) return XCCL_ERR_INVALID_PARAM;
    if (!cuda_available()) return XCCL_ERR_NO_RESOURCE;
    auto *w      = new MoeWorkspace;
    MoeParams &p = w->p;
    p.T = T; p.H = H; p.E = E; p.K = K;
    p.budget_ns = 4000000000ull;
    w->emulated = (oob == nullptr);
    p.tp        = w->emulated ? std::max(emu_ranks, 1) : oob->size;
    p.n_local   = w->emulated ? p.tp : 1;
    p.rank_base = w->emulated ? 0 : oob->rank;
    if (p.tp > kMaxRanks || E % p.tp != 0) {
        delete w;
        return XCCL_ERR_INVALID_PARAM;
    }
    const int EL = E / p.tp;
    p.cap_rows   = cap_rows > 0 ? cap_rows : p.tp * T * K;
    w->off_cnt   = align_up(nvl::kPadBytes, 4096);
    w->off_base  = align_up(w->off_cnt + (size_t)p.tp * EL * 4, 4096);
    w->off_rsrc  = align_up(w->off_base + (size_t)p.tp * EL * 4, 4096);
    w->off_recv  = align_up(w->off_rsrc + (size_t)p.cap_rows * 4, 4096);
    w->off_yout  = align_up(w->off_recv + (size_t)p.cap_rows * H * 2, 4096);
    w->total     = align_up(w->off_yout + (size_t)p.cap_rows * H * 2, 4096);
    xccl_status_t st = XCCL_OK;
    if (w->emulated) {
        for (int r = 0; r < p.tp && st == XCCL_OK; r++) {
            void *q = nullptr;
            if (cudaMalloc(&q, w->total) != cudaSuccess) {
                (void)cudaGetLastError();
                st = XCCL_ERR_NO_MEMORY;
                break;
            }
            w->allocs.push_back(q);
            cudaMemset(q, 0, w->off_recv);
            w->sym[r] = (char *)q;
        }
    } else {
        OobGroup g;
        g.oob = *oob; g.range.type = XCCL_EP_RANGE_UNDEFINED; g.rank = oob->rank; g.size = oob->size;
        st = nvl::SymmetricRegion::create(g, w->total, false, &w->region);
        if (st == XCCL_OK) {
            for (int r = 0; r < p.tp; r++) w->sym[r] = w->region->base[(size_t)r];
        }
    }
    for (int r = 0; r < p.tp && st == XCCL_OK; r++) {
        p.pad[r]  = (uint32_t *)w->sym[r];
        p.cnt[r]  = (uint32_t *)(w->sym[r] + w->off_cnt);
        p.base[r] = (uint32_t *)(w->sym[r] + w->off_base);
        p.rsrc[r] = (int32_t *)(w->sym[r] + w->off_rsrc);
        p.recv[r] = (__nv_bfloat16 *)(w->sym[r] + w->off_recv);
        p.yout[r] = (__nv_bfloat16 *)(w->sym[r] + w->off_yout);
    }
    auto dev_alloc = [&](size_t bytes) -> void * {
        void *q = nullptr;
        if (cudaMalloc(&q, bytes) != cudaSuccess) {
            st = XCCL_ERR_NO_MEMORY;
            return nullptr;
        }
        cudaMemset(q, 0, bytes);
        w->allocs.push_back(q);
        return q;
    };
    for (int l = 0; l < p.n_local && st == XCCL_OK; l++) {
        p.local_cnt[l]   = (uint32_t *)dev_alloc((size_t)E * 4);
        p.send_base[l]   = (uint32_t *)dev_alloc((size_t)E * 4);
        p.pos[l]         = (uint32_t *)dev_alloc((size_t)T * K * 4);
        p.slot[l]        = (uint32_t *)dev_alloc((size_t)T * K * 4);
        p.expert_rows[l] = (uint32_t *)dev_alloc((size_t)(EL + 1) * 4);
        p.error[l]       = (uint32_t *)dev_alloc(4);
    }
    int dev = 0, sms = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    w->blocks = std::max(1, sms / p.n_local);
    cudaDeviceSynchronize();
    if (st != XCCL_OK) {
        xccl_moe_ws_destroy(w);
        return st;
    }
    *out = w;
    return XCCL_OK;
}

void xccl_moe_ws_destroy(xccl_moe_ws_h w)
{
    if (w == nullptr) return;
    cudaDeviceSynchronize();
    for (void *q : w->allocs) cudaFree(q);
    delete w->region;
    delete w;
}

static xccl_status_t launch_coop(void *kernel, MoeWorkspace *w, cudaStream_t s)
{
    void *args[] = {&w->p};
    dim3  grid((unsigned)w->blocks, (unsigned)w->p.n_local), block(512);
    XCCL_CUDA_CHECK(cudaLaunchCooperativeKernel(kernel, grid, block, args, 0, s));
    return XCCL_OK;
}

xccl_status_t xccl_moe_dispatch(xccl_moe_ws_h w, const void *const *x, const int32_t *const *ids, void *stream)
{
    if (w == nullptr || x == nullptr || ids == nullptr) return XCCL_ERR_INVALID_PARAM;
    for (int l = 0; l < w->p.n_local; l++) {
        w->p.x[l]   = (const __nv_bfloat16 *)x[l];
        w->p.ids[l] = ids[l];
    }
    return launch_coop((void *)moe_dispatch_kernel, w, (cudaStream_t)stream);
}

xccl_status_t xccl_moe_combine(xccl_moe_ws_h w, const int32_t *const *ids, const float *const *weights, void *const *out,
                               void *stream)
{
    if (w == nullptr || ids == nullptr || weights == nullptr || out == nullptr) return XCCL_ERR_INVALID_PARAM;
    for (int l = 0; l < w->p.n_local; l++) {
        w->p.ids[l] = ids[l];
        w->p.w[l]   = weights[l];
        w->p.out[l] = (__nv_bfloat16 *)out[l];
    }
    return launch_coop((void *)moe_combine_kernel, w, (cudaStream_t)stream);
}

void *xccl_moe_ws_buffer(xccl_moe_ws_h w, int local_rank, int which)
{
    if (w == nullptr || local_rank < 0 || local_rank >= w->p.n_local) return nullptr;
    const int r = w->p.rank_base + local_rank;
    switch (which) {
    case XCCL_MOE_BUF_RECV: return w->p.recv[r];
    case XCCL_MOE_BUF_EXPERT_OUT: return w->p.yout[r];
    case XCCL_MOE_BUF_EXPERT_ROWS: return w->p.expert_rows[local_rank];
    case XCCL_MOE_BUF_ROW_SOURCE: return w->p.rsrc[r];
    default: return nullptr;
    }
}

int xccl_moe_ws_cap_rows(xccl_moe_ws_h w) { return w != nullptr ? w->p.cap_rows : 0; }

uint32_t xccl_moe_ws_error(xccl_moe_ws_h w)
{
    if (w == nullptr) return 0xffffffffu;
    uint32_t worst = 0;
    for (int l = 0; l < w->p.n_local; l++) {
        uint32_t v = 0;
        cudaMemcpy(&v, w->p.error[l], 4, cudaMemcpyDeviceToHost);
        if (v != 0) worst = v;
    }
    return worst;
}

}  // extern "C"
