// Single-GPU emulation of an N-rank NVLink world (see nvl_world.h).
#include <algorithm>
#include <cstring>

#include "../../cuda/cuda_common.h"
#include "nvl_world.h"

namespace xccl {
namespace nvl {

EmuWorld::~EmuWorld()
{
    for (void *p : allocs_) cudaFree(p);
    if (status_host_ != nullptr) cudaFreeHost(status_host_);
}

xccl_status_t EmuWorld::create(int nranks, size_t ws_bytes, EmuWorld **out)
{
    if (nranks < 1 || nranks > kMaxRanks || ws_bytes < (1u << 16)) return XCCL_ERR_INVALID_PARAM;
    if (!cuda_available()) return XCCL_ERR_NO_RESOURCE;
    auto *e = new EmuWorld;
    ws_bytes &= ~(size_t)511;
    World &w      = e->world;
    w.size        = nranks;
    w.rank_base   = 0;
    w.n_local     = nranks;
    w.mc_ws       = nullptr;
    w.ws_bytes    = ws_bytes;
    w.wait_budget_ns = e->budget_ns;
    cudaError_t err = cudaHostAlloc((void **)&e->status_host_, sizeof(HostStatus) * kMaxRanks, cudaHostAllocMapped);
    if (err != cudaSuccess) {
        delete e;
        return cuda_status(err);
    }
    std::memset(e->status_host_, 0, sizeof(HostStatus) * kMaxRanks);
    HostStatus *sdev = nullptr;
    cudaHostGetDevicePointer((void **)&sdev, e->status_host_, 0);
    for (int r = 0; r < nranks; r++) {
        void *pad = nullptr, *ws = nullptr;
        if (cudaMalloc(&pad, kPadBytes) != cudaSuccess || cudaMalloc(&ws, ws_bytes) != cudaSuccess) {
            (void)cudaGetLastError();
            if (pad != nullptr) cudaFree(pad);
            delete e;
            return XCCL_ERR_NO_MEMORY;
        }
        e->allocs_.push_back(pad);
        e->allocs_.push_back(ws);
        cudaMemset(pad, 0, kPadBytes);
        w.pad[r]    = (uint32_t *)pad;
        w.ws[r]     = (char *)ws;
        w.status[r] = (uint32_t *)(sdev + r);
    }
    cudaDeviceSynchronize();
    *out = e;
    return XCCL_OK;
}

HostStatus EmuWorld::status(int i) const { return status_host_[i]; }

void EmuWorld::clear_status() { std::memset(status_host_, 0, sizeof(HostStatus) * kMaxRanks); }

int chunks_used(const World &w, xccl_collective_type_t coll, size_t count, size_t len, xccl_dt_t dt, bool multicast)
{
    const size_t half = w.ws_bytes / 2, cap = half / 16;
    const size_t es   = std::max<size_t>(xccl_dt_size(dt), 1);
    size_t       packs = 0, div = 1;
    switch (coll) {
    case XCCL_ALLREDUCE:
    case XCCL_REDUCE: packs = (count * es + 15) / 16; break;
    case XCCL_REDUCE_SCATTER:
        packs = (count * es + 15) / 16;
        div   = (size_t)w.size;
        break;
    case XCCL_BCAST: packs = (len + 15) / 16; break;
    case XCCL_ALLGATHER: packs = (len / (size_t)w.size + 15) / 16; break;
    case XCCL_ALLTOALL:
        packs = (len + 15) / 16;
        div   = (size_t)w.size;
        break;
    default: return 1;
    }
    size_t c = std::max<size_t>(cap / div, 1);
    if (coll == XCCL_BCAST && multicast && w.mc_bcast_cap != 0) c = std::min(c, w.mc_bcast_cap);  // as in mover_kernel
    return (int)std::max<size_t>((packs + c - 1) / c, 1);
}

}  // namespace nvl
}  // namespace xccl

using namespace xccl;
using namespace xccl::nvl;

extern "C" {

xccl_status_t xccl_nvlink_emu_create(int nranks, size_t ws_bytes, void **world)
{
    EmuWorld     *e  = nullptr;
    xccl_status_t st = EmuWorld::create(nranks, ws_bytes, &e);
    if (st == XCCL_OK) *world = e;
    return st;
}

void xccl_nvlink_emu_destroy(void *world) { delete (EmuWorld *)world; }

xccl_status_t xccl_nvlink_emu_collective(void *world, int coll_type, const void *const *srcs, void *const *dsts,
                                         size_t count, size_t len, int dt, int out_dt, int op, int root, float scale,
                                         int alg, const uint32_t *const *vmeta, size_t max_src_bytes, int es,
                                         int blocks, void *stream)
{
    auto *e = (EmuWorld *)world;
    World w = e->world;
    Call  c{};
    for (int r = 0; r < w.size; r++) {
        c.src[r]   = srcs != nullptr ? srcs[r] : nullptr;
        c.dst[r]   = dsts != nullptr ? dsts[r] : nullptr;
        c.vmeta[r] = vmeta != nullptr ? vmeta[r] : nullptr;
    }
    c.count    = count;
    c.len      = len;
    c.op       = op;
    c.root     = root;
    c.scale    = scale;
    c.do_scale = (scale != 1.0f);
    c.parity   = e->parity & 1;
    c.src_es = c.dst_es = es;
    c.push   = (alg == ALG_ONE_SHOT && (coll_type == XCCL_ALLGATHER || coll_type == XCCL_ALLTOALL) && push_fits(w, coll_type, len)) ? 1 : 0;
    LaunchCfg cfg;
    cfg.cooperative = true;
    cfg.blocks      = blocks;
    cudaStream_t  s = (cudaStream_t)stream;
    xccl_status_t st;
    if (alg == ALG_DIRECT) {
        // emulated ranks share one address space: the "registered" peer buffers are the buffers themselves
        for (int r = 0; r < w.size; r++) {
            c.peer_src[r] = c.src[r];
            c.peer_dst[r] = c.dst[r];
        }
        st = launch_direct(w, c, coll_type, (xccl_dt_t)dt, (xccl_dt_t)out_dt, cfg, s);
        if (st != XCCL_OK) return st;
        XCCL_CUDA_CHECK(cudaStreamSynchronize(s));
        for (int r = 0; r < w.size; r++) {
            if (e->status(r).code == NVL_TIMEOUT) return XCCL_ERR_TIMED_OUT;
            if (e->status(r).code != NVL_OK) return XCCL_ERR_NO_MESSAGE;
        }
        return XCCL_OK;
    }
    switch (coll_type) {
    case XCCL_ALLREDUCE: {
        Alg a = (Alg)alg;
        if (a == ALG_AUTO) a = (count * xccl_dt_size((xccl_dt_t)dt) <= one_shot_limit(w) / 4) ? ALG_ONE_SHOT : ALG_TWO_SHOT;
        st = launch_allreduce(w, c, (xccl_dt_t)dt, (xccl_dt_t)out_dt, a, cfg, s);
        e->parity += (a == ALG_ONE_SHOT) ? 1 : chunks_used(w, XCCL_ALLREDUCE, count, len, (xccl_dt_t)dt);
        break;
    }
    case XCCL_REDUCE:
        st = launch_reduce(w, c, (xccl_dt_t)dt, (xccl_dt_t)out_dt, cfg, s);
        e->parity += chunks_used(w, XCCL_REDUCE, count, len, (xccl_dt_t)dt);
        break;
    case XCCL_REDUCE_SCATTER:
        st = launch_reduce_scatter(w, c, (xccl_dt_t)dt, (xccl_dt_t)out_dt, cfg, s);
        e->parity += chunks_used(w, XCCL_REDUCE_SCATTER, count, len, (xccl_dt_t)dt);
        break;
    case XCCL_BCAST:
        st = launch_bcast(w, c, cfg, s);
        e->parity += chunks_used(w, XCCL_BCAST, count, len, (xccl_dt_t)dt);
        break;
    case XCCL_ALLGATHER:
        st = launch_allgather(w, c, cfg, s);
        e->parity += chunks_used(w, XCCL_ALLGATHER, count, len, (xccl_dt_t)dt);
        break;
    case XCCL_ALLTOALL:
        st = launch_alltoall(w, c, cfg, s);
        e->parity += chunks_used(w, XCCL_ALLTOALL, count, len, (xccl_dt_t)dt);
        break;
    case XCCL_ALLTOALLV:
        st = launch_alltoallv(w, c, max_src_bytes, cfg, s);
        e->parity += 1;
        break;
    case XCCL_BARRIER:
    case XCCL_FANIN:
    case XCCL_FANOUT: st = launch_sync(w, c, coll_type, cfg, s); break;
    default: st = XCCL_ERR_UNSUPPORTED;
    }
    if (st != XCCL_OK) return st;
    XCCL_CUDA_CHECK(cudaStreamSynchronize(s));
    for (int r = 0; r < w.size; r++) {
        if (e->status(r).code == NVL_TIMEOUT) return XCCL_ERR_TIMED_OUT;
        if (e->status(r).code != NVL_OK) return XCCL_ERR_NO_MESSAGE;
    }
    return XCCL_OK;
}

xccl_status_t xccl_nvlink_emu_timeout_probe(void *world, int budget_ms, float *elapsed_ms, uint32_t *status4)
{
    auto *e = (EmuWorld *)world;
    e->clear_status();
    cudaEvent_t e0, e1;
    XCCL_CUDA_CHECK(cudaEventCreate(&e0));
    XCCL_CUDA_CHECK(cudaEventCreate(&e1));
    XCCL_CUDA_CHECK(cudaEventRecord(e0, nullptr));
    World w   = e->world;
    w.n_local = 1;  // only rank 0 probes
    xccl_status_t st = launch_timeout_probe(w, (unsigned long long)budget_ms * 1000000ull, nullptr);
    if (st != XCCL_OK) return st;
    XCCL_CUDA_CHECK(cudaEventRecord(e1, nullptr));
    XCCL_CUDA_CHECK(cudaEventSynchronize(e1));
    if (elapsed_ms != nullptr) cudaEventElapsedTime(elapsed_ms, e0, e1);
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    HostStatus hs = e->status(0);
    if (status4 != nullptr) {
        status4[0] = hs.code;
        status4[1] = hs.rank;
        status4[2] = hs.peer;
        status4[3] = hs.epoch;
    }
    e->clear_status();
    return hs.code == NVL_TIMEOUT ? XCCL_ERR_TIMED_OUT : XCCL_OK;
}

}  // extern "C"
