// Host-side owner of an NVLink "world": the workspaces, signal pads and (optionally) the NVLS
// multicast mapping that the kernels of nvl_kernels.cu operate on.
//
// Two ways to build one:
//  - create_emulated(): N ranks inside ONE process on ONE device. All ranks' buffers are plain
//    device allocations and a collective is a single cooperative launch with gridDim.y = N.
//    It exists so that every kernel can be tested on a single GPU (kernels that wait for each
//    other must never run as separate launches on one GPU).
//  - bootstrap over an OobGroup (nvl_team.cu): one process per GPU, CUDA VMM allocations shared
//    as POSIX file descriptors over unix sockets, peers mapped into this process.
#pragma once
#include <cuda_runtime.h>

#include <vector>

#include "nvl_kernels.cuh"

namespace xccl {
namespace nvl {

struct HostStatus {
    uint32_t code, rank, peer, epoch;
};

class EmuWorld {
public:
    ~EmuWorld();
    static xccl_status_t create(int nranks, size_t ws_bytes, EmuWorld **out);
    World          world{};
    int            parity = 0;
    // status of local rank i after the stream is idle
    HostStatus     status(int i) const;
    void           clear_status();
    unsigned long long budget_ns = 2000000000ull;

private:
    std::vector<void *> allocs_;
    HostStatus         *status_host_ = nullptr;  // mapped pinned memory, kMaxRanks entries
};

// Number of workspace halves a launch consumes (so the caller can advance `parity`).
int chunks_used(const World &w, xccl_collective_type_t coll, size_t count, size_t len, xccl_dt_t dt, bool multicast = false);

}  // namespace nvl
}  // namespace xccl

extern "C" {
// Test / benchmark hooks for the single-GPU emulation.
xccl_status_t xccl_nvlink_emu_create(int nranks, size_t ws_bytes, void **world);
void          xccl_nvlink_emu_destroy(void *world);
// Runs one collective over all emulated ranks and waits for it. srcs/dsts hold one device
// pointer per rank; vmeta (alltoallv only) one device array [4][nranks] of uint32 per rank.
// Returns XCCL_OK, an argument error, or XCCL_ERR_TIMED_OUT when a bounded wait expired.
xccl_status_t xccl_nvlink_emu_collective(void *world, int coll_type, const void *const *srcs, void *const *dsts,
                                         size_t count, size_t len, int dt, int out_dt, int op, int root, float scale,
                                         int alg, const uint32_t *const *vmeta, size_t max_src_bytes, int es,
                                         int blocks, void *stream);
xccl_status_t xccl_nvlink_emu_timeout_probe(void *world, int budget_ms, float *elapsed_ms, uint32_t *status4);
}
