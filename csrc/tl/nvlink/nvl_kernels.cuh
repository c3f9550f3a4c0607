// Launch interface of the NVLink collectives (implemented in nvl_kernels.cu).
#pragma once
#include <cuda_runtime.h>

#include "nvl_device.cuh"
#include "xccl/xccl.h"

namespace xccl {
namespace nvl {

// Per-launch arguments. Arrays are indexed by LOCAL rank (blockIdx.y): one entry in a real
// multi-process team, `size` entries when one kernel emulates every rank.
struct Call {
    const void     *src[kMaxRanks];
    void           *dst[kMaxRanks];
    const uint32_t *vmeta[kMaxRanks];  // alltoallv: device array [4][size] = src_counts, src_displs, dst_counts, dst_displs
    size_t          count;             // elements of the reduction
    size_t          len;               // bytes, meaning as in xccl_coll_buffer_info_t::len
    int             op;
    int             root;
    float           scale;
    int             do_scale;
    int             parity;            // which half of the workspace this launch uses
    int             src_es, dst_es;    // alltoallv element sizes
    int             push;              // allgather / alltoall: store into the destinations' workspaces (one chunk only)
    // Direct algorithms: every rank's user buffers as mapped in this process, by TEAM rank (peer
    // mappings of registered buffers in a real team, the plain pointers when ranks are emulated).
    const void     *peer_src[kMaxRanks];
    void           *peer_dst[kMaxRanks];
    // Symmetric algorithms: the buffers of this call seen through the multicast mapping of the symmetric
    // allocation they live in (same offset on every rank), by LOCAL rank.
    const void     *mc_src[kMaxRanks];
    void           *mc_dst[kMaxRanks];
};

enum Alg { ALG_AUTO = 0, ALG_ONE_SHOT = 1, ALG_TWO_SHOT = 2, ALG_NVLS = 3, ALG_DIRECT = 4, ALG_SYMMETRIC = 5 };

struct LaunchCfg {
    int  blocks  = 0;      // 0 = choose from the message size
    int  threads = 512;
    bool cooperative = false;  // all ranks in one launch: blocks wait on one another
    int  max_blocks = kMaxBlocks;
};

// Workspace bytes a collective needs in one half; 0 when it streams in chunks of any size.
size_t one_shot_limit(const World &w);

xccl_status_t launch_allreduce(const World &w, const Call &c, xccl_dt_t dt, xccl_dt_t out_dt, Alg alg,
                               const LaunchCfg &cfg, cudaStream_t stream);
// nvls = true: the reducing ranks read through the multicast mapping (multimem.ld_reduce; needs w.mc_ws, a sum of
// fp32 / fp16 / bf16)
xccl_status_t launch_reduce(const World &w, const Call &c, xccl_dt_t dt, xccl_dt_t out_dt, const LaunchCfg &cfg,
                            cudaStream_t stream, bool nvls = false);
xccl_status_t launch_reduce_scatter(const World &w, const Call &c, xccl_dt_t dt, xccl_dt_t out_dt,
                                    const LaunchCfg &cfg, cudaStream_t stream, bool nvls = false);
// multicast = true: root writes once through the NVSwitch multicast mapping (needs w.mc_ws)
xccl_status_t launch_bcast(const World &w, const Call &c, const LaunchCfg &cfg, cudaStream_t stream,
                           bool multicast = false);
xccl_status_t launch_allgather(const World &w, const Call &c, const LaunchCfg &cfg, cudaStream_t stream);
xccl_status_t launch_alltoall(const World &w, const Call &c, const LaunchCfg &cfg, cudaStream_t stream);
xccl_status_t launch_alltoallv(const World &w, const Call &c, size_t max_src_bytes, const LaunchCfg &cfg,
                               cudaStream_t stream);
// Direct (zero-copy) algorithms on registered user buffers, for messages where staging through the
// workspace costs more than it hides. coll: XCCL_ALLREDUCE, XCCL_REDUCE_SCATTER, XCCL_ALLGATHER or
// XCCL_ALLTOALL. All buffers 16-byte aligned, byte counts multiples of 16.
xccl_status_t launch_direct(const World &w, const Call &c, int coll, xccl_dt_t dt, xccl_dt_t out_dt, const LaunchCfg &cfg,
                            cudaStream_t stream);
bool          direct_shape_ok(int coll, const Call &c, xccl_dt_t dt, int team_size);
// Zero-copy NVLS on symmetric memory: c.mc_src / c.mc_dst are multicast addresses of the buffers (bcast: mc_dst only,
// c.src is the root's plain source). coll: XCCL_ALLREDUCE (sum of fp32 / fp16 / bf16, same output type) or XCCL_BCAST.
// Buffers 16-byte aligned, byte counts multiples of 16.
xccl_status_t launch_symmetric(const World &w, const Call &c, int coll, xccl_dt_t dt, const LaunchCfg &cfg, cudaStream_t stream);
// kind: XCCL_BARRIER, XCCL_FANIN or XCCL_FANOUT
xccl_status_t launch_sync(const World &w, const Call &c, int kind, const LaunchCfg &cfg, cudaStream_t stream);
// A barrier whose flags nobody sets, with a short budget: reports NVL_TIMEOUT in the status
// words and returns. Exercises the failure path without involving another rank.
xccl_status_t launch_timeout_probe(const World &w, unsigned long long budget_ns, cudaStream_t stream);

bool nvls_supported(xccl_dt_t dt, xccl_op_t op);
// allgather / alltoall: true when the whole exchange fits one workspace half in the push layout
bool push_fits(const World &w, int coll, size_t len);

}  // namespace nvl
}  // namespace xccl
