// Host point-to-point team ("ucx" id): every collective of the API on host buffers, and on
// CUDA buffers by staging through pinned host memory. Counterpart of the reference's UCX team
// (src/team_lib/ucx/, option table src/team_lib/ucx/xccl_ucx_lib.c:38-127).
#pragma once
#include <deque>
#include <mutex>
#include <vector>

#include "../../core/core.h"
#include "coro.h"
#include "transport.h"

namespace xccl {
namespace host {

struct HostCfg {
    int         barrier_radix = 4, bcast_radix = 4, reduce_radix = 4, allreduce_radix = 4;
    std::string allreduce_alg = "auto";
    int         a2a_chunk = 1, a2a_barrier = 0;
    bool        a2a_reverse = false, block_stream = false;
    size_t      ring_bytes = 1 << 20;
    size_t      sra_threshold = 4096;
    int         num_to_probe  = 10;  // transport polls per test call before it reports "in progress"
};

class HostTeam;

// Resolved view of a collective's arguments on host-addressable memory.
struct Bufs {
    char     *src = nullptr, *dst = nullptr;
    size_t    len = 0, count = 0;
    xccl_dt_t dt  = XCCL_DT_UNSUPPORTED;
    xccl_op_t op  = XCCL_OP_UNSUPPORTED;
    int       root = 0;
    std::vector<uint32_t> src_counts, src_displs, dst_counts, dst_displs;
    size_t    src_dt_size = 1, dst_dt_size = 1;
};

class HostReq final : public xccl_coll_req {
public:
    HostReq(HostTeam *team, const xccl_coll_op_args_t &args, xccl_memory_type_t mem);
    ~HostReq() override;
    xccl_status_t prepare();  // validates, picks the algorithm
    xccl_status_t post() override;
    xccl_status_t test() override;
    xccl_status_t finalize() override;

    // --- used by the algorithm coroutines
    P2pReq *send(int peer, const void *buf, size_t len);
    P2pReq *recv(int peer, void *buf, size_t len);
    bool    all_done();        // drives the transport, then checks every message posted so far
    void    drop_completed();  // forget finished messages (between rounds)
    void    progress();
    xccl_status_t reduce_multi(const void *a, const void *vecs, void *dst, size_t n, size_t count, size_t stride);
    char   *scratch(size_t bytes);  // grows; contents are not preserved across calls

    HostTeam           *team;
    xccl_coll_op_args_t args;
    xccl_memory_type_t  mem;
    Bufs                b;
    uint32_t            tag = 0;
    int                 alg = 0;

private:
    Coro run();
    Coro (*algo_)(HostReq &) = nullptr;
    Coro              coro_;
    bool              in_flight_ = false;
    xccl_status_t     last_      = XCCL_OK;
    std::deque<P2pReq> p2p_;
    std::vector<char>  scratch_;
    // CUDA staging
    char  *h_src_ = nullptr, *h_dst_ = nullptr;
    size_t h_src_bytes_ = 0, h_dst_bytes_ = 0;
    void  *d_src_ = nullptr, *d_dst_ = nullptr;
    void  *event_ = nullptr;
    struct StreamHoldRef;
    void  *hold_ = nullptr;
    // fused epilogue (scale, cast): the algorithm reduces into epi_buf_, the result is converted into epi_dst_
    bool              epi_ = false;
    float             epi_scale_ = 1.0f;
    xccl_dt_t         epi_out_dt_ = XCCL_DT_UNSUPPORTED;
    size_t            epi_count_ = 0;
    char             *epi_dst_ = nullptr;
    std::vector<char> epi_buf_;
};

class HostTeam final : public TlTeam {
public:
    HostTeam(TeamLib *tl, const OobGroup &g, const HostCfg &cfg);
    ~HostTeam() override;
    xccl_status_t create_test() override;
    xccl_status_t collective_init(const xccl_coll_op_args_t &args, xccl_memory_type_t mem, xccl_coll_req **req) override;

    TeamLib              *tl;
    OobGroup              oob;
    HostCfg               cfg;
    Transport             tr;
    std::recursive_mutex  mu;      // contexts in THREAD_MODE_MULTIPLE may progress a team from several threads
    uint16_t              seq = 0;
    xccl_status_t         start();

private:
    PeerInfo              mine_{};
    std::vector<PeerInfo> all_;
    void                 *oob_req_ = nullptr;
    int                   phase_   = 0;
};

// Algorithms (algorithms.cc). Each runs on r.b and returns XCCL_OK or an error.
Coro allreduce_knomial(HostReq &r);
Coro allreduce_sra(HostReq &r);
Coro reduce_knomial(HostReq &r);
Coro reduce_linear(HostReq &r);
Coro bcast_knomial(HostReq &r);
Coro bcast_linear(HostReq &r);
Coro barrier_knomial(HostReq &r);
Coro fanin_linear(HostReq &r);
Coro fanout_linear(HostReq &r);
Coro allgather_ring(HostReq &r);
Coro alltoall_pairwise(HostReq &r);
Coro alltoall_linear_shift(HostReq &r);
Coro alltoallv_pairwise(HostReq &r);
Coro reduce_scatter_pairwise(HostReq &r);

// Layout helper of the recursive k-nomial exchange, exposed for unit tests.
struct KnomialLayout {
    int radix, size, full_size, n_rounds;
    enum Role { BASE, PROXY, EXTRA } role;
    int partner;  // proxy of an extra / extra of a proxy, else -1
};
KnomialLayout knomial_layout(int rank, int size, int radix);
// peers of `rank` in round `round` (all < full_size), in ascending k order
std::vector<int> knomial_peers(const KnomialLayout &l, int rank, int round);

}  // namespace host
}  // namespace xccl

extern "C" {
// Test hook: writes the peers of (rank, round) into out[], returns how many; role/n_rounds via pointers.
int xccl_host_knomial_peers(int rank, int size, int radix, int round, int *out, int *role, int *n_rounds, int *partner);
}
