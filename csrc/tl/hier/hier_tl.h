// Hierarchy / schedule team library: collectives built from collectives of other team
// libraries on sub-groups of the team (node, socket, node leaders, socket leaders, flat).
// Counterpart of the reference's hier team (src/team_lib/hier/): the same sub-group rules and
// schedule shapes, expressed over the task engine of csrc/core/schedule.h. On an NVSwitch box
// the node level is served by the NVLink team for CUDA buffers.
#pragma once
#include <array>
#include <map>
#include <memory>
#include <vector>

#include "../../core/core.h"
#include "xccl/xccl_oob.h"

namespace xccl {
namespace hier {

enum SbgpType { SBGP_NODE = 0, SBGP_SOCKET, SBGP_NODE_LEADERS, SBGP_SOCKET_LEADERS, SBGP_FLAT, SBGP_LAST };
enum SbgpStatus { SBGP_NOT_EXISTS = 0, SBGP_DISABLED, SBGP_ENABLED };

struct ProcInfo {
    uint64_t node_hash;
    int32_t  socket_id;
    int32_t  pid;
};

struct Sbgp {
    SbgpType         type   = SBGP_FLAT;
    SbgpStatus       status = SBGP_NOT_EXISTS;
    int              group_rank = -1;
    std::vector<int> ranks;  // team ranks of the members, leader first
};

// Pure function of the placement table: exposed so that layouts can be unit-tested without
// processes. procs[i] describes team rank i.
struct Layout {
    std::array<Sbgp, SBGP_LAST> sbgp;
    int  n_nodes = 1, node_id = 0, node_leader = 0, max_ppn = 1, min_ppn = 1;
    bool sockets_usable = false;
    std::vector<int> node_of;      // node index of each team rank
    std::vector<int> leader_of;    // leader team rank of each node
};
Layout compute_layout(const std::vector<ProcInfo> &procs, int my_rank, int node_leader_rank_id);

enum PairId {
    PAIR_NODE_HOST = 0,      // node subgroup on the host team
    PAIR_NODE_DEVICE,        // node subgroup on the NVLink (or NCCL) team, CUDA buffers
    PAIR_SOCKET_HOST,
    PAIR_SOCKET_LEADERS_HOST,
    PAIR_NODE_LEADERS_HOST,
    PAIR_NODE_LEADERS_SHARP, // in-fabric reduction among node leaders when enabled
    PAIR_FLAT_HOST,
    PAIR_NODE_SHMSEG,            // shared-segment teams: FANOUT_GET broadcasts inside a node
    PAIR_SOCKET_SHMSEG,
    PAIR_SOCKET_LEADERS_SHMSEG,
    PAIR_LAST
};

struct Pair {
    const Sbgp            *sbgp = nullptr;
    xccl_team_h            team = nullptr;
    xccl_context_h         ctx  = nullptr;
    xccl_oob_collectives_t oob{};
    bool                   have_oob = false;
};

struct HierCfg {
    bool   enable_sharp = false, enable_shmseg = false, enable_hmc = false, enable_nccl = false, enable_nvlink = true;
    size_t bcast_pipeline_thresh = (size_t)-1;
    int    bcast_pipeline_depth  = 1;
    int    node_leader_rank_id   = 0;
    bool   bcast_sm_get          = false;  // host broadcasts inside a node through FANOUT_GET on the shared-segment team
    size_t bcast_sm_get_thresh   = 0;      // ... from this size on
};

class HierContext;

class HierTeam final : public TlTeam {
public:
    HierTeam(HierContext *c, const OobGroup &g);
    ~HierTeam() override;
    xccl_status_t init();
    xccl_status_t create_test() override { return XCCL_OK; }
    xccl_status_t collective_init(const xccl_coll_op_args_t &args, xccl_memory_type_t mem, xccl_coll_req **req) override;

    HierContext *hctx;
    OobGroup     oob;
    Layout       layout;
    std::vector<ProcInfo> procs;       // placement of every team rank
    xccl_ep_range_t       place_range{};  // team rank -> context rank when the team has its own OOB
    std::array<Pair, PAIR_LAST> pairs;
    bool pair_ok(PairId p) const { return pairs[p].team != nullptr; }

private:
    xccl_status_t create_pair(PairId id, SbgpType sbgp, xccl_tl_id_t tl);
    xccl_oob_collectives_t team_oob_{};
};

class HierContext final : public TlContext {
public:
    HierContext(const xccl_context_params_t &p, const HierCfg &c) : params(p), cfg(c) {}
    ~HierContext() override;
    xccl_status_t init();
    xccl_status_t progress() override;
    bool          has_progress() const override { return true; }
    xccl_status_t team_create_post(const xccl_team_params_t &tp, TlTeam **team) override;
    xccl_context_h sub(xccl_tl_id_t id) const
    {
        auto it = subctx.find(id);
        return it == subctx.end() ? nullptr : it->second;
    }

    xccl_context_params_t params;
    HierCfg               cfg;
    xccl_lib_h            lib = nullptr;
    std::map<xccl_tl_id_t, xccl_context_h> subctx;
    std::vector<ProcInfo> procs;  // by context rank
};

// One level of a schedule: a collective on one pair's team.
struct Step {
    PairId              pair;
    xccl_coll_op_args_t args;
    // which step of the same fragment has to complete first: kDepDefault = the schedule's own rule (a chain, or the
    // broadcast rule), kDepNone = starts with the schedule
    int                 after = kDepDefault;
    static constexpr int kDepDefault = -2, kDepNone = -1;
};

// Regions of a broadcast that runs its node-local levels through FANOUT_GET: one per sub-group this rank is in
// (mapped by the request before the steps are built). `offset` is where the fragment starts in the message.
struct SmGet {
    xccl_mem_h memh[SBGP_LAST] = {};
    size_t     offset          = 0;
};
// The shared-segment and host pairs that serve a node-local level.
PairId shmseg_pair(SbgpType s);
PairId host_pair(SbgpType s);

// Builders return the ordered steps THIS rank takes part in. `parallel` marks schedules whose
// steps have no dependency on each other (the two alltoallv halves).
xccl_status_t build_allreduce(HierTeam &t, const xccl_coll_op_args_t &a, xccl_memory_type_t mem, std::vector<Step> *s);
xccl_status_t build_barrier(HierTeam &t, const xccl_coll_op_args_t &a, std::vector<Step> *s);
// sm != nullptr: levels with a region in `sm` become FANOUT_GET + FANIN (the root may reuse its buffer once every
// reader has copied); every step then names its dependency itself.
xccl_status_t build_bcast(HierTeam &t, const xccl_coll_op_args_t &a, xccl_memory_type_t mem, std::vector<Step> *s,
                          int *first_dependency, const SmGet *sm = nullptr);
// The node-local levels of a broadcast this rank takes part in, with the level root's index in the group.
struct BcastLevel {
    SbgpType sbgp;
    int      root;
};
std::vector<BcastLevel> bcast_local_levels(const HierTeam &t, int root);
xccl_status_t build_alltoall(HierTeam &t, const xccl_coll_op_args_t &a, xccl_memory_type_t mem, std::vector<Step> *s,
                             bool *parallel, std::vector<std::vector<uint32_t>> *keep);

}  // namespace hier
}  // namespace xccl

extern "C" {
// Test hook: layout of `n` processes described by (node_hash[i], socket_id[i]) as seen by
// `my_rank`. out_* arrays have room for SBGP_LAST entries / n ranks.
int xccl_hier_layout_probe(int n, const uint64_t *node_hash, const int *socket_id, int my_rank, int leader_id,
                           int *status, int *group_rank, int *group_size, int *members /* [SBGP_LAST][n] */);
}
