// Schedule builders of the hierarchy layer: which collective runs on which sub-group, in what
// order, for THIS rank. Shapes follow the reference (src/team_lib/hier/xccl_hier_schedule_allreduce.c:16-141,
// xccl_hier_schedule_barrier.c:16-140, xccl_hier_schedule_bcast.c:172-311,
// xccl_hier_schedule_alltoall.c:11-120):
//
//   allreduce  reduce up the levels (socket -> socket leaders), allreduce on the highest level
//              that exists, broadcast back down; without socket binding: node -> node leaders
//   barrier    the same shape with fan-in / barrier / fan-out
//   bcast      every rank is a non-root in at most one level: that level runs first, the levels it
//              roots start together afterwards
//   alltoall   one node: one alltoall on the node team; several nodes: two independent alltoallv,
//              node-local peers on the node team and remote peers on the flat host team
#include <algorithm>

#include "hier_tl.h"

namespace xccl {
namespace hier {

namespace {

bool member(const HierTeam &t, SbgpType s) { return t.layout.sbgp[s].status == SBGP_ENABLED; }
bool exists(const HierTeam &t, SbgpType s) { return t.layout.sbgp[s].status != SBGP_NOT_EXISTS; }

// The team that serves the node level for this memory type.
PairId node_pair(const HierTeam &t, xccl_memory_type_t mem)
{
    return (mem == XCCL_MEMORY_TYPE_CUDA && t.pair_ok(PAIR_NODE_DEVICE)) ? PAIR_NODE_DEVICE : PAIR_NODE_HOST;
}

struct Level {
    SbgpType sbgp;
    PairId   pair;
};

// Levels, bottom to top, that exist for the team (not necessarily for this rank).
std::vector<Level> levels_of(const HierTeam &t, xccl_memory_type_t mem)
{
    std::vector<Level> lv;
    const bool sockets = t.layout.sockets_usable && exists(t, SBGP_SOCKET_LEADERS);
    if (sockets) {
        lv.push_back({SBGP_SOCKET, PAIR_SOCKET_HOST});
        lv.push_back({SBGP_SOCKET_LEADERS, PAIR_SOCKET_LEADERS_HOST});
    } else if (exists(t, SBGP_NODE)) {
        lv.push_back({SBGP_NODE, node_pair(t, mem)});
    }
    if (exists(t, SBGP_NODE_LEADERS)) {
        lv.push_back({SBGP_NODE_LEADERS,
                      t.pair_ok(PAIR_NODE_LEADERS_SHARP) ? PAIR_NODE_LEADERS_SHARP : PAIR_NODE_LEADERS_HOST});
    }
    return lv;
}

// With socket levels, the SOCKET group may be absent on a socket that holds a single rank while
// SOCKET_LEADERS still exists: exists() is per team, member() per rank.
xccl_status_t up_and_down(HierTeam &t, const xccl_coll_op_args_t &a, xccl_memory_type_t mem, xccl_collective_type_t up,
                          xccl_collective_type_t top, xccl_collective_type_t down, std::vector<Step> *out)
{
    std::vector<Level> lv = levels_of(t, mem);
    xccl_coll_op_args_t base = a;
    base.alg.set_by_user = 0;
    base.field_mask &= ~(uint64_t)XCCL_COLL_OP_ARGS_FIELD_EPILOGUE;
    if (lv.empty()) {
        // a team of one rank: nothing to exchange, but allreduce still has to produce dst
        return XCCL_ERR_UNSUPPORTED;
    }
    const size_t       top_idx = lv.size() - 1;
    std::vector<Step>  ups, downs;
    bool               first = true;
    for (size_t i = 0; i < lv.size(); i++) {
        if (!member(t, lv[i].sbgp)) continue;
        if (!t.pair_ok(lv[i].pair)) return XCCL_ERR_NO_RESOURCE;
        Step s{lv[i].pair, base};
        s.args.root = 0;
        if (!first && a.coll_type == XCCL_ALLREDUCE) {
            s.args.buffer_info.src_buffer = a.buffer_info.dst_buffer;  // partial results live in dst from now on
        }
        first = false;
        if (i == top_idx) {
            s.args.coll_type = top;
            ups.push_back(s);
        } else {
            s.args.coll_type = up;
            ups.push_back(s);
            Step d = s;
            d.args.coll_type              = down;
            d.args.buffer_info.src_buffer = a.buffer_info.dst_buffer;
            downs.push_back(d);
        }
    }
    // A rank that is not in the top level still took part in lower ones; the level list is the
    // same for all ranks, so "top" is decided per team, not per rank.
    *out = ups;
    for (auto it = downs.rbegin(); it != downs.rend(); ++it) out->push_back(*it);
    return out->empty() ? XCCL_ERR_NO_RESOURCE : XCCL_OK;
}

int index_in(const std::vector<int> &v, int x)
{
    auto it = std::find(v.begin(), v.end(), x);
    return it == v.end() ? -1 : (int)(it - v.begin());
}

}  // namespace

xccl_status_t build_allreduce(HierTeam &t, const xccl_coll_op_args_t &a, xccl_memory_type_t mem, std::vector<Step> *s)
{
    return up_and_down(t, a, mem, XCCL_REDUCE, XCCL_ALLREDUCE, XCCL_BCAST, s);
}

xccl_status_t build_barrier(HierTeam &t, const xccl_coll_op_args_t &a, std::vector<Step> *s)
{
    // synchronisation has no buffer: always the host teams
    return up_and_down(t, a, XCCL_MEMORY_TYPE_HOST, XCCL_FANIN, XCCL_BARRIER, XCCL_FANOUT, s);
}

PairId shmseg_pair(SbgpType s)
{
    return s == SBGP_SOCKET ? PAIR_SOCKET_SHMSEG : s == SBGP_SOCKET_LEADERS ? PAIR_SOCKET_LEADERS_SHMSEG : PAIR_NODE_SHMSEG;
}

PairId host_pair(SbgpType s)
{
    return s == SBGP_SOCKET ? PAIR_SOCKET_HOST : s == SBGP_SOCKET_LEADERS ? PAIR_SOCKET_LEADERS_HOST : PAIR_NODE_HOST;
}

std::vector<BcastLevel> bcast_local_levels(const HierTeam &t, int root)
{
    const Layout &L = t.layout;
    std::vector<BcastLevel> lv;
    const bool root_on_node   = L.node_of[(size_t)root] == L.node_id;
    const bool root_on_socket = root_on_node && t.procs[(size_t)root].socket_id == t.procs[(size_t)t.rank].socket_id;
    const bool sockets        = L.sockets_usable && exists(t, SBGP_SOCKET_LEADERS);
    if (sockets) {
        int r = 0;
        if (root_on_node) {
            const auto &ranks = L.sbgp[SBGP_SOCKET_LEADERS].ranks;
            for (size_t i = 0; i < ranks.size(); i++) {
                if (t.procs[(size_t)ranks[i]].socket_id == t.procs[(size_t)root].socket_id) r = (int)i;
            }
        }
        if (member(t, SBGP_SOCKET_LEADERS)) lv.push_back({SBGP_SOCKET_LEADERS, r});
        r = root_on_socket ? std::max(0, index_in(L.sbgp[SBGP_SOCKET].ranks, root)) : 0;
        if (member(t, SBGP_SOCKET)) lv.push_back({SBGP_SOCKET, r});
    } else {
        int r = root_on_node ? std::max(0, index_in(L.sbgp[SBGP_NODE].ranks, root)) : 0;
        if (member(t, SBGP_NODE)) lv.push_back({SBGP_NODE, r});
    }
    return lv;
}

// Reference shape: src/team_lib/hier/xccl_hier_schedule_bcast.c:172-311; the FANOUT_GET variant with its closing
// FANIN: the same file, :313-485 (there the regions are mapped by the schedule's first progress step, here by the
// request before it builds its fragments).
xccl_status_t build_bcast(HierTeam &t, const xccl_coll_op_args_t &a, xccl_memory_type_t mem, std::vector<Step> *out,
                          int *first_dependency, const SmGet *sm)
{
    const Layout &L    = t.layout;
    const int     root = a.root;
    if (root < 0 || root >= t.size) return XCCL_ERR_INVALID_PARAM;
    xccl_coll_op_args_t base  = a;
    base.alg.set_by_user      = 0;
    // the data ends up in dst on every rank; the root's src is read only in the level it roots
    int              dep = -1;      // the step in which this rank receives
    std::vector<int> mains;         // the data-moving step of each level
    std::vector<std::pair<int, int>> fanins;  // (step, its level's data-moving step)
    auto add = [&](SbgpType sb, PairId pair, int level_root) -> xccl_status_t {
        if (!member(t, sb)) return XCCL_OK;
        const bool get = sm != nullptr && sm->memh[sb] != nullptr;
        if (get) pair = shmseg_pair(sb);
        if (!t.pair_ok(pair)) return XCCL_ERR_NO_RESOURCE;
        Step s{pair, base};
        s.args.root = level_root;
        if (t.rank != root) s.args.buffer_info.src_buffer = a.buffer_info.dst_buffer;
        if (get) {
            s.args.coll_type             = XCCL_FANOUT_GET;
            s.args.field_mask            = 0;
            s.args.get_info.memh         = sm->memh[sb];
            s.args.get_info.offset       = (ptrdiff_t)sm->offset;
            s.args.get_info.len          = a.buffer_info.len;
            s.args.get_info.local_buffer = a.buffer_info.dst_buffer;
        }
        if (level_root != L.sbgp[sb].group_rank) dep = (int)out->size();
        mains.push_back((int)out->size());
        out->push_back(s);
        if (get) {
            // the level root learns that every reader has copied: its buffer and the window may be reused
            if (!t.pair_ok(host_pair(sb))) return XCCL_ERR_NO_RESOURCE;
            Step f{host_pair(sb), xccl_coll_op_args_t{}};
            f.args.coll_type = XCCL_FANIN;
            f.args.root      = level_root;
            fanins.push_back({(int)out->size(), mains.back()});
            out->push_back(f);
        }
        return XCCL_OK;
    };
    xccl_status_t st = XCCL_OK;
    if (exists(t, SBGP_NODE_LEADERS)) {
        PairId p = PAIR_NODE_LEADERS_HOST;
        st       = add(SBGP_NODE_LEADERS, p, L.node_of[(size_t)root]);
        if (st != XCCL_OK) return st;
    }
    for (const BcastLevel &lv : bcast_local_levels(t, root)) {
        st = add(lv.sbgp, lv.sbgp == SBGP_NODE ? node_pair(t, mem) : host_pair(lv.sbgp), lv.root);
        if (st != XCCL_OK) return st;
    }
    if (out->empty()) return XCCL_ERR_UNSUPPORTED;
    // Where the root is not the leader of its group, the leader RECEIVES in the lower level and
    // roots the upper one, so "the level where I am not the root" is the one to run first.
    *first_dependency = dep >= 0 ? dep : 0;
    if (sm != nullptr) {
        for (int m : mains) (*out)[(size_t)m].after = (m == *first_dependency) ? Step::kDepNone : *first_dependency;
        for (auto &f : fanins) (*out)[(size_t)f.first].after = f.second;
    }
    return XCCL_OK;
}

xccl_status_t build_alltoall(HierTeam &t, const xccl_coll_op_args_t &a, xccl_memory_type_t mem, std::vector<Step> *out,
                             bool *parallel, std::vector<std::vector<uint32_t>> *keep)
{
    const Layout &L = t.layout;
    *parallel       = false;
    if (t.size == 1) return XCCL_ERR_UNSUPPORTED;  // nothing to schedule: the next team library copies the block
    if (a.buffer_info.src_buffer == XCCL_IN_PLACE || a.buffer_info.src_buffer == a.buffer_info.dst_buffer) {
        return XCCL_ERR_UNSUPPORTED;
    }
    if (L.n_nodes == 1) {
        PairId p = node_pair(t, mem);
        if (!member(t, SBGP_NODE) || !t.pair_ok(p)) return XCCL_ERR_NO_RESOURCE;
        // member i of the node group is team rank ranks[i]; the plain alltoall needs identity order
        const auto &ranks = L.sbgp[SBGP_NODE].ranks;
        bool        ident = true;
        for (size_t i = 0; i < ranks.size(); i++) ident = ident && ranks[i] == (int)i;
        if (ident) {
            Step s{p, a};
            s.args.alg.set_by_user = 0;
            out->push_back(s);
            return XCCL_OK;
        }
    }
    if (a.buffer_info.len > 0xffffffffull) return XCCL_ERR_UNSUPPORTED;
    const uint32_t len = (uint32_t)a.buffer_info.len;
    auto vstep = [&](PairId pair, const std::vector<int> &ranks, bool local_part) {
        // counts in bytes (uint8 elements); blocks keep their place in the full-team buffers
        std::vector<uint32_t> cnt(ranks.size()), dsp(ranks.size());
        for (size_t i = 0; i < ranks.size(); i++) {
            bool on_node = L.node_of[(size_t)ranks[i]] == L.node_id;
            bool mine    = local_part ? true : !(on_node && member(t, SBGP_NODE));
            cnt[i]       = mine ? len : 0;
            dsp[i]       = (uint32_t)ranks[i] * len;
        }
        keep->push_back(cnt);
        keep->push_back(dsp);
        Step s{pair, a};
        s.args.coll_type                     = XCCL_ALLTOALLV;
        s.args.alg.set_by_user               = 0;
        s.args.buffer_info.src_datatype      = XCCL_DT_UINT8;
        s.args.buffer_info.dst_datatype      = XCCL_DT_UINT8;
        s.args.buffer_info.len               = 0;
        out->push_back(s);
    };
    if ((uint64_t)len * (uint64_t)t.size > 0xffffffffull) return XCCL_ERR_UNSUPPORTED;
    if (member(t, SBGP_NODE)) {
        if (!t.pair_ok(PAIR_NODE_HOST)) return XCCL_ERR_NO_RESOURCE;
        // variable-count exchange inside the node; the device team is used when it can take it
        vstep(node_pair(t, mem), L.sbgp[SBGP_NODE].ranks, true);
    }
    if (L.n_nodes > 1) {
        if (!t.pair_ok(PAIR_FLAT_HOST)) return XCCL_ERR_NO_RESOURCE;
        vstep(PAIR_FLAT_HOST, L.sbgp[SBGP_FLAT].ranks, false);
    }
    // pointers are taken only now: `keep` no longer reallocates
    size_t k = keep->size() - 2 * out->size();
    for (Step &s : *out) {
        s.args.buffer_info.src_counts        = (*keep)[k].data();
        s.args.buffer_info.dst_counts        = (*keep)[k].data();
        s.args.buffer_info.src_displacements = (*keep)[k + 1].data();
        s.args.buffer_info.dst_displacements = (*keep)[k + 1].data();
        k += 2;
    }
    *parallel = out->size() > 1;
    return out->empty() ? XCCL_ERR_UNSUPPORTED : XCCL_OK;
}

}  // namespace hier
}  // namespace xccl
