// Sub-group computation of the hierarchy layer. Rules (reference: src/team_lib/hier/xccl_hier_sbgp.c):
//  NODE            team ranks on my host; rotated so that the configured leader comes first
//  SOCKET          NODE members on my CPU socket; the node leader, if a member, sits at index 0
//  NODE_LEADERS    one rank per node; enabled on leaders, disabled elsewhere, absent on one node
//  SOCKET_LEADERS  first rank of every socket of my node, the node leader first
//  FLAT            everyone
// Every group's leader is its member 0, so rooted levels of a schedule always use root 0.
// Socket levels are dropped for the whole team when any rank is not bound to exactly one socket.
#include <algorithm>

#include "hier_tl.h"

namespace xccl {
namespace hier {

Layout compute_layout(const std::vector<ProcInfo> &procs, int me, int leader_id)
{
    Layout    L;
    const int n = (int)procs.size();
    L.node_of.assign((size_t)n, -1);
    std::vector<uint64_t>         hashes;
    std::vector<std::vector<int>> members;
    for (int i = 0; i < n; i++) {
        size_t k = 0;
        for (; k < hashes.size(); k++) {
            if (hashes[k] == procs[(size_t)i].node_hash) break;
        }
        if (k == hashes.size()) {
            hashes.push_back(procs[(size_t)i].node_hash);
            members.emplace_back();
        }
        members[k].push_back(i);
        L.node_of[(size_t)i] = (int)k;
    }
    L.n_nodes = (int)hashes.size();
    L.node_id = L.node_of[(size_t)me];
    L.max_ppn = 0;
    L.min_ppn = n;
    for (auto &m : members) {
        L.max_ppn = std::max(L.max_ppn, (int)m.size());
        L.min_ppn = std::min(L.min_ppn, (int)m.size());
        L.leader_of.push_back((leader_id > 0 && leader_id < (int)m.size()) ? m[(size_t)leader_id] : m[0]);
    }
    L.node_leader    = L.leader_of[(size_t)L.node_id];
    L.sockets_usable = true;
    for (auto &p : procs) L.sockets_usable = L.sockets_usable && p.socket_id >= 0;

    auto index_of = [](const std::vector<int> &v, int x) {
        auto it = std::find(v.begin(), v.end(), x);
        return it == v.end() ? -1 : (int)(it - v.begin());
    };

    // NODE
    Sbgp &node = L.sbgp[SBGP_NODE];
    node.type  = SBGP_NODE;
    node.ranks = members[(size_t)L.node_id];
    if (leader_id > 0 && leader_id < (int)node.ranks.size()) {
        std::rotate(node.ranks.begin(), node.ranks.begin() + leader_id, node.ranks.end());
    }
    node.group_rank = index_of(node.ranks, me);
    node.status     = node.ranks.size() > 1 ? SBGP_ENABLED : SBGP_NOT_EXISTS;

    // SOCKET
    Sbgp &sock = L.sbgp[SBGP_SOCKET];
    sock.type  = SBGP_SOCKET;
    if (L.sockets_usable) {
        for (int r : node.ranks) {
            if (procs[(size_t)r].socket_id == procs[(size_t)me].socket_id) sock.ranks.push_back(r);
        }
        int pos = index_of(sock.ranks, L.node_leader);
        if (pos > 0) std::swap(sock.ranks[0], sock.ranks[(size_t)pos]);
        sock.group_rank = index_of(sock.ranks, me);
        sock.status     = sock.ranks.size() > 1 ? SBGP_ENABLED : SBGP_NOT_EXISTS;
    }

    // NODE_LEADERS
    Sbgp &nl = L.sbgp[SBGP_NODE_LEADERS];
    nl.type  = SBGP_NODE_LEADERS;
    if (L.n_nodes > 1) {
        nl.ranks      = L.leader_of;
        nl.group_rank = index_of(nl.ranks, me);
        nl.status     = nl.group_rank >= 0 ? SBGP_ENABLED : SBGP_DISABLED;
    }

    // SOCKET_LEADERS
    Sbgp &sl = L.sbgp[SBGP_SOCKET_LEADERS];
    sl.type  = SBGP_SOCKET_LEADERS;
    if (L.sockets_usable) {
        std::vector<int> seen;
        for (int r : node.ranks) {  // leader first, so it represents its own socket at index 0
            int s = procs[(size_t)r].socket_id;
            if (std::find(seen.begin(), seen.end(), s) == seen.end()) {
                seen.push_back(s);
                sl.ranks.push_back(r);
            }
        }
        if (sl.ranks.size() > 1) {
            sl.group_rank = index_of(sl.ranks, me);
            sl.status     = sl.group_rank >= 0 ? SBGP_ENABLED : SBGP_DISABLED;
        } else {
            sl.ranks.clear();
        }
    }

    // FLAT
    Sbgp &flat = L.sbgp[SBGP_FLAT];
    flat.type  = SBGP_FLAT;
    for (int i = 0; i < n; i++) flat.ranks.push_back(i);
    flat.group_rank = me;
    flat.status     = n > 1 ? SBGP_ENABLED : SBGP_NOT_EXISTS;
    return L;
}

}  // namespace hier
}  // namespace xccl

extern "C" int xccl_hier_layout_probe(int n, const uint64_t *node_hash, const int *socket_id, int my_rank, int leader_id,
                                      int *status, int *group_rank, int *group_size, int *members)
{
    using namespace xccl::hier;
    std::vector<ProcInfo> procs((size_t)n);
    for (int i = 0; i < n; i++) procs[(size_t)i] = ProcInfo{node_hash[i], socket_id[i], i};
    Layout L = compute_layout(procs, my_rank, leader_id);
    for (int s = 0; s < SBGP_LAST; s++) {
        status[s]     = (int)L.sbgp[(size_t)s].status;
        group_rank[s] = L.sbgp[(size_t)s].group_rank;
        group_size[s] = (int)L.sbgp[(size_t)s].ranks.size();
        for (size_t k = 0; k < L.sbgp[(size_t)s].ranks.size(); k++) members[s * n + (int)k] = L.sbgp[(size_t)s].ranks[k];
    }
    return L.n_nodes;
}
