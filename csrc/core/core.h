// Objects behind the public handles and the process-wide state.
#pragma once
#include <memory>
#include <string>
#include <vector>

#include "config.h"
#include "schedule.h"
#include "tl.h"

namespace xccl {

// Read once per process (reference: xccl_constructor, src/core/xccl_init.c:126-164).
struct GlobalState {
    OptTable    opts;
    uint64_t    host_hash = 0;   // djb2 of the host name: equal on ranks of one node
    int         pid       = 0;
    int         socket_id = -1;  // logical CPU socket this process is bound to, -1 if not exactly one
    std::string host_name;
};
GlobalState &global_state();

}  // namespace xccl

struct xccl_lib_config {
    xccl::OptTable global;
    std::string    env_prefix;
};

struct xccl_lib {
    std::vector<xccl::TeamLib *> tls;   // TLs that passed the params filter
    xccl_lib_params_t            params{};
    // whether team library `id` opened on this machine and passed the filter (composite team libraries ask before
    // they try an optional level, so that a level that cannot exist here is left out without an error message)
    bool has(xccl_tl_id_t id) const
    {
        for (const xccl::TeamLib *t : tls) {
            if (t->id == id) return true;
        }
        return false;
    }
};

struct xccl_context_config {
    xccl_lib   *lib = nullptr;
    std::string env_prefix;
    // one table of context options per TL of the lib, in lib order
    std::vector<xccl::OptTable> tables;
};

struct xccl_context {
    xccl_lib                                     *lib = nullptr;
    xccl_context_params_t                         params{};
    std::vector<std::unique_ptr<xccl::TlContext>> tl_ctxs;
    std::unique_ptr<xccl::ProgressQueue>          pq;
};

struct xccl_team {
    xccl_context                              *ctx = nullptr;
    xccl_team_params_t                         params{};
    std::vector<int>                           range_map;  // owned copy of a MAP range
    std::vector<std::unique_ptr<xccl::TlTeam>> tl_teams;   // index = position in ctx->tl_ctxs at first, sorted by priority once created
    size_t                                     n_posted = 0;
    bool                                       created  = false;
    xccl_status_t                              failed   = XCCL_OK;
    double                                     t_posted = 0.0;  // steady-clock seconds of xccl_team_create_post
    int coll_team_id[XCCL_COLL_LAST][XCCL_MEMORY_TYPE_LAST];
};
