// Interface every team library (TL) implements, and the registry the core picks TLs from.
//
// The reference describes a TL as a C struct of function pointers loaded with dlopen
// (src/core/xccl_team_lib.h:42-97, src/core/xccl_init.c:59-124). Here a TL is a C++ object
// with four small classes - TeamLib, TlContext, TlTeam, xccl_coll_req - registered at static
// initialisation time; XCCL_TEAM_LIB_PATH may still name a directory of extra plugins, each
// exporting `xccl::TeamLib *xccl_team_lib_create(void)`.
#pragma once
#include <memory>
#include <string>
#include <vector>

#include "config.h"
#include "log.h"
#include "xccl/xccl.h"

struct xccl_lib;
struct xccl_context;
struct xccl_team;

// The public request handle IS the TL's request object.
namespace xccl {
class TlTeam;
}

struct xccl_coll_req {
    virtual ~xccl_coll_req() = default;
    virtual xccl_status_t post()     = 0;
    virtual xccl_status_t test()     = 0;
    virtual xccl_status_t wait();                      // default: spin on test + context progress
    virtual xccl_status_t finalize() { return XCCL_OK; }  // refuse (INPROGRESS / error) when in flight
    virtual double        elapsed_us() { return -1.0; }
    xccl_team *core_team = nullptr;
    int        coll_type = -1;   // xccl_collective_type_t, set by xccl_collective_init (tracing)
    xccl::TlTeam *tl_team = nullptr;  // the team-library team that serves the request (poisoned when a wait runs out)
};

struct xccl_mem_handle {
    virtual ~xccl_mem_handle() = default;
    virtual xccl_status_t test() = 0;
    virtual xccl_status_t unmap() { return XCCL_OK; }
};

namespace xccl {

class TeamLib;
class TlContext;

class TlTeam {
public:
    virtual ~TlTeam() = default;
    virtual xccl_status_t create_test() = 0;
    virtual xccl_status_t collective_init(const xccl_coll_op_args_t &args, xccl_memory_type_t mem,
                                          xccl_coll_req **req) = 0;
    virtual xccl_status_t mem_map_start(const xccl_mem_map_params_t &, xccl_mem_handle **) { return XCCL_ERR_NOT_IMPLEMENTED; }
    // symmetric device memory (xccl_team_mem_alloc / xccl_team_mem_free), collective over the team
    virtual xccl_status_t sym_alloc(size_t, void **) { return XCCL_ERR_NOT_IMPLEMENTED; }
    virtual xccl_status_t sym_free(void *) { return XCCL_ERR_NOT_IMPLEMENTED; }
    // false until the TL team can no longer make progress after an error (bounded wait expired)
    bool       poisoned = false;
    TlContext *ctx      = nullptr;
    int        rank = 0, size = 1;
};

class TlContext {
public:
    virtual ~TlContext() = default;
    virtual xccl_status_t progress() { return XCCL_OK; }
    virtual bool          has_progress() const { return false; }
    // Starts creating a team; may already finish, create_test() tells.
    virtual xccl_status_t team_create_post(const xccl_team_params_t &params, TlTeam **team) = 0;
    TeamLib      *tl   = nullptr;
    xccl_context *core = nullptr;
};

struct TlCaps {
    uint64_t                   coll_types   = 0;
    uint64_t                   mem_types    = 0;  // bit per xccl_memory_type_t
    // barrier / fanin / fanout carry no buffer and are dispatched as host memory; a device TL that
    // wants to serve them (as stream-ordered kernels) sets the host bit here only
    uint64_t                   sync_mem_types = ~0ull;  // ~0 = same as mem_types
    unsigned                   reproducible = XCCL_REPRODUCIBILITY_MODE_NON_REPRODUCIBLE;
    unsigned                   thread_mode  = XCCL_THREAD_MODE_SINGLE | XCCL_THREAD_MODE_MULTIPLE;
    uint64_t                   team_usage   = XCCL_LIB_PARAMS_TEAM_USAGE_SW_COLLECTIVES;
    xccl_context_create_mode_t ctx_mode     = XCCL_TEAM_LIB_CONTEXT_CREATE_MODE_LOCAL;
    // true: the TL applies xccl_coll_epilogue_t (scale, output cast) itself, fused into its last pass.
    // false: the core strips the epilogue from the arguments the TL sees and applies it as a local last
    // step when the TL's collective has completed (csrc/core/collective.cc, EpilogueReq).
    bool                       epilogue     = false;
};

class TeamLib {
public:
    TeamLib(xccl_tl_id_t id, int default_priority);
    virtual ~TeamLib() = default;

    // options every TL has: LOG_LEVEL and PRIORITY (reference: src/core/xccl_team_lib.c:3-24)
    virtual std::vector<OptField> lib_options() const { return {}; }
    virtual std::vector<OptField> context_options() const { return {}; }
    virtual xccl_status_t open() { return XCCL_OK; }   // after lib options are read
    virtual void          close() {}
    virtual xccl_status_t query(xccl_tl_attr_t *attr);
    virtual xccl_status_t context_create(xccl_lib *lib, const xccl_context_params_t &params,
                                         const OptTable &cfg, TlContext **ctx) = 0;

    std::string upper_name() const;
    std::string scope() const { return "TEAM_" + upper_name() + "_"; }

    xccl_tl_id_t id;
    const char  *name;
    int          priority;
    TlCaps       caps;
    LogComponent log;
    OptTable     lib_cfg;
    bool         opened = false;
};

// Registry: filled by static registrars in each TL's translation unit.
std::vector<TeamLib *> &team_lib_registry();
void                    register_team_lib(TeamLib *tl);
TeamLib                *find_team_lib(xccl_tl_id_t id);
void                    open_all_team_libs();  // idempotent; reads lib options, calls open()

struct TeamLibRegistrar {
    explicit TeamLibRegistrar(TeamLib *tl) { register_team_lib(tl); }
};

// The group a team bootstraps over: either the team's own OOB (whole coll_context) or the
// context's OOB restricted by the team's endpoint range.
struct OobGroup {
    xccl_oob_collectives_t oob{};
    xccl_ep_range_t        range{};   // passed to oob.allgather; UNDEFINED = whole coll_context
    int                    rank = 0, size = 1;

    int allgather(void *sbuf, void *rbuf, size_t bytes, void **req) const
    {
        return oob.allgather(sbuf, rbuf, bytes, rank, range, oob.coll_context, req);
    }
    xccl_status_t test(void *req) const { return oob.req_test(req); }
    void          free(void *req) const { oob.req_free(req); }
    // context rank of team member i (identity when the team brought its own OOB)
    int ctx_rank(int i) const { return range.type == XCCL_EP_RANGE_UNDEFINED ? i : xccl_range_to_rank(range, i); }
    xccl_status_t allgather_blocking(void *sbuf, void *rbuf, size_t bytes) const;
};
OobGroup make_oob_group(const xccl_team_params_t &team_params, const xccl_oob_collectives_t &ctx_oob);

// Blocking helper over the non-blocking OOB contract, with a deadline
// (XCCL_OOB_TIMEOUT seconds, default 120): returns XCCL_ERR_TIMED_OUT instead of spinning
// forever when a member never joins.
xccl_status_t oob_allgather_blocking(const xccl_oob_collectives_t &oob, void *sbuf, void *rbuf, size_t size);

}  // namespace xccl

#define tl_error(tl, ...) XCCL_LOG_AT((tl)->log, ::xccl::LOG_ERROR, __VA_ARGS__)
#define tl_warn(tl, ...)  XCCL_LOG_AT((tl)->log, ::xccl::LOG_WARN, __VA_ARGS__)
#define tl_info(tl, ...)  XCCL_LOG_AT((tl)->log, ::xccl::LOG_INFO, __VA_ARGS__)
#define tl_debug(tl, ...) XCCL_LOG_AT((tl)->log, ::xccl::LOG_DEBUG, __VA_ARGS__)
#define tl_trace(tl, ...) XCCL_LOG_AT((tl)->log, ::xccl::LOG_TRACE, __VA_ARGS__)
