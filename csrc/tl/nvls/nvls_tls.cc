// In-fabric offload team libraries for an NVSwitch box.
//
// The reference has two hardware-offload teams built on InfiniBand libraries that do not exist
// on this platform: "sharp" (switch-side reduction: allreduce + barrier,
// src/team_lib/sharp/xccl_sharp_lib.c:387-391) and "hmc" (hardware multicast: bcast only,
// src/team_lib/hmc/xccl_hmc_lib.c:132-212). Their NVSwitch counterparts are the multimem
// instructions: multimem.ld_reduce lets the switch add the ranks' buffers, multimem.st lets it
// replicate a store. Both team libraries keep the reference's ids, capabilities and option names
// and run on an inner NVLink team with the in-switch algorithms forced.
//
// The sharp team's two data paths (src/team_lib/sharp/xccl_sharp_collective.c:61-170) map as follows:
//   zero-copy   the reference registers the user's buffers with the SHARP library and lets the switch work on
//               them in place for messages of ZCOPY_THRESH bytes or more. Here the registered memory is what
//               xccl_team_mem_alloc hands out (symmetric, bound to the multicast object): from ZCOPY_THRESH on,
//               multimem.ld_reduce reads the source buffers and multimem.st writes the destinations directly.
//   bounce copy smaller messages, and buffers that are not registered memory, are staged through the team's
//               pre-registered bounce buffers: BCOPY_BUF_NUM buffers of BCOPY_BUF_SIZE bytes form the inner
//               team's workspace, which is bound to the multicast object at team creation.
//   RCACHE      the registration cache for ordinary device buffers: CUDA IPC mappings of the peers' allocations,
//               kept per allocation ("no" never registers; requests then always take the bounce path).
//   NET_DEVICES the fabric to use; only "nvswitch" exists on this platform, anything else fails context creation.
#include <algorithm>
#include <chrono>
#include <string>
#include <utility>
#include <vector>

#include "../../core/core.h"
#include "../../cuda/cuda_common.h"

namespace xccl {
namespace nvls {

namespace {

class FwdContext;

class FwdTeam final : public TlTeam {
public:
    FwdTeam(FwdContext *c) : fctx(c) {}
    ~FwdTeam() override
    {
        if (inner != nullptr) xccl_team_destroy(inner);
    }
    xccl_status_t create_test() override { return XCCL_OK; }
    xccl_status_t collective_init(const xccl_coll_op_args_t &args, xccl_memory_type_t, xccl_coll_req **req) override;
    // registered memory of this team: symmetric allocations of the inner NVLink team
    xccl_status_t sym_alloc(size_t bytes, void **ptr) override { return xccl_team_mem_alloc(inner, bytes, ptr); }
    xccl_status_t sym_free(void *ptr) override { return xccl_team_mem_free(inner, ptr); }
    FwdContext *fctx;
    xccl_team_h inner = nullptr;
};

// The inner request IS the request handed to the caller: nothing to add on the data path.
class FwdContext final : public TlContext {
public:
    FwdContext(const xccl_context_params_t &p, uint64_t colls) : params(p), colls_(colls) {}
    ~FwdContext() override
    {
        if (inner != nullptr) xccl_context_destroy(inner);
        if (lib != nullptr) xccl_lib_cleanup(lib);
    }
    // extra (name, value) pairs for the inner NVLink context
    std::vector<std::pair<std::string, std::string>> inner_opts;
    xccl_status_t init(const char *prefix)
    {
        xccl_lib_params_t lp{};
        xccl_status_t     st = xccl_lib_init(&lp, nullptr, &lib);
        if (st != XCCL_OK) return st;
        xccl_context_params_t cp = params;
        cp.field_mask |= XCCL_CONTEXT_PARAM_FIELD_TLS;
        cp.tls                    = XCCL_TL_NVLINK;
        xccl_context_config_t *cc = nullptr;
        st                        = xccl_context_config_read(lib, prefix, nullptr, &cc);
        if (st != XCCL_OK) return st;
        xccl_tl_id_t id = XCCL_TL_NVLINK;
        xccl_context_config_modify(&id, cc, "NVLS", "yes");
        for (auto &kv : inner_opts) xccl_context_config_modify(&id, cc, kv.first.c_str(), kv.second.c_str());
        st = xccl_context_create(lib, &cp, cc, &inner);
        xccl_context_config_release(cc);
        return st;
    }
    xccl_status_t team_create_post(const xccl_team_params_t &tp, TlTeam **team) override
    {
        auto               t = std::make_unique<FwdTeam>(this);
        xccl_team_params_t p = tp;
        xccl_status_t      s = xccl_team_create_post(inner, &p, &t->inner);
        if (s != XCCL_OK) return s;
        double limit = global_state().opts.real("OOB_TIMEOUT");
        auto   t0    = std::chrono::steady_clock::now();
        while ((s = xccl_team_create_test(t->inner)) == XCCL_INPROGRESS) {
            if (limit > 0 && std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count() > limit) {
                return XCCL_ERR_TIMED_OUT;
            }
        }
        if (s != XCCL_OK) return s;
        // Probe: an NVLS request must be accepted, otherwise the fabric offload is not there.
        OobGroup g = make_oob_group(tp, params.oob);
        t->rank    = g.rank;
        t->size    = g.size;
        *team      = t.release();
        return XCCL_OK;
    }
    xccl_context_params_t params;
    xccl_lib_h            lib   = nullptr;
    xccl_context_h        inner = nullptr;
    uint64_t              colls_;
};

xccl_status_t FwdTeam::collective_init(const xccl_coll_op_args_t &args, xccl_memory_type_t, xccl_coll_req **req)
{
    xccl_coll_op_args_t a = args;
    if (a.coll_type == XCCL_ALLREDUCE || a.coll_type == XCCL_BCAST) {
        a.alg.set_by_user = 1;
        a.alg.id          = XCCL_NVLINK_ALG_NVLS;
    }
    xccl_coll_req_h r  = nullptr;
    xccl_status_t   st = xccl_collective_init(&a, &r, inner);
    if (st != XCCL_OK) return st;
    *req = r;
    return XCCL_OK;
}

class SharpLib final : public TeamLib {
public:
    SharpLib() : TeamLib(XCCL_TL_SHARP, 90)
    {
        caps.coll_types     = XCCL_COLL_CAP_ALLREDUCE | XCCL_COLL_CAP_BARRIER;
        caps.mem_types      = XCCL_BIT(XCCL_MEMORY_TYPE_CUDA);
        caps.sync_mem_types = XCCL_BIT(XCCL_MEMORY_TYPE_HOST);
        caps.team_usage     = XCCL_LIB_PARAMS_TEAM_USAGE_HW_COLLECTIVES;
        caps.ctx_mode       = XCCL_TEAM_LIB_CONTEXT_CREATE_MODE_GLOBAL;
        caps.epilogue       = true;  // the arguments reach the NVLink team unchanged
    }
    xccl_status_t open() override { return cuda_available() ? XCCL_OK : XCCL_ERR_NO_RESOURCE; }
    std::vector<OptField> context_options() const override
    {
        return {
            {"RCACHE", "try", "Keep a cache of registrations (CUDA IPC mappings) of ordinary device buffers; no: never register", OptType::TERNARY},
            {"ZCOPY_THRESH", "1024", "Messages of at least this size in registered (xccl_team_mem_alloc) memory are reduced in place by the switch", OptType::MEMUNITS},
            {"BCOPY_BUF_NUM", "10", "Bounce buffers pre-registered with the fabric for the staged path", OptType::UINT},
            {"BCOPY_BUF_SIZE", "12800k", "Bytes of one bounce buffer", OptType::MEMUNITS},
            {"NET_DEVICES", "nvswitch", "Fabric to use; this platform has \"nvswitch\" only", OptType::STRING},
        };
    }
    xccl_status_t context_create(xccl_lib *, const xccl_context_params_t &params, const OptTable &cfg,
                                 TlContext **ctx) override
    {
        const std::string dev = cfg.str("NET_DEVICES");
        if (!dev.empty() && dev != "nvswitch" && dev != "all") {
            tl_error(this, "sharp: no fabric device \"%s\" (only \"nvswitch\")", dev.c_str());
            return XCCL_ERR_NO_RESOURCE;
        }
        auto c = std::make_unique<FwdContext>(params, caps.coll_types);
        const unsigned long long ws = std::max<unsigned long long>(
            (unsigned long long)cfg.num("BCOPY_BUF_NUM") * (unsigned long long)cfg.num("BCOPY_BUF_SIZE"), 1ull << 20);
        c->inner_opts.push_back({"WORKSPACE_SIZE", std::to_string(ws)});
        c->inner_opts.push_back({"SYMMETRIC_MIN", std::to_string((unsigned long long)cfg.num("ZCOPY_THRESH"))});
        const std::string rc = cfg.str("RCACHE");
        const bool        no_rcache = !rc.empty() && (rc[0] == 'n' || rc[0] == 'N' || rc[0] == '0' || rc == "off");
        c->inner_opts.push_back({"DIRECT", no_rcache ? "n" : "y"});
        xccl_status_t st = c->init("SHARP_nvlink");
        if (st != XCCL_OK) return st;
        *ctx = c.release();
        return XCCL_OK;
    }
};

class HmcLib final : public TeamLib {
public:
    HmcLib() : TeamLib(XCCL_TL_HMC, 100)
    {
        caps.coll_types = XCCL_COLL_CAP_BCAST;
        caps.mem_types  = XCCL_BIT(XCCL_MEMORY_TYPE_CUDA);
        caps.team_usage = XCCL_LIB_PARAMS_TEAM_USAGE_HW_COLLECTIVES;
    }
    xccl_status_t open() override { return cuda_available() ? XCCL_OK : XCCL_ERR_NO_RESOURCE; }
    xccl_status_t context_create(xccl_lib *, const xccl_context_params_t &params, const OptTable &,
                                 TlContext **ctx) override
    {
        auto          c  = std::make_unique<FwdContext>(params, caps.coll_types);
        xccl_status_t st = c->init("HMC_nvlink");
        if (st != XCCL_OK) return st;
        *ctx = c.release();
        return XCCL_OK;
    }
};

SharpLib         g_sharp_lib;
HmcLib           g_hmc_lib;
TeamLibRegistrar g_sharp_reg(&g_sharp_lib);
TeamLibRegistrar g_hmc_reg(&g_hmc_lib);

}  // namespace

}  // namespace nvls
}  // namespace xccl
