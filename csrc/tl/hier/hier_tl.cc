// Hierarchy team library: context (one sub-context per building-block team library), team
// (sub-groups and pairs) and the schedule-driven request. Reference: src/team_lib/hier/
// xccl_hier_context.c:15-217, xccl_hier_team.c:17-159, xccl_hier_lib.c:151-313,
// xccl_hier_schedule.c:329-358.
#include "hier_tl.h"

#include <algorithm>
#include <chrono>
#include <cstdlib>
#include <cstring>

#include "../../utils/topo.h"

namespace xccl {
namespace hier {

// ------------------------------------------------------------------ context

HierContext::~HierContext()
{
    for (auto &kv : subctx) xccl_context_destroy(kv.second);
    if (lib != nullptr) xccl_lib_cleanup(lib);
}

xccl_status_t HierContext::init()
{
    if (!(params.field_mask & XCCL_CONTEXT_PARAM_FIELD_OOB)) return XCCL_ERR_INVALID_PARAM;
    xccl_lib_params_t lp{};
    lp.field_mask = XCCL_LIB_PARAM_FIELD_THREAD_MODE;
    lp.thread_mode = params.thread_mode;
    xccl_status_t st = xccl_lib_init(&lp, nullptr, &lib);
    if (st != XCCL_OK) return st;
    // composite team libraries are never nested below hier
    std::vector<xccl_tl_id_t> want = {XCCL_TL_UCX};
    if (cfg.enable_nvlink) want.push_back(XCCL_TL_NVLINK);
    if (cfg.enable_nccl) want.push_back(XCCL_TL_NCCL);
    if (cfg.enable_sharp) want.push_back(XCCL_TL_SHARP);
    if (cfg.enable_hmc) want.push_back(XCCL_TL_HMC);
    if (cfg.enable_shmseg) want.push_back(XCCL_TL_SHMSEG);
    // optional levels whose team library did not open here (no CUDA device, no NCCL) are left out quietly
    for (xccl_tl_id_t id : want) {
        if (id != XCCL_TL_UCX && !lib->has(id)) continue;
        xccl_context_params_t cp = params;
        cp.field_mask |= XCCL_CONTEXT_PARAM_FIELD_TLS;
        cp.tls = (uint64_t)id;
        // options of a level: HIER_<tl>_XCCL_TEAM_<TL>_<NAME>, so each level can be tuned on its own
        std::string            prefix = std::string("HIER_") + xccl_tl_str(id);
        xccl_context_config_t *cc     = nullptr;
        if (xccl_context_config_read(lib, prefix.c_str(), nullptr, &cc) != XCCL_OK) continue;
        xccl_context_h c  = nullptr;
        xccl_status_t  cs = xccl_context_create(lib, &cp, cc, &c);
        xccl_context_config_release(cc);
        if (cs == XCCL_OK) {
            subctx[id] = c;
        } else if (id == XCCL_TL_UCX) {
            return cs;  // the host team is the one level hier cannot do without
        }
    }
    // placement of every context rank
    ProcInfo    mine{};
    const char *fake = std::getenv("XCCL_HIER_FAKE_NODE_ID");  // lets one host stand in for several nodes in tests
    mine.node_hash   = fake != nullptr ? (uint64_t)std::strtoull(fake, nullptr, 10) + 1 : global_state().host_hash;
    mine.socket_id   = global_state().socket_id;
    mine.pid         = global_state().pid;
    procs.resize((size_t)params.oob.size);
    return oob_allgather_blocking(params.oob, &mine, procs.data(), sizeof(ProcInfo));
}

xccl_status_t HierContext::progress()
{
    for (auto &kv : subctx) {
        xccl_status_t st = xccl_context_progress(kv.second);
        if (st < 0) return st;
    }
    return XCCL_OK;
}

xccl_status_t HierContext::team_create_post(const xccl_team_params_t &tp, TlTeam **team)
{
    OobGroup g = make_oob_group(tp, params.oob);
    if (g.rank < 0 || g.size < 1) return XCCL_ERR_INVALID_PARAM;
    if (tp.field_mask & XCCL_TEAM_PARAM_FIELD_OOB) {
        // placement is known per CONTEXT rank; a team that brings its own OOB must say which
        // context ranks it is made of through its endpoint range
        if (!(tp.field_mask & XCCL_TEAM_PARAM_FIELD_EP_RANGE) || tp.range.type == XCCL_EP_RANGE_UNDEFINED) {
            if (g.size != params.oob.size) return XCCL_ERR_UNSUPPORTED;
        }
    }
    auto *t = new HierTeam(this, g);
    if ((tp.field_mask & XCCL_TEAM_PARAM_FIELD_OOB) && (tp.field_mask & XCCL_TEAM_PARAM_FIELD_EP_RANGE) &&
        tp.range.type != XCCL_EP_RANGE_UNDEFINED && tp.range.type != XCCL_EP_RANGE_FULL) {
        t->place_range = tp.range;
    }
    xccl_status_t st = t->init();
    if (st != XCCL_OK) {
        delete t;
        return st;
    }
    *team = t;
    return XCCL_OK;
}

// ------------------------------------------------------------------ team

HierTeam::HierTeam(HierContext *c, const OobGroup &g) : hctx(c), oob(g)
{
    rank = g.rank;
    size = g.size;
}

HierTeam::~HierTeam()
{
    for (auto &p : pairs) {
        if (p.team != nullptr) xccl_team_destroy(p.team);
        if (p.have_oob) xccl_oob_sub_destroy(&p.oob);
    }
    if (team_oob_.coll_context != nullptr) xccl_oob_sub_destroy(&team_oob_);
}

xccl_status_t HierTeam::create_pair(PairId id, SbgpType st, xccl_tl_id_t tl)
{
    const Sbgp    &sb  = layout.sbgp[st];
    xccl_context_h ctx = hctx->sub(tl);
    if (sb.status != SBGP_ENABLED || ctx == nullptr) return XCCL_OK;  // not a member, or level not enabled
    Pair &p  = pairs[id];
    p.sbgp   = &sb;
    p.ctx    = ctx;
    xccl_status_t s = xccl_oob_sub_create(&team_oob_, sb.ranks.data(), (int)sb.ranks.size(), &p.oob);
    if (s != XCCL_OK) return s;
    p.have_oob = true;
    xccl_team_params_t tp{};
    tp.field_mask   = XCCL_TEAM_PARAM_FIELD_OOB | XCCL_TEAM_PARAM_FIELD_EP_RANGE;
    tp.oob          = p.oob;
    tp.range.type   = XCCL_EP_RANGE_FULL;
    tp.range.ep_num = (int)sb.ranks.size();
    s = xccl_team_create_post(ctx, &tp, &p.team);
    if (s != XCCL_OK) {
        p.team = nullptr;
        return (tl == XCCL_TL_UCX) ? s : XCCL_OK;
    }
    double limit = global_state().opts.real("OOB_TIMEOUT");
    auto   t0    = std::chrono::steady_clock::now();
    while ((s = xccl_team_create_test(p.team)) == XCCL_INPROGRESS) {
        xccl_context_progress(ctx);
        double dt = std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
        if (limit > 0 && dt > limit) {
            s = XCCL_ERR_TIMED_OUT;
            break;
        }
    }
    if (s != XCCL_OK) {
        xccl_team_destroy(p.team);
        p.team = nullptr;
        // an optional level that cannot come up (e.g. nvlink without peer access) is simply absent
        return (tl == XCCL_TL_UCX) ? s : XCCL_OK;
    }
    return XCCL_OK;
}

xccl_status_t HierTeam::init()
{
    // the team's own group as an OOB object, so that sub-groups can be cut out of it
    std::vector<int> ctx_ranks((size_t)size);
    for (int i = 0; i < size; i++) ctx_ranks[(size_t)i] = oob.ctx_rank(i);
    xccl_status_t st = xccl_oob_sub_create(&oob.oob, ctx_ranks.data(), size, &team_oob_);
    if (st != XCCL_OK) return st;
    procs.resize((size_t)size);
    for (int i = 0; i < size; i++) {
        int cr = place_range.type != XCCL_EP_RANGE_UNDEFINED ? xccl_range_to_rank(place_range, i) : ctx_ranks[(size_t)i];
        if (cr < 0 || cr >= (int)hctx->procs.size()) return XCCL_ERR_INVALID_PARAM;
        procs[(size_t)i] = hctx->procs[(size_t)cr];
    }
    layout = compute_layout(procs, rank, hctx->cfg.node_leader_rank_id);

    // Creation order is the same on every rank; members of a sub-group create its team together.
    struct Plan {
        PairId       id;
        SbgpType     sbgp;
        xccl_tl_id_t tl;
    };
    const xccl_tl_id_t device_tl = hctx->sub(XCCL_TL_NVLINK) != nullptr ? XCCL_TL_NVLINK : XCCL_TL_NCCL;
    const Plan         plan[]    = {
        {PAIR_NODE_HOST, SBGP_NODE, XCCL_TL_UCX},
        {PAIR_NODE_DEVICE, SBGP_NODE, device_tl},
        {PAIR_SOCKET_HOST, SBGP_SOCKET, XCCL_TL_UCX},
        {PAIR_SOCKET_LEADERS_HOST, SBGP_SOCKET_LEADERS, XCCL_TL_UCX},
        {PAIR_NODE_LEADERS_HOST, SBGP_NODE_LEADERS, XCCL_TL_UCX},
        {PAIR_NODE_LEADERS_SHARP, SBGP_NODE_LEADERS, XCCL_TL_SHARP},
        {PAIR_FLAT_HOST, SBGP_FLAT, XCCL_TL_UCX},
        {PAIR_NODE_SHMSEG, SBGP_NODE, XCCL_TL_SHMSEG},
        {PAIR_SOCKET_SHMSEG, SBGP_SOCKET, XCCL_TL_SHMSEG},
        {PAIR_SOCKET_LEADERS_SHMSEG, SBGP_SOCKET_LEADERS, XCCL_TL_SHMSEG},
    };
    for (const Plan &pl : plan) {
        st = create_pair(pl.id, pl.sbgp, pl.tl);
        if (st != XCCL_OK) return st;
    }
    tl_debug(hctx->tl, "hier team: rank %d/%d, %d node(s), node leader %d, sockets %s", rank, size, layout.n_nodes,
             layout.node_leader, layout.sockets_usable ? "used" : "not used");
    return XCCL_OK;
}

// ------------------------------------------------------------------ request

namespace {

// A step of the schedule as a task: its start handler inits and posts the collective on the
// pair's team and enqueues itself; its progress function polls the request and completes.
class StepTask final : public Task {
public:
    Step            step;
    HierTeam       *team = nullptr;
    xccl_coll_req_h req  = nullptr;

    // Requests are created when the schedule is built, in schedule order: members of a pair's
    // team then initialise their requests in the same order, which is what the host team's
    // per-team sequence tags rely on even when several fragments are in flight.
    xccl_status_t init()
    {
        const Pair &p = team->pairs[step.pair];
        if (p.team == nullptr) return XCCL_ERR_NO_RESOURCE;
        return xccl_collective_init(&step.args, &req, p.team);
    }
    xccl_status_t launch() { return req != nullptr ? xccl_collective_post(req) : XCCL_ERR_NO_RESOURCE; }
    ~StepTask() override
    {
        if (req != nullptr) xccl_collective_finalize(req);
    }
};

class HierReq final : public xccl_coll_req {
public:
    HierReq(HierTeam *t) : team_(t) {}
    ~HierReq() override
    {
        tasks_.clear();  // the FANOUT_GET requests go before the regions they read
        for (xccl_mem_h m : sm_.memh) {
            if (m != nullptr) xccl_global_mem_unmap(m);
        }
    }

    // Host broadcasts with BCAST_SM_GET: the node-local levels read the level root's buffer through a region of the
    // shared-segment team (FANOUT_GET). The regions are mapped here, once per request, by all members of each group.
    xccl_status_t map_regions(const xccl_coll_op_args_t &args, xccl_memory_type_t mem)
    {
        const HierCfg &cfg = team_->hctx->cfg;
        const size_t   len = args.buffer_info.len;
        if (args.coll_type != XCCL_BCAST || mem != XCCL_MEMORY_TYPE_HOST || !cfg.bcast_sm_get || len == 0 ||
            len < cfg.bcast_sm_get_thresh || args.root < 0 || args.root >= team_->size) {
            return XCCL_OK;
        }
        const double limit = global_state().opts.real("OOB_TIMEOUT");
        for (const BcastLevel &lv : bcast_local_levels(*team_, args.root)) {
            const Pair &p = team_->pairs[shmseg_pair(lv.sbgp)];
            if (p.team == nullptr || !team_->pair_ok(host_pair(lv.sbgp))) continue;
            const void *src = args.buffer_info.src_buffer;
            const bool  own = team_->rank == args.root && src != nullptr && src != XCCL_IN_PLACE;
            xccl_mem_map_params_t mp{};
            mp.field_mask = XCCL_MEM_MAP_PARAM_FIELD_ADDRESS | XCCL_MEM_MAP_PARAM_FIELD_LENGTH | XCCL_MEM_MAP_PARAM_FIELD_ROOT;
            mp.address    = own ? const_cast<void *>(src) : args.buffer_info.dst_buffer;
            mp.length     = len;
            mp.root       = lv.root;
            xccl_status_t st = xccl_global_mem_map_start(p.team, mp, &sm_.memh[lv.sbgp]);
            if (st != XCCL_OK) return st;
            auto t0 = std::chrono::steady_clock::now();
            while ((st = xccl_global_mem_map_test(sm_.memh[lv.sbgp])) == XCCL_INPROGRESS) {
                xccl_context_progress(p.ctx);
                if (limit > 0 && std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count() > limit) {
                    return XCCL_ERR_TIMED_OUT;
                }
            }
            if (st != XCCL_OK) return st;
            use_sm_ = true;
        }
        return XCCL_OK;
    }

    // Large broadcasts are cut into fragments of BCAST_PIPELINE_THRESH bytes; each fragment is a
    // complete schedule of its own and BCAST_PIPELINE_DEPTH of them are in flight at a time
    // (reference: fragmentation machinery of src/team_lib/hier/xccl_hier_schedule.c:197-326).
    xccl_status_t build(const xccl_coll_op_args_t &args, xccl_memory_type_t mem)
    {
        const HierCfg &cfg   = team_->hctx->cfg;
        xccl_status_t  mst   = map_regions(args, mem);
        if (mst != XCCL_OK) return mst;
        size_t         nfrag = 1, frag_bytes = args.buffer_info.len;
        if (args.coll_type == XCCL_BCAST && cfg.bcast_pipeline_thresh > 0 &&
            args.buffer_info.len > cfg.bcast_pipeline_thresh) {
            frag_bytes = cfg.bcast_pipeline_thresh;
            nfrag      = (args.buffer_info.len + frag_bytes - 1) / frag_bytes;
        }
        const size_t depth = (size_t)std::max(1, cfg.bcast_pipeline_depth);
        frags_.reserve(nfrag);
        for (size_t f = 0; f < nfrag; f++) {
            xccl_coll_op_args_t a = args;
            if (nfrag > 1) {
                size_t off = f * frag_bytes;
                a.buffer_info.len = std::min(frag_bytes, args.buffer_info.len - off);
                if (a.buffer_info.src_buffer != XCCL_IN_PLACE && a.buffer_info.src_buffer != nullptr) {
                    a.buffer_info.src_buffer = (char *)args.buffer_info.src_buffer + off;
                }
                a.buffer_info.dst_buffer = (char *)args.buffer_info.dst_buffer + off;
            }
            auto frag = std::make_unique<Schedule>();
            sm_.offset = nfrag > 1 ? f * frag_bytes : 0;
            xccl_status_t st = build_fragment(a, mem, frag.get());
            if (st != XCCL_OK) return st;
            auto kick = [](Task *self, Task *) { static_cast<Schedule *>(self)->start(); };
            frag->set_handler(EVENT_SCHEDULE_STARTED, kick);
            frag->set_handler(EVENT_COMPLETED, kick);
            sched_.add(frag.get());
            if (f < depth) {
                sched_.subscribe(EVENT_SCHEDULE_STARTED, frag.get());
            } else {
                frags_[f - depth]->subscribe(EVENT_COMPLETED, frag.get());
            }
            frags_.push_back(std::move(frag));
        }
        return XCCL_OK;
    }

    xccl_status_t build_fragment(const xccl_coll_op_args_t &args, xccl_memory_type_t mem, Schedule *frag)
    {
        std::vector<Step> steps;
        xccl_status_t     st;
        int               first_dep = -1;
        bool              parallel  = false;
        switch (args.coll_type) {
        case XCCL_ALLREDUCE: st = build_allreduce(*team_, args, mem, &steps); break;
        case XCCL_BARRIER: st = build_barrier(*team_, args, &steps); break;
        case XCCL_BCAST: st = build_bcast(*team_, args, mem, &steps, &first_dep, use_sm_ ? &sm_ : nullptr); break;
        case XCCL_ALLTOALL: st = build_alltoall(*team_, args, mem, &steps, &parallel, &keep_); break;
        default: return XCCL_ERR_UNSUPPORTED;
        }
        if (st != XCCL_OK) return st;
        const size_t base = tasks_.size();
        for (size_t i = 0; i < steps.size(); i++) {
            auto t  = std::make_unique<StepTask>();
            t->step = steps[i];
            t->team = team_;
            t->progress = [](Task *self) -> xccl_status_t {
                auto *s = static_cast<StepTask *>(self);
                for (int k = 0; k < 10; k++) {
                    xccl_status_t st = xccl_collective_test(s->req);
                    if (st == XCCL_INPROGRESS) continue;
                    s->complete(st);
                    return st;
                }
                return XCCL_OK;
            };
            auto start = [this](Task *self, Task *) {
                auto         *s  = static_cast<StepTask *>(self);
                xccl_status_t st = s->launch();
                if (st != XCCL_OK) {
                    s->complete(st);
                    return;
                }
                team_->hctx->core->pq->enqueue(s);
            };
            t->set_handler(EVENT_SCHEDULE_STARTED, start);
            t->set_handler(EVENT_COMPLETED, start);
            st = t->init();
            if (st != XCCL_OK) return st;
            tasks_.push_back(std::move(t));
        }
        // dependencies: a chain by default; all-at-once for independent steps; for a broadcast
        // the one level where this rank RECEIVES gates the levels where it sends
        for (size_t i = 0; i < steps.size(); i++) {
            Task *cur = tasks_[base + i].get();
            frag->add(cur);
            if (steps[i].after != Step::kDepDefault) {
                if (steps[i].after == Step::kDepNone) {
                    frag->subscribe(EVENT_SCHEDULE_STARTED, cur);
                } else {
                    tasks_[base + (size_t)steps[i].after]->subscribe(EVENT_COMPLETED, cur);
                }
            } else if (parallel) {
                frag->subscribe(EVENT_SCHEDULE_STARTED, cur);
            } else if (first_dep >= 0) {
                if ((int)i == first_dep) {
                    frag->subscribe(EVENT_SCHEDULE_STARTED, cur);
                } else {
                    tasks_[base + (size_t)first_dep]->subscribe(EVENT_COMPLETED, cur);
                }
            } else if (i == 0) {
                frag->subscribe(EVENT_SCHEDULE_STARTED, cur);
            } else {
                tasks_[base + i - 1]->subscribe(EVENT_COMPLETED, cur);
            }
        }
        return XCCL_OK;
    }

    xccl_status_t post() override
    {
        if (sched_.state.load() == TASK_INPROGRESS) return XCCL_ERR_NO_RESOURCE;
        sched_.rearm();
        sched_.start();
        return XCCL_OK;
    }

    xccl_status_t test() override
    {
        int s = sched_.state.load(std::memory_order_acquire);
        if (s == TASK_INPROGRESS) {
            xccl_context_progress(team_->hctx->core);
            s = sched_.state.load(std::memory_order_acquire);
        }
        if (s == TASK_INPROGRESS) return XCCL_INPROGRESS;
        if (s == TASK_IDLE) return XCCL_OK;
        return sched_.status;
    }

    xccl_status_t finalize() override { return sched_.state.load() == TASK_INPROGRESS ? XCCL_INPROGRESS : XCCL_OK; }

private:
    HierTeam                              *team_;
    Schedule                               sched_;
    std::vector<std::unique_ptr<StepTask>> tasks_;
    std::vector<std::unique_ptr<Schedule>> frags_;
    std::vector<std::vector<uint32_t>>     keep_;  // count / displacement arrays of alltoallv steps
    SmGet                                  sm_;     // regions of a FANOUT_GET broadcast, by sub-group
    bool                                   use_sm_ = false;
};

}  // namespace

xccl_status_t HierTeam::collective_init(const xccl_coll_op_args_t &args, xccl_memory_type_t mem, xccl_coll_req **req)
{
    auto         *r  = new HierReq(this);
    xccl_status_t st = r->build(args, mem);
    if (st != XCCL_OK) {
        delete r;
        return st;
    }
    *req = r;
    return XCCL_OK;
}

// ------------------------------------------------------------------ lib

namespace {

class HierLib final : public TeamLib {
public:
    HierLib() : TeamLib(XCCL_TL_HIER, 150)
    {
        caps.coll_types = XCCL_COLL_CAP_BARRIER | XCCL_COLL_CAP_BCAST | XCCL_COLL_CAP_ALLREDUCE | XCCL_COLL_CAP_ALLTOALL;
        caps.mem_types  = XCCL_BIT(XCCL_MEMORY_TYPE_HOST) | XCCL_BIT(XCCL_MEMORY_TYPE_CUDA);
    }
    std::vector<OptField> context_options() const override
    {
        return {
            {"NET_DEVICES", "all", "Accepted for compatibility", OptType::STRING},
            {"ENABLE_SHARP", "no", "Use the in-fabric reduction team among node leaders", OptType::BOOL},
            {"ENABLE_SHMSEG", "no", "Use the shared-segment team inside a node", OptType::BOOL},
            {"ENABLE_HMC", "no", "Use the hardware-multicast broadcast team", OptType::BOOL},
            {"ENABLE_NCCL", "no", "Use the NCCL team for CUDA buffers inside a node", OptType::BOOL},
            {"ENABLE_NVLINK", "yes", "Use the NVLink team for CUDA buffers inside a node", OptType::BOOL},
            {"BCAST_PIPELINE_THRESH", "inf", "Broadcasts above this size are cut into fragments", OptType::MEMUNITS},
            {"BCAST_PIPELINE_DEPTH", "1", "Fragments in flight", OptType::UINT},
            {"BCAST_SM_GET", "0", "Host broadcasts inside a node read the level root's buffer through FANOUT_GET on the shared-segment team (needs ENABLE_SHMSEG)", OptType::BOOL},
            {"BCAST_SM_GET_THRESH", "0", "Smallest broadcast that takes the FANOUT_GET path", OptType::MEMUNITS},
            {"NODE_LEADER_RANK_ID", "0", "Local index of the rank that leads its node", OptType::UINT},
        };
    }
    xccl_status_t context_create(xccl_lib *, const xccl_context_params_t &params, const OptTable &cfg,
                                 TlContext **ctx) override
    {
        HierCfg c;
        c.enable_sharp          = cfg.flag("ENABLE_SHARP");
        c.enable_shmseg         = cfg.flag("ENABLE_SHMSEG");
        c.enable_hmc            = cfg.flag("ENABLE_HMC");
        c.enable_nccl           = cfg.flag("ENABLE_NCCL");
        c.enable_nvlink         = cfg.flag("ENABLE_NVLINK");
        c.bcast_pipeline_thresh = (size_t)cfg.num("BCAST_PIPELINE_THRESH");
        c.bcast_pipeline_depth  = (int)cfg.num("BCAST_PIPELINE_DEPTH");
        c.node_leader_rank_id   = (int)cfg.num("NODE_LEADER_RANK_ID");
        c.bcast_sm_get          = cfg.flag("BCAST_SM_GET") && c.enable_shmseg;
        c.bcast_sm_get_thresh   = (size_t)cfg.num("BCAST_SM_GET_THRESH");
        auto         *h  = new HierContext(params, c);
        h->tl            = this;
        xccl_status_t st = h->init();
        if (st != XCCL_OK) {
            delete h;
            return st;
        }
        *ctx = h;
        return XCCL_OK;
    }
};

HierLib          g_hier_lib;
TeamLibRegistrar g_hier_reg(&g_hier_lib);

}  // namespace

}  // namespace hier
}  // namespace xccl
