// Multirail team library: replicates another team library REPLICAS_NUMBER times and splits every
// buffer into that many byte ranges, one sub-collective per replica, so that several rails (or,
// on an NVSwitch box, several concurrently running kernels) carry one collective.
// Counterpart of the reference's mrail team (src/team_lib/multirail/xccl_mrail_lib.c): barrier,
// bcast and allreduce; optional progress threads that poll the replicas' requests and sleep on a
// condition variable when nothing is in flight.
#include <algorithm>
#include <atomic>
#include <chrono>
#include <condition_variable>
#include <cstring>
#include <mutex>
#include <thread>

#include "../../core/core.h"

namespace xccl {
namespace mrail {

namespace {

struct MrailCfg {
    std::string replicate = "hier";
    int         replicas  = 2;
    int         threads   = 0;
    int         poll      = 3;
};

class MrailContext;

struct SubReq {
    xccl_coll_req_h   req = nullptr;
    std::atomic<int>  state{0};  // 0 idle, 1 in flight, 2 done
    xccl_status_t     status = XCCL_OK;
};

// Progress threads: thread t owns the replicas r with r % n_threads == t.
class Workers {
public:
    Workers(int n, int poll) : poll_(std::max(poll, 1))
    {
        for (int i = 0; i < n; i++) threads_.emplace_back([this, i, n] { run(i, n); });
    }
    ~Workers()
    {
        {
            std::lock_guard<std::mutex> lock(mu_);
            stop_ = true;
        }
        cv_.notify_all();
        for (auto &t : threads_) t.join();
    }
    void submit(int replica, SubReq *s)
    {
        {
            std::lock_guard<std::mutex> lock(mu_);
            work_.push_back({replica, s});
        }
        cv_.notify_all();
    }
    int count() const { return (int)threads_.size(); }

private:
    struct Item {
        int     replica;
        SubReq *sub;
    };
    void run(int me, int n)
    {
        std::vector<Item> mine;
        for (;;) {
            {
                std::unique_lock<std::mutex> lock(mu_);
                if (mine.empty()) cv_.wait(lock, [&] { return stop_ || has_work_for(me, n); });
                if (stop_) return;
                for (size_t i = 0; i < work_.size();) {
                    if (work_[i].replica % n == me) {
                        mine.push_back(work_[i]);
                        work_.erase(work_.begin() + (long)i);
                    } else {
                        i++;
                    }
                }
            }
            for (size_t i = 0; i < mine.size();) {
                xccl_status_t st = XCCL_INPROGRESS;
                for (int k = 0; k < poll_ && st == XCCL_INPROGRESS; k++) st = xccl_collective_test(mine[i].sub->req);
                if (st != XCCL_INPROGRESS) {
                    mine[i].sub->status = st;
                    mine[i].sub->state.store(2, std::memory_order_release);
                    mine.erase(mine.begin() + (long)i);
                } else {
                    i++;
                }
            }
        }
    }
    bool has_work_for(int me, int n) const
    {
        for (auto &w : work_)
            if (w.replica % n == me) return true;
        return false;
    }
    std::vector<std::thread> threads_;
    std::mutex               mu_;
    std::condition_variable  cv_;
    std::vector<Item>        work_;
    bool                     stop_ = false;
    int                      poll_;
};

class MrailTeam final : public TlTeam {
public:
    explicit MrailTeam(MrailContext *c) : mctx(c) {}
    ~MrailTeam() override
    {
        for (xccl_team_h t : teams)
            if (t != nullptr) xccl_team_destroy(t);
    }
    xccl_status_t create_test() override { return XCCL_OK; }
    xccl_status_t collective_init(const xccl_coll_op_args_t &args, xccl_memory_type_t mem, xccl_coll_req **req) override;
    MrailContext            *mctx;
    std::vector<xccl_team_h> teams;
};

class MrailContext final : public TlContext {
public:
    MrailContext(const xccl_context_params_t &p, const MrailCfg &c) : params(p), cfg(c) {}
    ~MrailContext() override
    {
        workers.reset();
        for (xccl_context_h c : ctxs) xccl_context_destroy(c);
        if (lib != nullptr) xccl_lib_cleanup(lib);
    }
    xccl_status_t init()
    {
        xccl_tl_id_t id = xccl_tls_str_to_bitmap(cfg.replicate.c_str());
        if (id == XCCL_TL_NULL || (id & XCCL_TL_MRAIL)) return XCCL_ERR_INVALID_PARAM;
        xccl_lib_params_t lp{};
        xccl_status_t     st = xccl_lib_init(&lp, nullptr, &lib);
        if (st != XCCL_OK) return st;
        for (int r = 0; r < cfg.replicas; r++) {
            xccl_context_params_t cp = params;
            cp.field_mask |= XCCL_CONTEXT_PARAM_FIELD_TLS | XCCL_CONTEXT_PARAM_FIELD_THREAD_MODE;
            cp.tls         = (uint64_t)id | XCCL_TL_UCX;  // composite replicas need the host team underneath
            cp.thread_mode = cfg.threads > 0 ? XCCL_THREAD_MODE_MULTIPLE : params.thread_mode;
            std::string            prefix = "MRAIL" + std::to_string(r);
            xccl_context_config_t *cc     = nullptr;
            if (xccl_context_config_read(lib, prefix.c_str(), nullptr, &cc) != XCCL_OK) return XCCL_ERR_NO_MESSAGE;
            xccl_context_h c = nullptr;
            st               = xccl_context_create(lib, &cp, cc, &c);
            xccl_context_config_release(cc);
            if (st != XCCL_OK) return st;
            ctxs.push_back(c);
        }
        if (cfg.threads > 0) workers = std::make_unique<Workers>(std::min(cfg.threads, cfg.replicas), cfg.poll);
        return XCCL_OK;
    }
    xccl_status_t progress() override
    {
        if (workers) return XCCL_OK;  // the threads own the replicas
        for (xccl_context_h c : ctxs) {
            xccl_status_t st = xccl_context_progress(c);
            if (st < 0) return st;
        }
        return XCCL_OK;
    }
    bool          has_progress() const override { return true; }
    xccl_status_t team_create_post(const xccl_team_params_t &tp, TlTeam **team) override
    {
        auto t = std::make_unique<MrailTeam>(this);
        OobGroup g = make_oob_group(tp, params.oob);
        t->rank    = g.rank;
        t->size    = g.size;
        for (xccl_context_h c : ctxs) {
            xccl_team_params_t p  = tp;
            xccl_team_h        st = nullptr;
            xccl_status_t      s  = xccl_team_create_post(c, &p, &st);
            if (s != XCCL_OK) return s;
            double limit = global_state().opts.real("OOB_TIMEOUT");
            auto   t0    = std::chrono::steady_clock::now();
            while ((s = xccl_team_create_test(st)) == XCCL_INPROGRESS) {
                xccl_context_progress(c);
                if (limit > 0 && std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count() > limit) {
                    s = XCCL_ERR_TIMED_OUT;
                    break;
                }
            }
            if (s != XCCL_OK) {
                xccl_team_destroy(st);
                return s;
            }
            t->teams.push_back(st);
        }
        *team = t.release();
        return XCCL_OK;
    }
    xccl_context_params_t       params;
    MrailCfg                    cfg;
    xccl_lib_h                  lib = nullptr;
    std::vector<xccl_context_h> ctxs;
    std::unique_ptr<Workers>    workers;
};

class MrailReq final : public xccl_coll_req {
public:
    explicit MrailReq(MrailTeam *t) : team_(t) {}
    ~MrailReq() override
    {
        for (auto &s : subs_)
            if (s->req != nullptr) xccl_collective_finalize(s->req);
    }
    xccl_status_t build(const xccl_coll_op_args_t &a)
    {
        const int n = (int)team_->teams.size();
        if (a.coll_type == XCCL_BARRIER) return add(0, a);
        // equal ranges of whole elements; the last replica takes the remainder
        const size_t es    = a.coll_type == XCCL_ALLREDUCE ? xccl_dt_size(a.reduce_info.dt) : 1;
        const size_t total = a.coll_type == XCCL_ALLREDUCE ? a.reduce_info.count : a.buffer_info.len;
        const size_t per   = total / (size_t)n;
        char        *src   = (char *)a.buffer_info.src_buffer, *dst = (char *)a.buffer_info.dst_buffer;
        const bool   inpl  = (a.buffer_info.src_buffer == XCCL_IN_PLACE);
        for (int r = 0; r < n; r++) {
            size_t off = per * (size_t)r, cnt = (r == n - 1) ? total - off : per;
            if (cnt == 0) continue;
            xccl_coll_op_args_t s = a;
            if (!inpl && src != nullptr) s.buffer_info.src_buffer = src + off * es;
            s.buffer_info.dst_buffer = dst + off * es;
            s.buffer_info.len        = cnt * es;
            s.reduce_info.count      = cnt;
            xccl_status_t st         = add(r, s);
            if (st != XCCL_OK) return st;
        }
        return XCCL_OK;
    }
    xccl_status_t post() override
    {
        for (size_t i = 0; i < subs_.size(); i++) {
            xccl_status_t st = xccl_collective_post(subs_[i]->req);
            if (st != XCCL_OK) return st;
            subs_[i]->state.store(1, std::memory_order_release);
            if (team_->mctx->workers) team_->mctx->workers->submit(replica_[i], subs_[i].get());
        }
        return XCCL_OK;
    }
    xccl_status_t test() override
    {
        xccl_status_t result = XCCL_OK;
        for (auto &s : subs_) {
            int st = s->state.load(std::memory_order_acquire);
            if (st == 1 && !team_->mctx->workers) {
                xccl_status_t t = xccl_collective_test(s->req);
                if (t != XCCL_INPROGRESS) {
                    s->status = t;
                    s->state.store(2, std::memory_order_release);
                    st = 2;
                }
            }
            if (st == 1) return XCCL_INPROGRESS;
            if (st == 2 && s->status != XCCL_OK) result = s->status;
        }
        return result;
    }
    xccl_status_t finalize() override
    {
        for (auto &s : subs_)
            if (s->state.load() == 1) return XCCL_INPROGRESS;
        return XCCL_OK;
    }

private:
    xccl_status_t add(int replica, const xccl_coll_op_args_t &a)
    {
        auto                s    = std::make_unique<SubReq>();
        xccl_coll_op_args_t args = a;
        xccl_status_t       st   = xccl_collective_init(&args, &s->req, team_->teams[(size_t)replica]);
        if (st != XCCL_OK) return st;
        subs_.push_back(std::move(s));
        replica_.push_back(replica);
        return XCCL_OK;
    }
    MrailTeam                           *team_;
    std::vector<std::unique_ptr<SubReq>> subs_;
    std::vector<int>                     replica_;
};

xccl_status_t MrailTeam::collective_init(const xccl_coll_op_args_t &args, xccl_memory_type_t, xccl_coll_req **req)
{
    if (args.coll_type != XCCL_BARRIER && args.coll_type != XCCL_BCAST && args.coll_type != XCCL_ALLREDUCE) {
        return XCCL_ERR_UNSUPPORTED;
    }
    auto          r  = std::make_unique<MrailReq>(this);
    xccl_status_t st = r->build(args);
    if (st != XCCL_OK) return st;
    *req = r.release();
    return XCCL_OK;
}

class MrailLib final : public TeamLib {
public:
    MrailLib() : TeamLib(XCCL_TL_MRAIL, 100)
    {
        caps.coll_types = XCCL_COLL_CAP_BARRIER | XCCL_COLL_CAP_BCAST | XCCL_COLL_CAP_ALLREDUCE;
        caps.mem_types  = XCCL_BIT(XCCL_MEMORY_TYPE_HOST) | XCCL_BIT(XCCL_MEMORY_TYPE_CUDA);
    }
    std::vector<OptField> context_options() const override
    {
        return {
            {"REPLICATE_TEAM", "hier", "Team library to replicate", OptType::STRING},
            {"REPLICAS_NUMBER", "2", "How many replicas (rails)", OptType::UINT},
            {"THREADS_NUMBER", "2", "Progress threads that drive the replicas (reference default, src/team_lib/multirail/xccl_mrail_lib.c:40); 0 = the caller progresses", OptType::UINT},
            {"ASYNC_POLL_COUNT", "3", "Tests per request before a progress thread moves on", OptType::UINT},
            {"NET_DEVICES", "all", "Accepted for compatibility", OptType::STRING},
        };
    }
    xccl_status_t context_create(xccl_lib *, const xccl_context_params_t &params, const OptTable &cfg,
                                 TlContext **ctx) override
    {
        if (!(params.field_mask & XCCL_CONTEXT_PARAM_FIELD_OOB)) return XCCL_ERR_INVALID_PARAM;
        MrailCfg c;
        c.replicate = cfg.str("REPLICATE_TEAM");
        c.replicas  = std::max(1, (int)cfg.num("REPLICAS_NUMBER"));
        c.threads   = (int)cfg.num("THREADS_NUMBER");
        c.poll      = (int)cfg.num("ASYNC_POLL_COUNT");
        auto *m     = new MrailContext(params, c);
        m->tl       = this;
        xccl_status_t st = m->init();
        if (st != XCCL_OK) {
            delete m;
            return st;
        }
        *ctx = m;
        return XCCL_OK;
    }
};

MrailLib         g_mrail_lib;
TeamLibRegistrar g_mrail_reg(&g_mrail_lib);

}  // namespace

}  // namespace mrail
}  // namespace xccl
