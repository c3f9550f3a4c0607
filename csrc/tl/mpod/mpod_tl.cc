// Pod-split ("multi-pod") team library: a fast team inside each pod of POD_SIZE consecutive
// ranks (NVLink, else NCCL, for CUDA buffers) and the host team across pods.
// Counterpart of the reference's mpod team (src/team_lib/mpod/): the same decomposition
//   pod_id = rank / pod_size, slice_id = rank % pod_size
//   pod team    ranks of my pod            slice team   ranks with my slice_id in every pod
//   flat team   everyone (host team): host buffers, barrier and alltoallv go straight to it
// and the same algorithms for CUDA buffers, expressed as fragments of a CompositeReq:
//   allreduce  replicate: pod allreduce -> slice allreduce of the whole chunk
//              split:     pod reduce-scatter -> slice allreduce of my 1/pod_size share -> pod allgather
//                         (the share follows slice_id; the reference's variant sizes it by pod count)
//              coalesce:  pod allreduce -> slice 0 allreduces across pods -> pod bcast
//              chunked by ALLREDUCE_CHUNK_SIZE, chunks pipelined
//   allgather  pod allgather -> slice-0 allgather across pods -> pod bcast
//   bcast      bcast across pods on the root's slice -> pod bcast
//   alltoall   alltoall across pods (len * pod_size per peer) -> block transpose -> alltoall in the pod
//              (len * num_pods per peer) -> block transpose
// Requests of one team are serialised through a FIFO, as in the reference
// (src/team_lib/mpod/xccl_mpod_lib.c:482-567).
#include <algorithm>
#include <chrono>
#include <cstdlib>
#include <cstring>
#include <deque>
#include <mutex>

#include "../../core/composite.h"
#include "../../core/core.h"
#include "../../cuda/mem_cuda.h"
#include "../../utils/mem.h"
#include "xccl/xccl_oob.h"

namespace xccl {
namespace mpod {

namespace {

struct MpodCfg {
    int         pod_size = 0;  // 0 = whole team is one pod
    std::string allreduce_alg = "replicate";
    size_t      chunk_bytes   = 256u << 20;
    bool        host_hierarchy = false;  // run the pod algorithms on host buffers too (testing, CPU-only nodes)
};

class MpodContext;

class MpodTeam final : public TlTeam {
public:
    MpodTeam(MpodContext *c, const OobGroup &g) : mctx(c), oob(g)
    {
        rank = g.rank;
        size = g.size;
    }
    ~MpodTeam() override;
    xccl_status_t init();
    xccl_status_t create_test() override { return XCCL_OK; }
    xccl_status_t collective_init(const xccl_coll_op_args_t &args, xccl_memory_type_t mem, xccl_coll_req **req) override;

    MpodContext *mctx;
    OobGroup     oob;
    int          pod_size = 1, num_pods = 1, pod_id = 0, slice_id = 0;
    xccl_team_h  pod_dev = nullptr, pod_host = nullptr, slice = nullptr, flat = nullptr;
    std::deque<xccl_coll_req *> fifo;  // posted requests in order; only the head runs
    std::mutex                  fifo_mu;

private:
    xccl_status_t make_team(xccl_context_h ctx, const std::vector<int> &ranks, xccl_team_h *out, bool optional);
    xccl_oob_collectives_t              team_oob_{};
    std::vector<xccl_oob_collectives_t> sub_oobs_;
};

class MpodContext final : public TlContext {
public:
    MpodContext(const xccl_context_params_t &p, const MpodCfg &c) : params(p), cfg(c) {}
    ~MpodContext() override
    {
        if (dev != nullptr) xccl_context_destroy(dev);
        if (host != nullptr) xccl_context_destroy(host);
        if (lib != nullptr) xccl_lib_cleanup(lib);
    }
    xccl_status_t init()
    {
        xccl_lib_params_t lp{};
        xccl_status_t     st = xccl_lib_init(&lp, nullptr, &lib);
        if (st != XCCL_OK) return st;
        auto make = [&](uint64_t tls, const char *prefix, xccl_context_h *out) {
            xccl_context_params_t cp = params;
            cp.field_mask |= XCCL_CONTEXT_PARAM_FIELD_TLS;
            cp.tls                    = tls;
            xccl_context_config_t *cc = nullptr;
            if (xccl_context_config_read(lib, prefix, nullptr, &cc) != XCCL_OK) return XCCL_ERR_NO_MESSAGE;
            xccl_status_t s = xccl_context_create(lib, &cp, cc, out);
            xccl_context_config_release(cc);
            return s;
        };
        st = make(XCCL_TL_UCX, "MPOD_ucx", &host);
        if (st != XCCL_OK) return st;
        // the device level is optional: NVLink team first, NCCL team second, neither on a machine without GPUs
        if (!lib->has(XCCL_TL_NVLINK) || make(XCCL_TL_NVLINK, "MPOD_nvlink", &dev) != XCCL_OK) {
            dev = nullptr;
            if (!lib->has(XCCL_TL_NCCL) || make(XCCL_TL_NCCL, "MPOD_nccl", &dev) != XCCL_OK) dev = nullptr;
        }
        return XCCL_OK;
    }
    xccl_status_t progress() override
    {
        xccl_status_t st = xccl_context_progress(host);
        if (st < 0) return st;
        return dev != nullptr ? xccl_context_progress(dev) : XCCL_OK;
    }
    bool          has_progress() const override { return true; }
    xccl_status_t team_create_post(const xccl_team_params_t &tp, TlTeam **team) override
    {
        OobGroup g = make_oob_group(tp, params.oob);
        if (g.rank < 0 || g.size < 1) return XCCL_ERR_INVALID_PARAM;
        auto         *t  = new MpodTeam(this, g);
        xccl_status_t st = t->init();
        if (st != XCCL_OK) {
            delete t;
            return st;
        }
        *team = t;
        return XCCL_OK;
    }
    xccl_context_params_t params;
    MpodCfg               cfg;
    xccl_lib_h            lib = nullptr;
    xccl_context_h        dev = nullptr, host = nullptr;
};

MpodTeam::~MpodTeam()
{
    for (xccl_team_h t : {pod_dev, pod_host, slice, flat}) {
        if (t != nullptr) xccl_team_destroy(t);
    }
    for (auto &o : sub_oobs_) xccl_oob_sub_destroy(&o);
    if (team_oob_.coll_context != nullptr) xccl_oob_sub_destroy(&team_oob_);
}

xccl_status_t MpodTeam::make_team(xccl_context_h ctx, const std::vector<int> &ranks, xccl_team_h *out, bool optional)
{
    *out = nullptr;
    if (ctx == nullptr || ranks.size() < 2) return XCCL_OK;  // a group of one needs no team
    xccl_oob_collectives_t sub{};
    xccl_status_t          st = xccl_oob_sub_create(&team_oob_, ranks.data(), (int)ranks.size(), &sub);
    if (st != XCCL_OK) return st;
    sub_oobs_.push_back(sub);
    xccl_team_params_t tp{};
    tp.field_mask   = XCCL_TEAM_PARAM_FIELD_OOB | XCCL_TEAM_PARAM_FIELD_EP_RANGE;
    tp.oob          = sub;
    tp.range.type   = XCCL_EP_RANGE_FULL;
    tp.range.ep_num = (int)ranks.size();
    xccl_team_h t   = nullptr;
    st              = xccl_team_create_post(ctx, &tp, &t);
    if (st == XCCL_OK) {
        double limit = global_state().opts.real("OOB_TIMEOUT");
        auto   t0    = std::chrono::steady_clock::now();
        while ((st = xccl_team_create_test(t)) == XCCL_INPROGRESS) {
            xccl_context_progress(ctx);
            if (limit > 0 && std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count() > limit) {
                st = XCCL_ERR_TIMED_OUT;
                break;
            }
        }
        if (st != XCCL_OK) {
            xccl_team_destroy(t);
            t = nullptr;
        }
    }
    if (st != XCCL_OK) return optional ? XCCL_OK : st;
    *out = t;
    return XCCL_OK;
}

xccl_status_t MpodTeam::init()
{
    const MpodCfg &cfg = mctx->cfg;
    pod_size           = cfg.pod_size > 0 ? cfg.pod_size : size;
    if (size % pod_size != 0) {
        tl_error(mctx->tl, "mpod: team size %d is not a multiple of the pod size %d", size, pod_size);
        return XCCL_ERR_INVALID_PARAM;
    }
    num_pods = size / pod_size;
    pod_id   = rank / pod_size;
    slice_id = rank % pod_size;
    std::vector<int> ctx_ranks((size_t)size), pod, sl, all;
    for (int i = 0; i < size; i++) {
        ctx_ranks[(size_t)i] = oob.ctx_rank(i);
        all.push_back(i);
        if (i / pod_size == pod_id) pod.push_back(i);
        if (i % pod_size == slice_id) sl.push_back(i);
    }
    xccl_status_t st = xccl_oob_sub_create(&oob.oob, ctx_ranks.data(), size, &team_oob_);
    if (st != XCCL_OK) return st;
    // same creation order everywhere; each sub-team's members create it together
    if ((st = make_team(mctx->dev, pod, &pod_dev, true)) != XCCL_OK) return st;
    if ((st = make_team(mctx->host, pod, &pod_host, false)) != XCCL_OK) return st;
    if ((st = make_team(mctx->host, sl, &slice, false)) != XCCL_OK) return st;
    if ((st = make_team(mctx->host, all, &flat, false)) != XCCL_OK) return st;
    tl_debug(mctx->tl, "mpod team: rank %d/%d, pod %d of %d, slice %d of %d, device pod team %s", rank, size, pod_id,
             num_pods, slice_id, pod_size, pod_dev != nullptr ? "yes" : "no");
    return XCCL_OK;
}

// A CompositeReq that waits its turn in the team FIFO.
class MpodReq final : public CompositeReq {
public:
    MpodReq(MpodTeam *t) : CompositeReq(t->mctx->core), team_(t) {}
    ~MpodReq() override
    {
        for (auto &b : tmp_) mem_free(b.first, b.second);
    }
    xccl_status_t post() override
    {
        std::lock_guard<std::mutex> lock(team_->fifo_mu);
        if (queued_ || running_) return XCCL_ERR_NO_RESOURCE;
        last_ = XCCL_INPROGRESS;
        team_->fifo.push_back(this);
        queued_ = true;
        if (team_->fifo.front() == this) return start_locked();
        return XCCL_OK;
    }
    xccl_status_t test() override
    {
        std::unique_lock<std::mutex> lock(team_->fifo_mu);
        if (!queued_ && !running_) return last_ == XCCL_INPROGRESS ? XCCL_OK : last_;
        MpodReq *head = static_cast<MpodReq *>(team_->fifo.front());
        if (!head->running_) {
            xccl_status_t st = head->start_locked();
            if (st != XCCL_OK) return st;
        }
        lock.unlock();
        xccl_status_t hst = head->CompositeReq::test();
        lock.lock();
        if (hst != XCCL_INPROGRESS && !team_->fifo.empty() && team_->fifo.front() == head && head->running_) {
            head->running_ = false;
            head->queued_  = false;
            head->last_    = hst;
            team_->fifo.pop_front();
        }
        if (head == this) return hst;
        return (queued_ || running_) ? XCCL_INPROGRESS : last_;
    }
    xccl_status_t finalize() override
    {
        std::lock_guard<std::mutex> lock(team_->fifo_mu);
        return (queued_ || running_) ? XCCL_INPROGRESS : XCCL_OK;
    }
    void *scratch(size_t bytes, xccl_memory_type_t mem)
    {
        void *p = nullptr;
        if (mem_alloc(&p, bytes, mem) != XCCL_OK) return nullptr;
        tmp_.emplace_back(p, mem);
        return p;
    }

private:
    xccl_status_t start_locked()
    {
        running_ = true;
        return CompositeReq::post();
    }
    MpodTeam     *team_;
    bool          queued_ = false, running_ = false;
    xccl_status_t last_   = XCCL_OK;
    std::vector<std::pair<void *, xccl_memory_type_t>> tmp_;
};

CompositeStep coll(xccl_team_h team, const xccl_coll_op_args_t &base, xccl_collective_type_t type, void *src, void *dst,
                   size_t len, size_t count, int root)
{
    CompositeStep s;
    s.team                        = team;
    s.args                        = base;
    s.args.coll_type              = type;
    s.args.alg.set_by_user        = 0;
    s.args.buffer_info.src_buffer = src;
    s.args.buffer_info.dst_buffer = dst;
    s.args.buffer_info.len        = len;
    s.args.reduce_info.count      = count;
    s.args.root                   = root;
    s.args.field_mask &= ~(uint64_t)XCCL_COLL_OP_ARGS_FIELD_EPILOGUE;
    return s;
}

}  // namespace

xccl_status_t MpodTeam::collective_init(const xccl_coll_op_args_t &a, xccl_memory_type_t mem, xccl_coll_req **req)
{
    auto                          r   = std::make_unique<MpodReq>(this);
    const xccl_coll_buffer_info_t &bi = a.buffer_info;
    const bool sync_only = (a.coll_type == XCCL_BARRIER);
    const bool hierarchical = !sync_only && a.coll_type != XCCL_ALLTOALLV &&
                              (mem == XCCL_MEMORY_TYPE_CUDA || mctx->cfg.host_hierarchy) && num_pods > 1 && pod_size > 1;
    xccl_team_h   pod = (mem == XCCL_MEMORY_TYPE_CUDA && pod_dev != nullptr) ? pod_dev : pod_host;
    xccl_status_t st  = XCCL_OK;
    void *src = bi.src_buffer, *dst = bi.dst_buffer;
    if (!sync_only && (src == XCCL_IN_PLACE || src == nullptr)) src = dst;

    if (!hierarchical) {
        // one level only: the flat host team, or the pod team when the team is a single pod
        xccl_team_h t = flat;
        if (num_pods == 1 && mem == XCCL_MEMORY_TYPE_CUDA && pod_dev != nullptr && a.coll_type != XCCL_BARRIER) t = pod_dev;
        if (t == nullptr) return XCCL_ERR_UNSUPPORTED;
        CompositeStep s;
        s.team = t;
        s.args = a;
        st     = r->add_fragment({s});
    } else if (a.coll_type == XCCL_ALLREDUCE) {
        const size_t es    = xccl_dt_size(a.reduce_info.dt);
        const size_t total = a.reduce_info.count;
        size_t       chunk = std::max<size_t>(mctx->cfg.chunk_bytes / std::max<size_t>(es, 1), 1);
        const std::string &alg = mctx->cfg.allreduce_alg;
        for (size_t off = 0; off < total && st == XCCL_OK; off += chunk) {
            const size_t n = std::min(chunk, total - off);
            char        *s = (char *)src + off * es, *d = (char *)dst + off * es;
            std::vector<CompositeStep> f;
            if (alg == "split" && n % (size_t)pod_size == 0) {
                const size_t share = n / (size_t)pod_size;
                char        *mine  = d + (size_t)slice_id * share * es;
                f.push_back(coll(pod, a, XCCL_REDUCE_SCATTER, s, mine, n * es, share, 0));
                f.push_back(coll(slice, a, XCCL_ALLREDUCE, mine, mine, share * es, share, 0));
                f.push_back(coll(pod, a, XCCL_ALLGATHER, XCCL_IN_PLACE, d, n * es, 0, 0));
            } else if (alg == "coalesce") {
                f.push_back(coll(pod, a, XCCL_ALLREDUCE, s, d, n * es, n, 0));
                if (slice_id == 0) f.push_back(coll(slice, a, XCCL_ALLREDUCE, d, d, n * es, n, 0));
                f.push_back(coll(pod, a, XCCL_BCAST, d, d, n * es, 0, 0));
            } else {
                f.push_back(coll(pod, a, XCCL_ALLREDUCE, s, d, n * es, n, 0));
                f.push_back(coll(slice, a, XCCL_ALLREDUCE, d, d, n * es, n, 0));
            }
            st = r->add_fragment(f);
        }
    } else if (a.coll_type == XCCL_ALLGATHER) {
        const size_t blk = bi.len / (size_t)size, pod_bytes = blk * (size_t)pod_size;
        char        *region = (char *)dst + (size_t)pod_id * pod_bytes;
        void        *my_src = (bi.src_buffer == XCCL_IN_PLACE) ? (void *)XCCL_IN_PLACE : src;
        std::vector<CompositeStep> f;
        // in place: the caller's block already sits at dst + rank * blk, its slot in the pod region
        f.push_back(coll(pod, a, XCCL_ALLGATHER, my_src, region, pod_bytes, 0, 0));
        if (slice_id == 0) f.push_back(coll(slice, a, XCCL_ALLGATHER, XCCL_IN_PLACE, dst, bi.len, 0, 0));
        f.push_back(coll(pod, a, XCCL_BCAST, dst, dst, bi.len, 0, 0));
        st = r->add_fragment(f);
    } else if (a.coll_type == XCCL_BCAST) {
        const int root_pod = a.root / pod_size, root_slice = a.root % pod_size;
        std::vector<CompositeStep> f;
        if (slice_id == root_slice) f.push_back(coll(slice, a, XCCL_BCAST, rank == a.root ? src : dst, dst, bi.len, 0, root_pod));
        f.push_back(coll(pod, a, XCCL_BCAST, dst, dst, bi.len, 0, root_slice));
        st = r->add_fragment(f);
    } else if (a.coll_type == XCCL_ALLTOALL) {
        if (src == dst) return XCCL_ERR_UNSUPPORTED;
        const size_t len = bi.len, all_bytes = len * (size_t)size;
        char *t1 = (char *)r->scratch(all_bytes, mem), *t2 = (char *)r->scratch(all_bytes, mem);
        if (t1 == nullptr || t2 == nullptr) return XCCL_ERR_NO_MEMORY;
        const int P = num_pods, S = pod_size;
        void *stream = ((a.field_mask & XCCL_COLL_OP_ARGS_FIELD_STREAM) && a.stream.stream != nullptr)
                           ? *(void **)a.stream.stream
                           : nullptr;
        auto transpose = [mem, len, stream](char *to, const char *from, int rows, int cols) {
            CompositeStep s;
            s.local = [=]() -> xccl_status_t {
                if (mem == XCCL_MEMORY_TYPE_CUDA) {
                    void         *q  = stream != nullptr ? stream : cuda_internal_stream();
                    xccl_status_t st = cuda_block_transpose(to, from, rows, cols, len, q);
                    return st != XCCL_OK ? st : cuda_stream_sync(q);
                }
                for (int i = 0; i < rows; i++)
                    for (int j = 0; j < cols; j++)
                        std::memcpy(to + ((size_t)j * rows + i) * len, from + ((size_t)i * cols + j) * len, len);
                return XCCL_OK;
            };
            return s;
        };
        std::vector<CompositeStep> f;
        f.push_back(coll(slice, a, XCCL_ALLTOALL, src, t1, len * (size_t)S, 0, 0));  // t1[p''][s'] from pod p''
        f.push_back(transpose(t2, t1, P, S));                                         // t2[s'][p'']
        f.push_back(coll(pod, a, XCCL_ALLTOALL, t2, t1, len * (size_t)P, 0, 0));      // t1[s][p''] from slice s
        f.push_back(transpose((char *)dst, t1, S, P));                                // dst[p''][s] = rank order
        st = r->add_fragment(f);
    } else {
        return XCCL_ERR_UNSUPPORTED;
    }
    if (st != XCCL_OK) return st;
    *req = r.release();
    return XCCL_OK;
}

namespace {

class MpodLib final : public TeamLib {
public:
    MpodLib() : TeamLib(XCCL_TL_MPOD, 90)
    {
        caps.coll_types = XCCL_COLL_CAP_BARRIER | XCCL_COLL_CAP_BCAST | XCCL_COLL_CAP_ALLREDUCE | XCCL_COLL_CAP_ALLGATHER |
                          XCCL_COLL_CAP_ALLTOALL | XCCL_COLL_CAP_ALLTOALLV;
        caps.mem_types = XCCL_BIT(XCCL_MEMORY_TYPE_HOST) | XCCL_BIT(XCCL_MEMORY_TYPE_CUDA);
    }
    std::vector<OptField> context_options() const override
    {
        return {
            {"POD_SIZE", "0", "Ranks per pod (XCCL_POD_SIZE is honoured too); 0 = one pod", OptType::UINT},
            {"ALLREDUCE_ALGORITHM", "replicate", "replicate, split or coalesce (XCCL_MPOD_ALLREDUCE_ALGORITHM too)", OptType::STRING},
            {"ALLREDUCE_CHUNK_SIZE", "256m", "Bytes per pipelined chunk (XCCL_MPOD_ALLREDUCE_CHUNK_SIZE too)", OptType::MEMUNITS},
            {"HOST_HIERARCHY", "no", "Use the pod algorithms for host buffers as well", OptType::BOOL},
        };
    }
    xccl_status_t context_create(xccl_lib *, const xccl_context_params_t &params, const OptTable &cfg,
                                 TlContext **ctx) override
    {
        MpodCfg c;
        c.pod_size       = (int)cfg.num("POD_SIZE");
        c.allreduce_alg  = cfg.str("ALLREDUCE_ALGORITHM");
        c.chunk_bytes    = (size_t)cfg.num("ALLREDUCE_CHUNK_SIZE");
        c.host_hierarchy = cfg.flag("HOST_HIERARCHY");
        // the reference reads these three straight from the environment
        if (const char *e = std::getenv("XCCL_POD_SIZE")) c.pod_size = std::atoi(e);
        if (const char *e = std::getenv("XCCL_MPOD_ALLREDUCE_ALGORITHM")) c.allreduce_alg = e;
        if (const char *e = std::getenv("XCCL_MPOD_ALLREDUCE_CHUNK_SIZE")) {
            bool      ok = true;
            long long v  = parse_memunits(e, &ok);
            if (ok && v > 0) c.chunk_bytes = (size_t)v;
        }
        if (!(params.field_mask & XCCL_CONTEXT_PARAM_FIELD_OOB)) return XCCL_ERR_INVALID_PARAM;
        auto *m = new MpodContext(params, c);
        m->tl   = this;
        xccl_status_t st = m->init();
        if (st != XCCL_OK) {
            delete m;
            return st;
        }
        *ctx = m;
        return XCCL_OK;
    }
};

MpodLib          g_mpod_lib;
TeamLibRegistrar g_mpod_reg(&g_mpod_lib);

}  // namespace

}  // namespace mpod
}  // namespace xccl
