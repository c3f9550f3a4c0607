// Host team library: lib / context / team / request glue around the algorithms.
// Reference: src/team_lib/ucx/xccl_ucx_lib.c:162-671 (request life cycle, option table,
// stream-ordered start), src/team_lib/ucx/xccl_ucx_team.c:23-118 (non-blocking team creation).
#include "host_tl.h"

#include <cstdlib>
#include <cstring>

#include "../../cuda/mem_cuda.h"
#include "../../utils/mem.h"

namespace xccl {
namespace host {

// ------------------------------------------------------------------ team

HostTeam::HostTeam(TeamLib *tl_, const OobGroup &g, const HostCfg &c)
    : tl(tl_), oob(g), cfg(c), tr(g.rank, g.size, c.ring_bytes), all_((size_t)g.size)
{
    rank = g.rank;
    size = g.size;
}

HostTeam::~HostTeam()
{
    if (oob_req_ != nullptr) oob.free(oob_req_);
}

xccl_status_t HostTeam::start()
{
    xccl_status_t st = tr.create_local(&mine_);
    if (st != XCCL_OK) return st;
    if (oob.allgather(&mine_, all_.data(), sizeof(PeerInfo), &oob_req_) != 0) return XCCL_ERR_NO_MESSAGE;
    phase_ = 1;
    return XCCL_OK;
}

xccl_status_t HostTeam::create_test()
{
    if (phase_ == 2) return XCCL_OK;
    if (phase_ != 1) return XCCL_ERR_NO_MESSAGE;
    xccl_status_t st = oob.test(oob_req_);
    if (st != XCCL_OK) return st;
    oob.free(oob_req_);
    oob_req_ = nullptr;
    st       = tr.connect(all_.data());
    if (st != XCCL_OK) {
        phase_ = -1;
        return st;
    }
    phase_ = 2;
    tl_debug(tl, "host team ready: rank %d of %d, ring %zu bytes per peer", rank, size, cfg.ring_bytes);
    return XCCL_OK;
}

xccl_status_t HostTeam::collective_init(const xccl_coll_op_args_t &args, xccl_memory_type_t mem, xccl_coll_req **req)
{
    auto         *r  = new HostReq(this, args, mem);
    xccl_status_t st = r->prepare();
    if (st != XCCL_OK) {
        delete r;
        return st;
    }
    *req = r;
    return XCCL_OK;
}

// ------------------------------------------------------------------ request

HostReq::HostReq(HostTeam *t, const xccl_coll_op_args_t &a, xccl_memory_type_t m) : team(t), args(a), mem(m) {}

HostReq::~HostReq()
{
    coro_.reset();
    if (h_src_ != nullptr) std::free(h_src_);
    if (h_dst_ != nullptr) std::free(h_dst_);
    if (event_ != nullptr) cuda_event_release(event_);
}

P2pReq *HostReq::send(int peer, const void *buf, size_t len)
{
    std::lock_guard<std::recursive_mutex> lock(team->mu);
    p2p_.emplace_back();
    team->tr.send_nb(peer, buf, len, tag, &p2p_.back());
    return &p2p_.back();
}

P2pReq *HostReq::recv(int peer, void *buf, size_t len)
{
    std::lock_guard<std::recursive_mutex> lock(team->mu);
    p2p_.emplace_back();
    team->tr.recv_nb(peer, buf, len, tag, &p2p_.back());
    return &p2p_.back();
}

void HostReq::progress()
{
    std::lock_guard<std::recursive_mutex> lock(team->mu);
    team->tr.progress();
}

// Polls the transport up to NUM_TO_PROBE times (reference: the probe count of xccl_ucx_req_test,
// src/team_lib/ucx/xccl_ucx_sendrecv.h:200-216) before the caller's test returns "in progress".
bool HostReq::all_done()
{
    const int probes = std::max(1, team->cfg.num_to_probe);
    bool      done   = false;
    for (int k = 0; k < probes && !done; k++) {
        progress();
        done = true;
        for (const P2pReq &q : p2p_) {
            if (!q.done) {
                done = false;
                break;
            }
        }
    }
    if (!done) return false;
    for (const P2pReq &q : p2p_) {
        if (q.status != XCCL_OK && last_ == XCCL_OK) last_ = q.status;
    }
    return true;
}

void HostReq::drop_completed()
{
    while (!p2p_.empty() && p2p_.front().done) p2p_.pop_front();
}

xccl_status_t HostReq::reduce_multi(const void *a, const void *vecs, void *dst, size_t n, size_t count, size_t stride)
{
    return host_reduce_multi(a, vecs, dst, n, count, stride, b.dt, b.op);
}

char *HostReq::scratch(size_t bytes)
{
    if (scratch_.size() < bytes) scratch_.resize(bytes);
    return scratch_.data();
}

xccl_status_t HostReq::prepare()
{
    const xccl_coll_buffer_info_t &bi = args.buffer_info;
    const int                      n  = team->size;
    b.root                            = args.root;
    b.dt                              = args.reduce_info.dt;
    b.op                              = args.reduce_info.op;
    b.count                           = args.reduce_info.count;
    b.len                             = bi.len;
    tag                               = team->seq++;
    size_t src_bytes = 0, dst_bytes = 0;
    bool   user_alg = args.alg.set_by_user != 0;
    int    alg_id   = args.alg.id;

    switch (args.coll_type) {
    case XCCL_ALLREDUCE: {
        if (!host_reduce_supported(b.dt, b.op)) return XCCL_ERR_UNSUPPORTED;
        if (b.len == 0) b.len = b.count * xccl_dt_size(b.dt);
        src_bytes = dst_bytes = b.len;
        bool sra;
        if (user_alg) {
            sra = (alg_id == XCCL_HOST_ALG_SRA);
        } else if (team->cfg.allreduce_alg == "knomial") {
            sra = false;
        } else if (team->cfg.allreduce_alg == "sra") {
            sra = true;
        } else {
            sra = b.len >= team->cfg.sra_threshold;
        }
        algo_ = sra ? allreduce_sra : allreduce_knomial;
        break;
    }
    case XCCL_REDUCE:
        if (!host_reduce_supported(b.dt, b.op)) return XCCL_ERR_UNSUPPORTED;
        if (b.len == 0) b.len = b.count * xccl_dt_size(b.dt);
        src_bytes = dst_bytes = b.len;
        algo_ = (user_alg && alg_id == XCCL_HOST_ALG_LINEAR) ? reduce_linear : reduce_knomial;
        break;
    case XCCL_REDUCE_SCATTER:
        if (!host_reduce_supported(b.dt, b.op)) return XCCL_ERR_UNSUPPORTED;
        if (bi.src_buffer == XCCL_IN_PLACE) return XCCL_ERR_UNSUPPORTED;
        if (b.len == 0) b.len = b.count * xccl_dt_size(b.dt) * (size_t)n;
        b.count   = b.len / (size_t)n / xccl_dt_size(b.dt);
        src_bytes = b.len;
        dst_bytes = b.len / (size_t)n;
        algo_     = reduce_scatter_pairwise;
        break;
    case XCCL_BCAST:
        src_bytes = dst_bytes = b.len;
        algo_ = (user_alg && alg_id == XCCL_HOST_ALG_LINEAR) ? bcast_linear : bcast_knomial;
        break;
    case XCCL_BARRIER: algo_ = barrier_knomial; break;
    case XCCL_FANIN: algo_ = fanin_linear; break;
    case XCCL_FANOUT: algo_ = fanout_linear; break;
    case XCCL_ALLGATHER:
        src_bytes = b.len / (size_t)n;
        dst_bytes = b.len;
        algo_     = allgather_ring;
        break;
    case XCCL_ALLTOALL:
        src_bytes = dst_bytes = b.len * (size_t)n;
        if (bi.src_buffer == XCCL_IN_PLACE || bi.src_buffer == bi.dst_buffer ||
            (user_alg && alg_id == XCCL_HOST_ALG_KNOMIAL)) {
            algo_ = alltoall_linear_shift;
        } else {
            algo_ = alltoall_pairwise;
        }
        break;
    case XCCL_ALLTOALLV: {
        if (bi.src_buffer == XCCL_IN_PLACE || bi.src_buffer == bi.dst_buffer) return XCCL_ERR_UNSUPPORTED;
        if (bi.src_counts == nullptr || bi.dst_counts == nullptr || bi.src_displacements == nullptr ||
            bi.dst_displacements == nullptr) {
            return XCCL_ERR_INVALID_PARAM;
        }
        b.src_counts.assign(bi.src_counts, bi.src_counts + n);
        b.dst_counts.assign(bi.dst_counts, bi.dst_counts + n);
        b.src_displs.assign(bi.src_displacements, bi.src_displacements + n);
        b.dst_displs.assign(bi.dst_displacements, bi.dst_displacements + n);
        b.src_dt_size = xccl_dt_size(bi.src_datatype);
        b.dst_dt_size = xccl_dt_size(bi.dst_datatype);
        if (b.src_dt_size == 0 || b.dst_dt_size == 0) return XCCL_ERR_INVALID_PARAM;
        for (int p = 0; p < n; p++) {
            src_bytes = std::max(src_bytes, ((size_t)b.src_displs[(size_t)p] + b.src_counts[(size_t)p]) * b.src_dt_size);
            dst_bytes = std::max(dst_bytes, ((size_t)b.dst_displs[(size_t)p] + b.dst_counts[(size_t)p]) * b.dst_dt_size);
        }
        algo_ = alltoallv_pairwise;
        break;
    }
    default: return XCCL_ERR_UNSUPPORTED;
    }

    const bool reduction = (args.coll_type == XCCL_ALLREDUCE || args.coll_type == XCCL_REDUCE ||
                            args.coll_type == XCCL_REDUCE_SCATTER);
    if (reduction && (args.field_mask & XCCL_COLL_OP_ARGS_FIELD_EPILOGUE)) {
        epi_out_dt_ = args.epilogue.out_dt;
        if (epi_out_dt_ == XCCL_DT_UNSUPPORTED || epi_out_dt_ == XCCL_DT_LAST_PREDEFINED) epi_out_dt_ = b.dt;
        epi_scale_  = args.epilogue.scale;
        epi_        = (epi_scale_ != 1.0f) || (epi_out_dt_ != b.dt);
        epi_count_  = dst_bytes / xccl_dt_size(b.dt);
        // probe the conversion once so that an unsupported pair fails at init
        char probe_in[16] = {0}, probe_out[16] = {0};
        if (epi_ && host_scale_cast(probe_in, b.dt, probe_out, epi_out_dt_, 1, 1.0f) != XCCL_OK) return XCCL_ERR_UNSUPPORTED;
    }
    char *src = (char *)bi.src_buffer, *dst = (char *)bi.dst_buffer;
    bool  sync_only = (args.coll_type == XCCL_BARRIER || args.coll_type == XCCL_FANIN || args.coll_type == XCCL_FANOUT);
    if (!sync_only) {
        if (src == (char *)XCCL_IN_PLACE || src == nullptr) src = dst;
        if (args.coll_type == XCCL_ALLGATHER && bi.src_buffer == XCCL_IN_PLACE) {
            src = dst + (size_t)team->rank * (b.len / (size_t)n);
        }
    }
    if (mem == XCCL_MEMORY_TYPE_CUDA && !sync_only) {
        // CUDA buffers are staged through host memory around the host algorithm
        d_src_       = src;
        d_dst_       = dst;
        h_src_bytes_ = src_bytes;
        h_dst_bytes_ = epi_ ? epi_count_ * xccl_dt_size(epi_out_dt_) : dst_bytes;
        h_dst_       = (char *)std::malloc(std::max<size_t>(std::max(dst_bytes, h_dst_bytes_), 1));
        bool aliased = (src == dst);
        h_src_       = aliased ? nullptr : (char *)std::malloc(std::max<size_t>(src_bytes, 1));
        if (h_dst_ == nullptr || (!aliased && h_src_ == nullptr)) return XCCL_ERR_NO_MEMORY;
        b.dst = h_dst_;
        b.src = aliased ? h_dst_ : h_src_;
        if (args.coll_type == XCCL_ALLGATHER && bi.src_buffer == XCCL_IN_PLACE) {
            b.src = h_dst_ + (size_t)team->rank * (b.len / (size_t)n);
        }
    } else {
        b.src = src;
        b.dst = dst;
    }
    if (epi_) {
        // reduce in the input datatype into a private buffer, convert into the real destination
        epi_dst_ = b.dst;
        epi_buf_.resize(std::max<size_t>(dst_bytes, 1));
        if (b.src == b.dst) {
            // in place: the private buffer starts as a copy of the input (made at post time)
            b.src = nullptr;
        }
        b.dst = epi_buf_.data();
    }
    return XCCL_OK;
}

Coro HostReq::run()
{
    const bool staged = (d_dst_ != nullptr);
    if (staged) {
        // start only after work already queued on the caller's stream has finished
        if (event_ != nullptr) {
            xccl_status_t est;
            while ((est = cuda_event_query(event_)) == XCCL_INPROGRESS) co_await std::suspend_always{};
            if (est != XCCL_OK) co_return est;
        }
        // dst first: for aliased or in-place layouts the device dst holds the input
        bool in_place_gather = (args.coll_type == XCCL_ALLGATHER && args.buffer_info.src_buffer == XCCL_IN_PLACE);
        if (h_src_ == nullptr || in_place_gather) {
            xccl_status_t st = cuda_copy(h_dst_, d_dst_, h_dst_bytes_, nullptr);
            if (st != XCCL_OK) co_return st;
        } else {
            xccl_status_t st = cuda_copy(h_src_, d_src_, h_src_bytes_, nullptr);
            if (st != XCCL_OK) co_return st;
        }
    }
    if (epi_ && b.src == nullptr) {
        // in-place call: seed the private buffer with the input that sits in the destination
        std::memcpy(epi_buf_.data(), epi_dst_, epi_buf_.size());
        b.src = epi_buf_.data();
        XCCL_CO_CALL(algo_(*this));
        b.src = nullptr;
    } else {
        XCCL_CO_CALL(algo_(*this));
    }
    if (epi_ && !(args.coll_type == XCCL_REDUCE && team->rank != b.root)) {
        xccl_status_t cst = host_scale_cast(epi_buf_.data(), b.dt, epi_dst_, epi_out_dt_, epi_count_, epi_scale_);
        if (cst != XCCL_OK) co_return cst;
    }
    if (staged) {
        bool has_result = true;
        if (args.coll_type == XCCL_REDUCE && team->rank != b.root) has_result = false;
        if (has_result) {
            xccl_status_t st = cuda_copy(d_dst_, h_dst_, h_dst_bytes_, nullptr);
            if (st != XCCL_OK) co_return st;
        }
    }
    co_return last_;
}

xccl_status_t HostReq::post()
{
    if (in_flight_) return XCCL_ERR_NO_RESOURCE;
    if (team->poisoned) return XCCL_ERR_NO_PROGRESS;
    p2p_.clear();
    last_ = XCCL_OK;
    if (event_ != nullptr) {
        cuda_event_release(event_);
        event_ = nullptr;
    }
    if (d_dst_ != nullptr && (args.field_mask & XCCL_COLL_OP_ARGS_FIELD_STREAM) && args.stream.stream != nullptr) {
        void         *stream = *(void **)args.stream.stream;
        xccl_status_t st     = cuda_event_record(stream, &event_);
        if (st != XCCL_OK) return st;
        if (team->cfg.block_stream) {
            StreamHold *h = nullptr;
            st            = hold_start(stream, &h);
            if (st != XCCL_OK) return st;
            hold_ = h;
        }
    }
    coro_      = run();
    in_flight_ = true;
    test();  // first progress call, as the reference's start functions do
    return XCCL_OK;
}

xccl_status_t HostReq::test()
{
    if (!in_flight_) return last_;
    if (!coro_.step()) return XCCL_INPROGRESS;
    in_flight_ = false;
    last_      = coro_.result();
    coro_.reset();
    if (hold_ != nullptr) {
        hold_release((StreamHold *)hold_);
        xccl_status_t hst = hold_finish((StreamHold *)hold_);
        hold_             = nullptr;
        if (hst != XCCL_OK && last_ == XCCL_OK) last_ = hst;
    }
    if (last_ < 0) team->poisoned = true;
    return last_;
}

xccl_status_t HostReq::finalize() { return in_flight_ ? XCCL_INPROGRESS : XCCL_OK; }

// ------------------------------------------------------------------ context + lib

namespace {

class HostContext final : public TlContext {
public:
    HostContext(const xccl_context_params_t &p, const HostCfg &c) : params_(p), cfg_(c) {}
    xccl_status_t team_create_post(const xccl_team_params_t &tp, TlTeam **team) override
    {
        OobGroup g = make_oob_group(tp, params_.oob);
        if (g.rank < 0 || g.size < 1) return XCCL_ERR_INVALID_PARAM;
        auto         *t  = new HostTeam(tl, g, cfg_);
        xccl_status_t st = t->start();
        if (st != XCCL_OK) {
            delete t;
            return st;
        }
        *team = t;
        return XCCL_OK;
    }

private:
    xccl_context_params_t params_;
    HostCfg               cfg_;
};

class HostLib final : public TeamLib {
public:
    HostLib() : TeamLib(XCCL_TL_UCX, 10)
    {
        caps.coll_types = XCCL_COLL_CAP_BARRIER | XCCL_COLL_CAP_BCAST | XCCL_COLL_CAP_ALLREDUCE | XCCL_COLL_CAP_REDUCE |
                          XCCL_COLL_CAP_ALLTOALL | XCCL_COLL_CAP_ALLTOALLV | XCCL_COLL_CAP_ALLGATHER |
                          XCCL_COLL_CAP_FANIN | XCCL_COLL_CAP_FANOUT | XCCL_COLL_CAP_REDUCE_SCATTER;
        caps.mem_types    = XCCL_BIT(XCCL_MEMORY_TYPE_HOST) | XCCL_BIT(XCCL_MEMORY_TYPE_CUDA);
        caps.reproducible = XCCL_REPRODUCIBILITY_MODE_REPRODUCIBLE | XCCL_REPRODUCIBILITY_MODE_NON_REPRODUCIBLE;
        caps.epilogue     = true;
    }

    std::vector<OptField> context_options() const override
    {
        return {
            {"BLOCK_STREAM", "no", "Hold the caller's CUDA stream until a host-progressed collective finishes", OptType::BOOL},
            {"NET_DEVICES", "all", "Accepted for compatibility; the transport is shared memory", OptType::STRING},
            {"BARRIER_KN_RADIX", "4", "Radix of the k-nomial barrier", OptType::UINT},
            {"BCAST_KN_RADIX", "4", "Radix of the k-nomial broadcast tree", OptType::UINT},
            {"REDUCE_KN_RADIX", "4", "Radix of the k-nomial reduction tree", OptType::UINT},
            {"ALLREDUCE_ALG", "auto", "auto, knomial or sra", OptType::STRING},
            {"ALLREDUCE_KN_RADIX", "4", "Radix of both allreduce algorithms", OptType::UINT},
            {"ALLREDUCE_SRA_THRESH", "4096", "auto: messages of at least this many bytes use sra", OptType::MEMUNITS},
            {"NUM_TO_PROBE", "10", "Transport polls per test call before it reports that the collective is still in progress", OptType::UINT},
            {"ALLTOALL_PAIRWISE_CHUNK", "1", "Exchange steps in flight; 0 = all of them", OptType::UINT},
            {"ALLTOALL_PAIRWISE_REVERSE", "0", "Walk peers in the opposite direction", OptType::BOOL},
            {"ALLTOALL_PAIRWISE_BARRIER", "0", "Insert a barrier every N steps; 0 = never", OptType::UINT},
            {"PRE_MEM_MAP", "0", "Accepted for compatibility; nothing to pre-register", OptType::BOOL},
            {"PPN", "32", "Expected ranks per node (hint only)", OptType::UINT},
            {"RING_SIZE", "1m", "Bytes of the shared-memory ring per peer", OptType::MEMUNITS},
        };
    }

    xccl_status_t context_create(xccl_lib *, const xccl_context_params_t &params, const OptTable &cfg,
                                 TlContext **ctx) override
    {
        HostCfg c;
        c.block_stream    = cfg.flag("BLOCK_STREAM");
        c.barrier_radix   = (int)cfg.num("BARRIER_KN_RADIX");
        c.bcast_radix     = (int)cfg.num("BCAST_KN_RADIX");
        c.reduce_radix    = (int)cfg.num("REDUCE_KN_RADIX");
        c.allreduce_radix = (int)cfg.num("ALLREDUCE_KN_RADIX");
        c.allreduce_alg   = cfg.str("ALLREDUCE_ALG");
        c.sra_threshold   = (size_t)cfg.num("ALLREDUCE_SRA_THRESH");
        c.a2a_chunk       = (int)cfg.num("ALLTOALL_PAIRWISE_CHUNK");
        c.a2a_reverse     = cfg.flag("ALLTOALL_PAIRWISE_REVERSE");
        c.a2a_barrier     = (int)cfg.num("ALLTOALL_PAIRWISE_BARRIER");
        c.ring_bytes      = (size_t)cfg.num("RING_SIZE");
        c.num_to_probe    = (int)cfg.num("NUM_TO_PROBE");
        *ctx              = new HostContext(params, c);
        return XCCL_OK;
    }
};

HostLib          g_host_lib;
TeamLibRegistrar g_host_reg(&g_host_lib);

}  // namespace

}  // namespace host
}  // namespace xccl
