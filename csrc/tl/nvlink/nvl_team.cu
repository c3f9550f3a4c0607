// NVLink team library: the product path for CUDA buffers on one NVSwitch box.
//
// A team owns one symmetric region per rank (signal pad + workspace, optionally bound to an
// NVSwitch multicast object) and serves every collective with the kernels of nvl_kernels.cu,
// launched on the caller's stream (or on an internal one). A request completes when its CUDA
// event does; the kernels' status words, kept in mapped host memory, turn an expired device
// wait into XCCL_ERR_TIMED_OUT and poison the team.
// Allreduce picks one-shot / two-shot / NVLS per message size; the thresholds are options so that
// a measured table can be applied without rebuilding.
#include <cstdlib>
#include <cstring>
#include <map>
#include <string>
#include <vector>

#include "../../core/core.h"
#include "../../cuda/cuda_common.h"
#include "nvl_kernels.cuh"
#include "nvl_shm.h"
#include "nvl_world.h"

namespace xccl {
namespace nvl {

namespace {

constexpr size_t kNever = ~(size_t)0;  // a threshold no message reaches

struct NvlCfg {
    size_t ws_bytes      = 128u << 20;
    bool   nvls          = true;
    size_t one_shot_max  = 128u << 10;
    size_t nvls_min      = 256u << 10;
    size_t bcast_mc_min  = 0;
    size_t bcast_mc_max  = 0;           // 0: by team size
    size_t bcast_mc_chunk = 0;          // 0: one workspace half per step
    size_t direct_min    = ~(size_t)0;  // messages from this size register their buffers and skip the workspace
    bool   direct_min_set = false;      // given explicitly: a tuning file does not override it
    bool   direct        = true;
    bool   direct_cache  = true;        // keep peer mappings of registered buffers until the team goes
    bool   symmetric     = true;        // zero-copy NVLS on buffers from xccl_team_mem_alloc
    size_t symmetric_min = 32u << 10;
    size_t push_max      = 1u << 20;  // allgather / alltoall up to this many bytes per rank use the push form
    std::string tuning_file;
    int    max_blocks    = 64;
    int    threads       = 512;
    double wait_timeout_ms = 5000.0;
    bool   timing        = false;
};

class NvlTeam;

}  // namespace

// Reads the line of a tuning file that matches `team_size` (`team_size one_shot_max nvls_min [direct_min]`, `#`
// starts a comment, -1 keeps the built-in value; the last matching line wins). Returns the number of values set.
extern "C" int xccl_nvlink_tuning_lookup(const char *path, int team_size, long long *one_shot_max, long long *nvls_min,
                                         long long *direct_min)
{
    if (path == nullptr || path[0] == '\0') return 0;
    FILE *f = std::fopen(path, "r");
    if (f == nullptr) return 0;
    char line[256];
    int  set = 0;
    while (std::fgets(line, sizeof(line), f) != nullptr) {
        if (line[0] == '#') continue;
        long long n = 0, a = -1, b = -1, c = -1;
        int       got = std::sscanf(line, "%lld %lld %lld %lld", &n, &a, &b, &c);
        if (got < 3 || n != team_size) continue;
        set = 0;
        if (a >= 0 && one_shot_max != nullptr) { *one_shot_max = a; set++; }
        if (b >= 0 && nvls_min != nullptr) { *nvls_min = b; set++; }
        if (got >= 4 && c >= 0 && direct_min != nullptr) { *direct_min = c; set++; }
    }
    std::fclose(f);
    return set;
}

namespace {

class NvlReq final : public xccl_coll_req {
public:
    NvlReq(NvlTeam *t, const xccl_coll_op_args_t &a) : team_(t), args_(a) {}
    ~NvlReq() override;
    xccl_status_t prepare();
    xccl_status_t post() override;
    xccl_status_t test() override;
    xccl_status_t wait() override;
    xccl_status_t finalize() override { return in_flight_ ? XCCL_INPROGRESS : XCCL_OK; }
    double        elapsed_us() override { return elapsed_us_; }
    bool          in_flight() const { return in_flight_; }
    cudaEvent_t   done_event() const { return done_; }

private:
    xccl_status_t complete();
    bool          push_wanted(int coll, size_t total_bytes) const;
    NvlTeam            *team_;
    xccl_coll_op_args_t args_;
    cudaEvent_t         done_ = nullptr, start_ = nullptr;
    bool                in_flight_ = false;
    xccl_status_t       last_ = XCCL_OK;
    double              elapsed_us_ = -1.0;
    uint32_t           *vmeta_ = nullptr;
    size_t              max_src_bytes_ = 0;
    // direct algorithms: every rank's buffers of this request, mapped here at init
    xccl_status_t       register_buffers(void *src, void *dst, size_t src_bytes, size_t dst_bytes);
    bool                direct_ = false;
    std::vector<std::string> mappings_;  // peer mappings this request holds a count on
    const void         *peer_src_[kMaxRanks] = {nullptr};
    void               *peer_dst_[kMaxRanks] = {nullptr};
    // symmetric algorithms: the buffers lie in memory of xccl_team_mem_alloc; their multicast addresses
    bool                sym_    = false;
    const void         *mc_src_ = nullptr;
    void               *mc_dst_ = nullptr;
};

class NvlTeam final : public TlTeam {
public:
    NvlTeam(TeamLib *tl, const NvlCfg &cfg) : tl_(tl), cfg(cfg) {}
    ~NvlTeam() override
    {
        if (stream != nullptr) {
            cudaStreamSynchronize(stream);
            cudaStreamDestroy(stream);
        }
        // which algorithm served how many posts (log level info): the quickest check of a selection table
        tl_info(tl_, "nvlink team rank %d: allreduce posts one-shot %llu, two-shot %llu, NVLS %llu, direct %llu; other "
                "collectives %llu (direct %llu); on symmetric memory %llu", rank, stats.one_shot, stats.two_shot, stats.nvls,
                stats.direct_allreduce, stats.other, stats.direct_other, stats.symmetric);
        for (auto &kv : ipc_cache) cudaIpcCloseMemHandle(kv.second.ptr);
        for (SymmetricRegion *r : sym_regions) delete r;
        delete region;
        if (status_host != nullptr) cudaFreeHost(status_host);
    }

    // Mapping of a peer's allocation (legacy CUDA IPC), opened once per allocation and counted per request that uses
    // it. With DIRECT_CACHE (default) it is kept until the team goes; without, release_peer closes it with its last user.
    void *open_peer(const cudaIpcMemHandle_t &h, std::vector<std::string> *used)
    {
        std::string key((const char *)&h, sizeof(h));
        auto        it = ipc_cache.find(key);
        if (it == ipc_cache.end()) {
            void *p = nullptr;
            if (cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) {
                (void)cudaGetLastError();
                return nullptr;
            }
            it = ipc_cache.emplace(key, PeerMapping{p, 0}).first;
        }
        it->second.refs++;
        used->push_back(key);
        return it->second.ptr;
    }
    void release_peer(const std::string &key)
    {
        auto it = ipc_cache.find(key);
        if (it == ipc_cache.end() || --it->second.refs > 0 || cfg.direct_cache) return;
        cudaIpcCloseMemHandle(it->second.ptr);
        ipc_cache.erase(it);
    }
    size_t peer_mappings() const { return ipc_cache.size(); }

    xccl_status_t init(const OobGroup &g)
    {
        oob  = g;
        rank = g.rank;
        size = g.size;
        if (size > kMaxRanks) return XCCL_ERR_UNSUPPORTED;
        size_t        total = kPadBytes + cfg.ws_bytes;
        xccl_status_t st    = SymmetricRegion::create(g, total, cfg.nvls, &region);
        if (st != XCCL_OK) return st;
        XCCL_CUDA_CHECK(cudaHostAlloc((void **)&status_host, sizeof(HostStatus), cudaHostAllocMapped));
        std::memset(status_host, 0, sizeof(HostStatus));
        uint32_t *sdev = nullptr;
        XCCL_CUDA_CHECK(cudaHostGetDevicePointer((void **)&sdev, status_host, 0));
        int lo = 0, hi = 0;
        cudaDeviceGetStreamPriorityRange(&lo, &hi);
        XCCL_CUDA_CHECK(cudaStreamCreateWithPriority(&stream, cudaStreamNonBlocking, hi));
        world.size      = size;
        world.rank_base = rank;
        world.n_local   = 1;
        world.ws_bytes  = cfg.ws_bytes;
        world.mc_bcast_cap = cfg.bcast_mc_chunk / 16;
        // crossover points measured on NVSwitch systems: with 8 ranks the one-shot kernel's all-to-all
        // traffic loses to the two-step kernels earlier than with 4 or fewer
        if (!cfg.tuning_file.empty()) {
            // thresholds measured on this machine by `python -m xccl_b200.bench.collectives --table FILE`
            long long a = -1, b = -1, c = -1;
            if (xccl_nvlink_tuning_lookup(cfg.tuning_file.c_str(), size, &a, &b, &c) > 0) {
                if (a >= 0 && cfg.one_shot_max == 0) cfg.one_shot_max = (size_t)a;
                if (b >= 0 && cfg.nvls_min == 0) cfg.nvls_min = (size_t)b;
                if (c >= 0 && !cfg.direct_min_set) cfg.direct_min = (size_t)c;
                tl_info(tl_, "nvlink team: thresholds of %d ranks from %s: one-shot <= %lld, NVLS >= %lld, direct >= %lld",
                        size, cfg.tuning_file.c_str(), a, b, c);
            }
        }
        // Two ranks: a multimem load or store sends the local half through the switch as well, so the in-switch
        // paths move twice the bytes of a plain peer access and lose at every size measured; the one-shot kernel
        // (one flag round trip) wins up to 4 MiB, and from a few MiB a broadcast is faster pulled by its one reader.
        if (cfg.one_shot_max == 0) cfg.one_shot_max = size >= 8 ? (256u << 10) : size == 2 ? (4u << 20) : (1u << 20);
        if (cfg.nvls_min == 0) cfg.nvls_min = size >= 8 ? (1u << 20) : size == 2 ? kNever : (128u << 10);
        if (cfg.bcast_mc_max == 0) cfg.bcast_mc_max = size == 2 ? (1u << 20) : kNever;
        world.wait_budget_ns = (unsigned long long)(cfg.wait_timeout_ms * 1e6);
        for (int p = 0; p < size; p++) {
            world.pad[p] = (uint32_t *)region->base[(size_t)p];
            world.ws[p]  = region->base[(size_t)p] + kPadBytes;
        }
        world.status[0] = sdev;
        world.mc_ws     = region->mc_base != nullptr ? region->mc_base + kPadBytes : nullptr;
        tl_info(tl_, "nvlink team: rank %d/%d, workspace %zu MiB, NVLS %s", rank, size, cfg.ws_bytes >> 20,
                world.mc_ws != nullptr ? "on" : "off");
        return XCCL_OK;
    }

    xccl_status_t create_test() override { return XCCL_OK; }

    // Symmetric allocations (xccl_team_mem_alloc): one more region like the workspace, owned by the caller.
    xccl_status_t sym_alloc(size_t bytes, void **ptr) override
    {
        SymmetricRegion *r  = nullptr;
        xccl_status_t    st = SymmetricRegion::create(oob, bytes, cfg.nvls, &r);
        if (st != XCCL_OK) return st;
        sym_regions.push_back(r);
        *ptr = r->base[(size_t)rank];
        return XCCL_OK;
    }
    xccl_status_t sym_free(void *ptr) override
    {
        for (size_t i = 0; i < sym_regions.size(); i++) {
            if (sym_regions[i]->base[(size_t)rank] == (char *)ptr) {
                if (stream != nullptr) cudaStreamSynchronize(stream);
                cudaDeviceSynchronize();
                // nobody unmaps while a peer may still be inside a collective on this memory
                int              one = 1;
                std::vector<int> all((size_t)size);
                xccl_status_t    st = oob.allgather_blocking(&one, all.data(), sizeof(int));
                delete sym_regions[i];
                sym_regions.erase(sym_regions.begin() + (long)i);
                return st;
            }
        }
        return XCCL_ERR_NO_ELEM;
    }
    // The multicast address of [p, p + bytes) when that range lies inside one symmetric allocation bound to the
    // multicast object; nullptr otherwise.
    char *mc_address(const void *p, size_t bytes) const
    {
        for (const SymmetricRegion *r : sym_regions) {
            const char *b = r->base[(size_t)rank];
            if (r->mc_base != nullptr && (const char *)p >= b && (const char *)p + bytes <= b + r->bytes) {
                return r->mc_base + ((const char *)p - b);
            }
        }
        return nullptr;
    }

    xccl_status_t collective_init(const xccl_coll_op_args_t &args, xccl_memory_type_t, xccl_coll_req **req) override
    {
        auto         *r  = new NvlReq(this, args);
        xccl_status_t st = r->prepare();
        if (st != XCCL_OK) {
            delete r;
            return st;
        }
        *req = r;
        return XCCL_OK;
    }

    TeamLib         *tl_;
    NvlCfg           cfg;
    OobGroup         oob;
    struct PeerMapping {
        void *ptr;
        int   refs;
    };
    std::map<std::string, PeerMapping> ipc_cache;
    std::vector<SymmetricRegion *> sym_regions;
    struct {
        unsigned long long one_shot = 0, two_shot = 0, nvls = 0, direct_allreduce = 0, other = 0, direct_other = 0, symmetric = 0;
    } stats;
    SymmetricRegion *region = nullptr;
    World            world{};
    HostStatus      *status_host = nullptr;
    cudaStream_t     stream = nullptr;
    int              phase  = 0;  // workspace halves consumed so far
    // All requests of the team share the workspace, the signal pads and the epoch counters, so their kernels
    // must run in post order. Posts on one stream are ordered by it; when a post arrives on another stream it
    // first waits for the event of the last post that may still be running.
    NvlReq          *last_req    = nullptr;
    cudaStream_t     last_stream = nullptr;
    xccl_status_t    order_after_last_post(cudaStream_t s);
    void             posted(NvlReq *r, cudaStream_t s)
    {
        last_req    = r;
        last_stream = s;
    }
};

xccl_status_t NvlTeam::order_after_last_post(cudaStream_t s)
{
    if (last_req != nullptr && last_stream != s && last_req->in_flight()) {
        XCCL_CUDA_CHECK(cudaStreamWaitEvent(s, last_req->done_event(), 0));
    }
    return XCCL_OK;
}

NvlReq::~NvlReq()
{
    if (team_->last_req == this) {
        // a request is only finalized when it is no longer in flight, so nothing is left to order after
        team_->last_req = nullptr;
    }
    if (done_ != nullptr) cudaEventDestroy(done_);
    if (start_ != nullptr) cudaEventDestroy(start_);
    if (vmeta_ != nullptr) cudaFree(vmeta_);
    // a finalized request has no kernel in flight: its count on the peers' mappings can go
    for (const std::string &k : mappings_) team_->release_peer(k);
}

xccl_status_t NvlReq::prepare()
{
    const auto &bi = args_.buffer_info;
    const int   n  = team_->size;
    switch (args_.coll_type) {
    case XCCL_ALLREDUCE:
    case XCCL_REDUCE:
    case XCCL_REDUCE_SCATTER:
        if (xccl_dt_size(args_.reduce_info.dt) == 0) return XCCL_ERR_UNSUPPORTED;
        break;
    case XCCL_ALLTOALLV: {
        if (bi.src_counts == nullptr || bi.dst_counts == nullptr || bi.src_displacements == nullptr ||
            bi.dst_displacements == nullptr) {
            return XCCL_ERR_INVALID_PARAM;
        }
        if (bi.src_buffer == XCCL_IN_PLACE || bi.src_buffer == bi.dst_buffer) return XCCL_ERR_UNSUPPORTED;
        if (xccl_dt_size(bi.src_datatype) == 0 || xccl_dt_size(bi.dst_datatype) == 0) return XCCL_ERR_INVALID_PARAM;
        std::vector<uint32_t> meta((size_t)4 * n);
        size_t                total = 0;
        for (int p = 0; p < n; p++) {
            meta[(size_t)p]         = bi.src_counts[p];
            meta[(size_t)n + p]     = bi.src_displacements[p];
            meta[(size_t)2 * n + p] = bi.dst_counts[p];
            meta[(size_t)3 * n + p] = bi.dst_displacements[p];
            total += ((size_t)bi.src_counts[p] * xccl_dt_size(bi.src_datatype) + 15) / 16 * 16;
        }
        max_src_bytes_ = total;
        XCCL_CUDA_CHECK(cudaMalloc((void **)&vmeta_, meta.size() * 4));
        XCCL_CUDA_CHECK(cudaMemcpy(vmeta_, meta.data(), meta.size() * 4, cudaMemcpyHostToDevice));
        break;
    }
    case XCCL_BCAST:
    case XCCL_ALLGATHER:
    case XCCL_ALLTOALL:
    case XCCL_BARRIER:
    case XCCL_FANIN:
    case XCCL_FANOUT: break;
    default: return XCCL_ERR_UNSUPPORTED;
    }
    XCCL_CUDA_CHECK(cudaEventCreateWithFlags(&done_, team_->cfg.timing ? cudaEventDefault : cudaEventDisableTiming));
    if (team_->cfg.timing) XCCL_CUDA_CHECK(cudaEventCreate(&start_));
    // Large messages (or an explicit request for the direct algorithm) register their buffers with the
    // peers now: one out-of-band exchange at init buys posts that never touch the workspace.
    const bool forced = args_.alg.set_by_user && args_.alg.id == ALG_DIRECT;
    size_t     src_bytes = 0, dst_bytes = 0, msg = 0;
    switch (args_.coll_type) {
    case XCCL_ALLREDUCE:
        src_bytes = dst_bytes = msg = args_.reduce_info.count * xccl_dt_size(args_.reduce_info.dt);
        if (args_.field_mask & XCCL_COLL_OP_ARGS_FIELD_EPILOGUE) {
            xccl_dt_t o = args_.epilogue.out_dt;
            if (o != XCCL_DT_UNSUPPORTED && o != XCCL_DT_LAST_PREDEFINED) dst_bytes = args_.reduce_info.count * xccl_dt_size(o);
        }
        break;
    case XCCL_REDUCE_SCATTER: {
        size_t cnt = args_.reduce_info.count;
        if (cnt == 0 && bi.len != 0) cnt = bi.len / xccl_dt_size(args_.reduce_info.dt) / (size_t)n;
        src_bytes = msg = cnt * xccl_dt_size(args_.reduce_info.dt) * (size_t)n;
        dst_bytes = 0;  // written locally only
        break;
    }
    case XCCL_ALLGATHER:
        src_bytes = bi.len / (size_t)n;
        msg       = bi.len;
        break;
    case XCCL_ALLTOALL:
        src_bytes = msg = bi.len * (size_t)n;
        break;
    default: break;
    }
    // Buffers in symmetric memory (same offset on every rank: the caller's contract) need no registration and
    // no workspace: in-switch reduction and multicast act on them directly.
    if (team_->cfg.symmetric && !team_->sym_regions.empty()) {
        void *src = bi.src_buffer, *dst = bi.dst_buffer;
        if (src == XCCL_IN_PLACE || src == nullptr) src = dst;
        const bool same_out = !(args_.field_mask & XCCL_COLL_OP_ARGS_FIELD_EPILOGUE) ||
                              args_.epilogue.out_dt == XCCL_DT_UNSUPPORTED || args_.epilogue.out_dt == XCCL_DT_LAST_PREDEFINED ||
                              args_.epilogue.out_dt == args_.reduce_info.dt;
        if (args_.coll_type == XCCL_ALLREDUCE && same_out && msg != 0 && msg % 16 == 0 &&
            nvls_supported(args_.reduce_info.dt, args_.reduce_info.op) && (((uintptr_t)src | (uintptr_t)dst) & 15) == 0) {
            mc_src_ = team_->mc_address(src, msg);
            mc_dst_ = team_->mc_address(dst, msg);
            sym_    = mc_src_ != nullptr && mc_dst_ != nullptr;
        } else if (args_.coll_type == XCCL_BCAST && bi.len != 0 && bi.len % 16 == 0 && (((uintptr_t)src | (uintptr_t)dst) & 15) == 0) {
            mc_dst_ = team_->mc_address(dst, bi.len);
            sym_    = mc_dst_ != nullptr;
        }
        if (sym_) return XCCL_OK;
    }
    if (args_.alg.set_by_user && args_.alg.id == ALG_SYMMETRIC) return XCCL_ERR_INVALID_PARAM;  // not symmetric memory
    if (msg != 0 && team_->cfg.direct && (forced || msg >= team_->cfg.direct_min)) {
        void *src = bi.src_buffer, *dst = bi.dst_buffer;
        if (src == XCCL_IN_PLACE || src == nullptr) {
            src = dst;
            if (args_.coll_type == XCCL_ALLGATHER) src = (char *)dst + (size_t)team_->rank * (bi.len / (size_t)n);
        }
        xccl_status_t st = register_buffers(src, dst, src_bytes, dst_bytes);
        if (st != XCCL_OK) return st;
    }
    return XCCL_OK;
}

// Collective over the team (every member calls collective_init in the same order): exchanges CUDA IPC
// handles of the allocations that hold src and dst, maps the peers', and agrees on whether all succeeded.
xccl_status_t NvlReq::register_buffers(void *src, void *dst, size_t src_bytes, size_t dst_bytes)
{
    struct Info {
        cudaIpcMemHandle_t src_h, dst_h;
        size_t             src_off, dst_off;
        int                src_ok, dst_ok;
    };
    const int n = team_->size;
    XCCL_DRIVER_FN(cuMemGetAddressRange);
    auto describe = [&](void *p, size_t bytes, cudaIpcMemHandle_t *h, size_t *off) -> int {
        if (p == nullptr || bytes == 0) return 0;
        CUdeviceptr base = 0;
        size_t      size = 0;
        if (cuMemGetAddressRange(&base, &size, (CUdeviceptr)p) != CUDA_SUCCESS) return 0;
        if ((CUdeviceptr)p + bytes > base + size) return 0;
        if (cudaIpcGetMemHandle(h, (void *)base) != cudaSuccess) {
            (void)cudaGetLastError();
            return 0;
        }
        *off = (size_t)((CUdeviceptr)p - base);
        return 1;
    };
    Info mine{};
    mine.src_ok = describe(src, src_bytes, &mine.src_h, &mine.src_off);
    mine.dst_ok = dst_bytes != 0 ? describe(dst, dst_bytes, &mine.dst_h, &mine.dst_off) : 1;
    std::vector<Info> all((size_t)n);
    xccl_status_t     st = team_->oob.allgather_blocking(&mine, all.data(), sizeof(Info));
    if (st != XCCL_OK) return st;
    int ok = 1;
    for (int p = 0; p < n && ok; p++) ok = all[(size_t)p].src_ok && all[(size_t)p].dst_ok;
    for (int p = 0; p < n && ok; p++) {
        if (p == team_->rank) {
            peer_src_[p] = src;
            peer_dst_[p] = dst;
            continue;
        }
        char *ms = (char *)team_->open_peer(all[(size_t)p].src_h, &mappings_);
        if (ms == nullptr) {
            ok = 0;
            break;
        }
        peer_src_[p] = ms + all[(size_t)p].src_off;
        if (dst_bytes != 0) {
            char *md = (char *)team_->open_peer(all[(size_t)p].dst_h, &mappings_);
            if (md == nullptr) {
                ok = 0;
                break;
            }
            peer_dst_[p] = md + all[(size_t)p].dst_off;
        }
    }
    // one rank that could not map a peer sends everybody back to the staged kernels
    std::vector<int> oks((size_t)n);
    st = team_->oob.allgather_blocking(&ok, oks.data(), sizeof(int));
    if (st != XCCL_OK) return st;
    for (int p = 0; p < n; p++) ok = ok && oks[(size_t)p];
    direct_ = ok != 0;
    if (!direct_) tl_debug(team_->tl_, "nvlink: buffers of this request could not be registered, staging through the workspace");
    return XCCL_OK;
}

// allgather / alltoall: the push form when asked for (alg one-shot), never when the pull form is asked for (alg
// two-shot), otherwise up to PUSH_MAX bytes per rank; always only when the exchange fits one workspace half.
bool NvlReq::push_wanted(int coll, size_t total_bytes) const
{
    const size_t len = args_.buffer_info.len;
    if (!push_fits(team_->world, coll, len)) return false;
    if (args_.alg.set_by_user && args_.alg.id == ALG_ONE_SHOT) return true;
    if (args_.alg.set_by_user && args_.alg.id == ALG_TWO_SHOT) return false;
    return total_bytes <= team_->cfg.push_max;
}

xccl_status_t NvlReq::post()
{
    // A request that is still in flight may be posted again: posts of one request are ordered by its stream, and
    // test / wait then refer to the latest post (the reference's NCCL team behaves the same way).
    if (team_->poisoned) return XCCL_ERR_NO_PROGRESS;
    const auto  &bi = args_.buffer_info;
    cudaStream_t s  = team_->stream;
    if ((args_.field_mask & XCCL_COLL_OP_ARGS_FIELD_STREAM) && args_.stream.stream != nullptr) {
        s = *(cudaStream_t *)args_.stream.stream;
    }
    const World &w = team_->world;
    Call         c{};
    void        *src = bi.src_buffer, *dst = bi.dst_buffer;
    bool         sync_only = (args_.coll_type == XCCL_BARRIER || args_.coll_type == XCCL_FANIN || args_.coll_type == XCCL_FANOUT);
    if (!sync_only && (src == XCCL_IN_PLACE || src == nullptr)) {
        src = dst;
        if (args_.coll_type == XCCL_ALLGATHER) src = (char *)dst + (size_t)team_->rank * (bi.len / (size_t)team_->size);
    }
    c.src[0]   = src;
    c.dst[0]   = dst;
    c.vmeta[0] = vmeta_;
    c.count    = args_.reduce_info.count;
    c.len      = bi.len;
    c.op       = (int)args_.reduce_info.op;
    c.root     = args_.root;
    c.scale    = 1.0f;
    xccl_dt_t out_dt = XCCL_DT_UNSUPPORTED;
    if (args_.field_mask & XCCL_COLL_OP_ARGS_FIELD_EPILOGUE) {
        c.scale = args_.epilogue.scale;
        out_dt  = args_.epilogue.out_dt;
    }
    c.do_scale = (c.scale != 1.0f);
    c.parity   = team_->phase & 1;
    LaunchCfg cfg;
    cfg.threads    = team_->cfg.threads;
    cfg.max_blocks = team_->cfg.max_blocks;
    const xccl_dt_t dt = args_.reduce_info.dt;
    xccl_status_t st = team_->order_after_last_post(s);
    if (st != XCCL_OK) return st;
    if (start_ != nullptr) XCCL_CUDA_CHECK(cudaEventRecord(start_, s));
    if (sym_) {
        const size_t bytes = args_.coll_type == XCCL_BCAST ? c.len : c.count * xccl_dt_size(dt);
        const bool   user  = args_.alg.set_by_user && args_.alg.id != ALG_AUTO;
        // Asked for by name: always. Asked for NVLS (the in-switch path, e.g. by the sharp / hmc team libraries):
        // zero-copy from the threshold on, staged below it. Not asked for anything: additionally, small reductions
        // stay with the one-shot kernel (one flag round trip instead of two barriers).
        bool take;
        if (user) {
            take = args_.alg.id == ALG_SYMMETRIC || (args_.alg.id == ALG_NVLS && bytes >= team_->cfg.symmetric_min);
        } else {
            take = bytes >= team_->cfg.symmetric_min &&
                   (args_.coll_type == XCCL_BCAST ? bytes <= team_->cfg.bcast_mc_max
                                                  : bytes > team_->cfg.one_shot_max && team_->cfg.nvls_min != kNever);
        }
        if (take) {
            c.mc_src[0] = mc_src_;
            c.mc_dst[0] = mc_dst_;
            st          = launch_symmetric(w, c, (int)args_.coll_type, dt, cfg, s);
            if (st != XCCL_OK) return st;
            team_->stats.symmetric++;
            XCCL_CUDA_CHECK(cudaEventRecord(done_, s));
            in_flight_ = true;
            team_->posted(this, s);
            return XCCL_OK;
        }
    }
    if (direct_) {
        for (int p = 0; p < team_->size; p++) {
            c.peer_src[p] = peer_src_[p];
            c.peer_dst[p] = peer_dst_[p];
        }
        if (args_.coll_type == XCCL_REDUCE_SCATTER && c.count == 0 && c.len != 0) {
            c.count = c.len / xccl_dt_size(dt) / (size_t)team_->size;
        }
        if (direct_shape_ok((int)args_.coll_type, c, dt, team_->size)) {
            st = launch_direct(w, c, (int)args_.coll_type, dt, out_dt, cfg, s);
            if (st == XCCL_OK) {
                (args_.coll_type == XCCL_ALLREDUCE ? team_->stats.direct_allreduce : team_->stats.direct_other)++;
                XCCL_CUDA_CHECK(cudaEventRecord(done_, s));
                in_flight_ = true;
                team_->posted(this, s);
                return XCCL_OK;
            }
            if (st != XCCL_ERR_UNSUPPORTED) return st;
        }
        direct_ = false;  // shape or type outside the direct kernels: same answer on every rank
    }
    switch (args_.coll_type) {
    case XCCL_ALLREDUCE: {
        const size_t bytes = c.count * xccl_dt_size(dt);
        Alg          alg   = ALG_AUTO;
        if (args_.alg.set_by_user) alg = (Alg)args_.alg.id;
        if (alg == ALG_AUTO) {
            if (bytes <= team_->cfg.one_shot_max && bytes + 16 <= one_shot_limit(w)) {
                alg = ALG_ONE_SHOT;
            } else if (w.mc_ws != nullptr && nvls_supported(dt, (xccl_op_t)c.op) && bytes >= team_->cfg.nvls_min) {
                alg = ALG_NVLS;
            } else {
                alg = ALG_TWO_SHOT;
            }
        }
        st = launch_allreduce(w, c, dt, out_dt, alg, cfg, s);
        (alg == ALG_ONE_SHOT ? team_->stats.one_shot : alg == ALG_NVLS ? team_->stats.nvls : team_->stats.two_shot)++;
        team_->phase += (alg == ALG_ONE_SHOT) ? 1 : chunks_used(w, XCCL_ALLREDUCE, c.count, c.len, dt);
        break;
    }
    case XCCL_REDUCE: {
        // in-switch reduction at the root: asked for by name, or from the size where NVLS wins for allreduce
        const bool can  = w.mc_ws != nullptr && nvls_supported(dt, (xccl_op_t)c.op);
        const bool nvls = can && (args_.alg.set_by_user ? args_.alg.id == ALG_NVLS
                                                        : c.count * xccl_dt_size(dt) >= team_->cfg.nvls_min);
        st = launch_reduce(w, c, dt, out_dt, cfg, s, nvls);
        if (nvls) team_->stats.nvls++;
        team_->phase += chunks_used(w, XCCL_REDUCE, c.count, c.len, dt);
        break;
    }
    case XCCL_REDUCE_SCATTER:
        if (c.count == 0 && c.len != 0) c.count = c.len / xccl_dt_size(dt) / (size_t)team_->size;
        st = launch_reduce_scatter(w, c, dt, out_dt, cfg, s,
                                   args_.alg.set_by_user && args_.alg.id == ALG_NVLS && w.mc_ws != nullptr &&
                                       nvls_supported(dt, (xccl_op_t)c.op));
        team_->phase += chunks_used(w, XCCL_REDUCE_SCATTER, c.count, c.len, dt);
        break;
    case XCCL_BCAST: {
        bool mc = w.mc_ws != nullptr && c.len >= team_->cfg.bcast_mc_min && c.len <= team_->cfg.bcast_mc_max;
        if (args_.alg.set_by_user) mc = (args_.alg.id == ALG_NVLS);
        st = launch_bcast(w, c, cfg, s, mc);
        team_->phase += chunks_used(w, XCCL_BCAST, c.count, c.len, dt, mc);
        break;
    }
    case XCCL_ALLGATHER:
        c.push = push_wanted(XCCL_ALLGATHER, c.len) ? 1 : 0;
        st = launch_allgather(w, c, cfg, s);
        team_->phase += chunks_used(w, XCCL_ALLGATHER, c.count, c.len, dt);
        break;
    case XCCL_ALLTOALL:
        c.push = push_wanted(XCCL_ALLTOALL, c.len * (size_t)team_->size) ? 1 : 0;
        st = launch_alltoall(w, c, cfg, s);
        team_->phase += chunks_used(w, XCCL_ALLTOALL, c.count, c.len, dt);
        break;
    case XCCL_ALLTOALLV:
        c.src_es = (int)xccl_dt_size(bi.src_datatype);
        c.dst_es = (int)xccl_dt_size(bi.dst_datatype);
        st       = launch_alltoallv(w, c, max_src_bytes_, cfg, s);
        team_->phase += 1;
        break;
    default: st = launch_sync(w, c, (int)args_.coll_type, cfg, s); break;
    }
    if (st != XCCL_OK) return st;
    if (args_.coll_type != XCCL_ALLREDUCE) team_->stats.other++;
    XCCL_CUDA_CHECK(cudaEventRecord(done_, s));
    in_flight_ = true;
    team_->posted(this, s);
    return XCCL_OK;
}

xccl_status_t NvlReq::complete()
{
    in_flight_ = false;
    last_      = XCCL_OK;
    if (team_->status_host->code != NVL_OK) {
        tl_error(team_->tl_, "nvlink: device wait expired (code %u, rank %u waiting for rank %u, epoch %u)",
                 team_->status_host->code, team_->status_host->rank, team_->status_host->peer,
                 team_->status_host->epoch);
        team_->poisoned = true;
        last_           = XCCL_ERR_TIMED_OUT;
    }
    if (start_ != nullptr) {
        float ms = 0;
        if (cudaEventElapsedTime(&ms, start_, done_) == cudaSuccess) elapsed_us_ = (double)ms * 1000.0;
    }
    return last_;
}

xccl_status_t NvlReq::test()
{
    if (!in_flight_) return last_;
    cudaError_t e = cudaEventQuery(done_);
    if (e == cudaErrorNotReady) return XCCL_INPROGRESS;
    if (e != cudaSuccess) {
        in_flight_ = false;
        last_      = cuda_status(e);
        return last_;
    }
    return complete();
}

xccl_status_t NvlReq::wait()
{
    if (!in_flight_) return last_;
    cudaError_t e = cudaEventSynchronize(done_);
    if (e != cudaSuccess) {
        in_flight_ = false;
        last_      = cuda_status(e);
        return last_;
    }
    return complete();
}

class NvlContext final : public TlContext {
public:
    NvlContext(const xccl_context_params_t &p, const NvlCfg &c) : params_(p), cfg_(c) {}
    xccl_status_t team_create_post(const xccl_team_params_t &tp, TlTeam **team) override
    {
        OobGroup g = make_oob_group(tp, params_.oob);
        if (g.rank < 0 || g.size < 1) return XCCL_ERR_INVALID_PARAM;
        auto         *t  = new NvlTeam(tl, cfg_);
        xccl_status_t st = t->init(g);
        if (st != XCCL_OK) {
            delete t;
            return st;
        }
        *team = t;
        return XCCL_OK;
    }

private:
    xccl_context_params_t params_;
    NvlCfg                cfg_;
};

class NvlLib final : public TeamLib {
public:
    NvlLib() : TeamLib(XCCL_TL_NVLINK, 120)
    {
        caps.coll_types = XCCL_COLL_CAP_BARRIER | XCCL_COLL_CAP_BCAST | XCCL_COLL_CAP_ALLREDUCE | XCCL_COLL_CAP_REDUCE |
                          XCCL_COLL_CAP_ALLTOALL | XCCL_COLL_CAP_ALLTOALLV | XCCL_COLL_CAP_ALLGATHER |
                          XCCL_COLL_CAP_FANIN | XCCL_COLL_CAP_FANOUT | XCCL_COLL_CAP_REDUCE_SCATTER;
        caps.mem_types      = XCCL_BIT(XCCL_MEMORY_TYPE_CUDA);
        caps.sync_mem_types = XCCL_BIT(XCCL_MEMORY_TYPE_HOST);
        caps.team_usage     = XCCL_LIB_PARAMS_TEAM_USAGE_HW_COLLECTIVES | XCCL_LIB_PARAMS_TEAM_USAGE_SW_COLLECTIVES;
        caps.reproducible   = XCCL_REPRODUCIBILITY_MODE_REPRODUCIBLE | XCCL_REPRODUCIBILITY_MODE_NON_REPRODUCIBLE;
        caps.epilogue       = true;  // fused into the kernels' last pass
    }

    xccl_status_t open() override { return cuda_available() ? XCCL_OK : XCCL_ERR_NO_RESOURCE; }

    std::vector<OptField> context_options() const override
    {
        return {
            {"WORKSPACE_SIZE", "128m", "Bytes of symmetric workspace per rank (two alternating halves)", OptType::MEMUNITS},
            {"NVLS", "try", "Bind the workspace to an NVSwitch multicast object and use multimem kernels", OptType::TERNARY},
            {"ONE_SHOT_MAX", "0", "Allreduce messages up to this size use the one-shot kernel (0: by team size, 256k from 8 ranks, 4m with 2, else 1m)", OptType::MEMUNITS},
            {"NVLS_MIN", "0", "Allreduce messages from this size use NVLS when available (0: by team size, 1m from 8 ranks, never with 2, else 128k)", OptType::MEMUNITS},
            {"BCAST_MC_CHUNK", "0", "Multicast broadcasts move this many bytes per step, copy-out overlapping the next push (0: a workspace half)", OptType::MEMUNITS},
            {"BCAST_MC_MIN", "0", "Broadcasts from this size go through the NVSwitch multicast mapping when available", OptType::MEMUNITS},
            {"BCAST_MC_MAX", "0", "Broadcasts above this size are pulled from the root's workspace instead (0: by team size, 1m with 2 ranks, else no limit)", OptType::MEMUNITS},
            {"DIRECT", "y", "Register the buffers of large messages with the peers (CUDA IPC) and run zero-copy kernels on them", OptType::BOOL},
            {"DIRECT_CACHE", "y", "Keep the peers' mappings of registered buffers until the team is destroyed (a registration cache); n: a mapping is closed when the last request that uses it is finalized, after which its owner may free the buffer", OptType::BOOL},
            {"DIRECT_MIN", "0", "Messages from this size register their buffers and use the direct (zero-copy) kernels (0: from the tuning file, else only on request; measured crossover 32m-256m)", OptType::MEMUNITS},
            {"PUSH_MAX", "1m", "Allgather / alltoall messages up to this size (bytes per rank) store into the destinations' workspaces instead of being pulled", OptType::MEMUNITS},
            {"SYMMETRIC", "y", "Run collectives whose buffers come from xccl_team_mem_alloc zero-copy through the multicast mapping", OptType::BOOL},
            {"SYMMETRIC_MIN", "32k", "Smallest message that takes the symmetric (zero-copy NVLS) path", OptType::MEMUNITS},
            {"TUNING_FILE", "", "Measured thresholds, lines of `team_size one_shot_max nvls_min direct_min` (see bench/collectives.py --table)", OptType::STRING},
            {"MAX_BLOCKS", "128", "Upper bound of thread blocks per collective kernel (at most 128)", OptType::UINT},
            {"THREADS", "512", "Threads per block of the collective kernels", OptType::UINT},
            {"WAIT_TIMEOUT_MS", "5000", "Budget of every device-side wait for a peer", OptType::DOUBLE},
            {"TIMING", "no", "Record CUDA events around each collective (xccl_collective_elapsed_us)", OptType::BOOL},
        };
    }

    xccl_status_t query(xccl_tl_attr_t *attr) override
    {
        TeamLib::query(attr);
        if (attr->field_mask & XCCL_TL_ATTR_FIELD_DEVICES_COUNT) {
            int n = 0;
            if (cudaGetDeviceCount(&n) != cudaSuccess) n = 0;
            attr->devices_count = n;
        }
        return XCCL_OK;
    }

    xccl_status_t context_create(xccl_lib *, const xccl_context_params_t &params, const OptTable &cfg,
                                 TlContext **ctx) override
    {
        if (!cuda_available()) return XCCL_ERR_NO_RESOURCE;
        if (!(params.field_mask & XCCL_CONTEXT_PARAM_FIELD_OOB)) {
            // teams may still bring their own OOB; nothing to check here
        }
        NvlCfg c;
        c.ws_bytes        = ((size_t)cfg.num("WORKSPACE_SIZE") + 4095) & ~(size_t)4095;
        c.nvls            = cfg.flag("NVLS");
        c.one_shot_max    = (size_t)cfg.num("ONE_SHOT_MAX");
        c.nvls_min        = (size_t)cfg.num("NVLS_MIN");
        c.bcast_mc_min    = (size_t)cfg.num("BCAST_MC_MIN");
        c.bcast_mc_max    = (size_t)cfg.num("BCAST_MC_MAX");
        c.bcast_mc_chunk  = (size_t)cfg.num("BCAST_MC_CHUNK");
        c.direct_min      = (size_t)cfg.num("DIRECT_MIN");
        c.direct_min_set  = c.direct_min != 0;
        // Not given: registration happens only on request (XCCL_NVLINK_ALG_DIRECT) or from a tuning file. Registered
        // buffers must stay allocated while the team lives (the peers keep the allocation mapped), which a
        // caller has to know about - the same contract as explicit buffer registration in other libraries.
        if (!c.direct_min_set) c.direct_min = ~(size_t)0;
        c.tuning_file     = cfg.str("TUNING_FILE");
        c.direct          = cfg.flag("DIRECT");
        c.direct_cache    = cfg.flag("DIRECT_CACHE");
        c.push_max        = (size_t)cfg.num("PUSH_MAX");
        c.symmetric       = cfg.flag("SYMMETRIC");
        c.symmetric_min   = (size_t)cfg.num("SYMMETRIC_MIN");
        c.max_blocks      = std::max(1, std::min((int)cfg.num("MAX_BLOCKS"), kMaxBlocks));
        c.threads         = std::max(32, std::min((int)cfg.num("THREADS"), 512)) / 32 * 32;
        c.wait_timeout_ms = cfg.real("WAIT_TIMEOUT_MS");
        c.timing          = cfg.flag("TIMING");
        *ctx              = new NvlContext(params, c);
        return XCCL_OK;
    }
};

NvlLib           g_nvl_lib;
TeamLibRegistrar g_nvl_reg(&g_nvl_lib);

}  // namespace

// Peer mappings (registered buffers of other ranks, one per allocation) that the NVLink part of `team` holds right
// now; -1 when the team has none. With DIRECT_CACHE=n it falls back to 0 once the requests that registered buffers
// have been finalized.
extern "C" int xccl_nvlink_peer_mappings(xccl_team_h team)
{
    if (team == nullptr) return -1;
    for (auto &t : team->tl_teams) {
        if (auto *n = dynamic_cast<NvlTeam *>(t.get())) return (int)n->peer_mappings();
    }
    return -1;
}

}  // namespace nvl
}  // namespace xccl
