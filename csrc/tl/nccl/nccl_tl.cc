// NCCL team library: library calls issued the way the reference's NCCL team issues them
// (src/team_lib/nccl/xccl_nccl_collective.c:40-231, src/team_lib/nccl/xccl_nccl_lib.c:169-350).
// It is the baseline the NVLink team is measured against and the carrier of pipeline-parallel
// send/recv. The NCCL library is opened at run time so that the core has no link dependency.
#include <cuda_runtime.h>
#include <dlfcn.h>
#include <nccl.h>

#include <algorithm>
#include <cstdlib>
#include <cstring>
#include <mutex>

#include "../../core/core.h"
#include "../../cuda/cuda_common.h"
#include "../../cuda/mem_cuda.h"
#include "../../utils/mem.h"
#include "nccl_tl.h"

namespace xccl {
namespace nccltl {

namespace {

struct Api {
    void *handle = nullptr;
    decltype(&::ncclGetUniqueId)   GetUniqueId   = nullptr;
    decltype(&::ncclCommInitRank)  CommInitRank  = nullptr;
    decltype(&::ncclCommDestroy)   CommDestroy   = nullptr;
    decltype(&::ncclGetErrorString) GetErrorString = nullptr;
    decltype(&::ncclAllReduce)     AllReduce     = nullptr;
    decltype(&::ncclReduce)        Reduce        = nullptr;
    decltype(&::ncclReduceScatter) ReduceScatter = nullptr;
    decltype(&::ncclBroadcast)     Broadcast     = nullptr;
    decltype(&::ncclAllGather)     AllGather     = nullptr;
    decltype(&::ncclSend)          Send          = nullptr;
    decltype(&::ncclRecv)          Recv          = nullptr;
    decltype(&::ncclGroupStart)    GroupStart    = nullptr;
    decltype(&::ncclGroupEnd)      GroupEnd      = nullptr;
    decltype(&::ncclGetVersion)    GetVersion    = nullptr;
    bool ok = false;
};

Api &api()
{
    static Api a = [] {
        Api         x;
        const char *over = std::getenv("XCCL_TEAM_NCCL_LIB");
        const char *names[] = {over, "libnccl.so.2", "libnccl.so"};
        for (const char *n : names) {
            if (n == nullptr) continue;
            x.handle = dlopen(n, RTLD_NOW | RTLD_GLOBAL);
            if (x.handle != nullptr) break;
        }
        if (x.handle == nullptr) return x;
#define LOAD(sym) x.sym = reinterpret_cast<decltype(x.sym)>(dlsym(x.handle, "nccl" #sym))
        LOAD(GetUniqueId); LOAD(CommInitRank); LOAD(CommDestroy); LOAD(GetErrorString); LOAD(AllReduce); LOAD(Reduce);
        LOAD(ReduceScatter); LOAD(Broadcast); LOAD(AllGather); LOAD(Send); LOAD(Recv); LOAD(GroupStart); LOAD(GroupEnd);
        LOAD(GetVersion);
#undef LOAD
        x.ok = x.GetUniqueId && x.CommInitRank && x.CommDestroy && x.AllReduce && x.Broadcast && x.AllGather && x.Send &&
               x.Recv && x.GroupStart && x.GroupEnd && x.Reduce && x.ReduceScatter;
        return x;
    }();
    return a;
}

bool to_nccl_dt(xccl_dt_t dt, ncclDataType_t *out)
{
    switch (dt) {
    case XCCL_DT_INT8: *out = ncclInt8; return true;
    case XCCL_DT_INT32: *out = ncclInt32; return true;
    case XCCL_DT_INT64: *out = ncclInt64; return true;
    case XCCL_DT_UINT8: *out = ncclUint8; return true;
    case XCCL_DT_UINT32: *out = ncclUint32; return true;
    case XCCL_DT_UINT64: *out = ncclUint64; return true;
    case XCCL_DT_FLOAT16: *out = ncclFloat16; return true;
    case XCCL_DT_FLOAT32: *out = ncclFloat32; return true;
    case XCCL_DT_FLOAT64: *out = ncclFloat64; return true;
    case XCCL_DT_BFLOAT16: *out = ncclBfloat16; return true;
    default: return false;
    }
}

bool to_nccl_op(xccl_op_t op, ncclRedOp_t *out)
{
    switch (op) {
    case XCCL_OP_SUM: *out = ncclSum; return true;
    case XCCL_OP_PROD: *out = ncclProd; return true;
    case XCCL_OP_MAX: *out = ncclMax; return true;
    case XCCL_OP_MIN: *out = ncclMin; return true;
    default: return false;
    }
}

#define NCCL_TRY(tl, expr)                                                                             \
    do {                                                                                               \
        ncclResult_t _r = (expr);                                                                      \
        if (_r != ncclSuccess) {                                                                       \
            tl_error(tl, "%s failed: %s", #expr, api().GetErrorString ? api().GetErrorString(_r) : "?"); \
            return XCCL_ERR_NO_MESSAGE;                                                                \
        }                                                                                              \
    } while (0)

class NcclTeam;

class NcclReq final : public xccl_coll_req {
public:
    NcclReq(NcclTeam *t, const xccl_coll_op_args_t &a) : team_(t), args_(a) {}
    ~NcclReq() override
    {
        if (done_ != nullptr) cudaEventDestroy(done_);
        if (start_ != nullptr) cudaEventDestroy(start_);
        if (epi_tmp_ != nullptr) cuda_free(epi_tmp_);
    }
    xccl_status_t prepare();
    xccl_status_t post() override;
    xccl_status_t test() override
    {
        if (!in_flight_) return last_;
        cudaError_t e = cudaEventQuery(done_);
        if (e == cudaErrorNotReady) return XCCL_INPROGRESS;
        return finish(e);
    }
    xccl_status_t wait() override
    {
        if (!in_flight_) return last_;
        return finish(cudaEventSynchronize(done_));
    }
    xccl_status_t finalize() override { return in_flight_ ? XCCL_INPROGRESS : XCCL_OK; }
    double        elapsed_us() override { return elapsed_us_; }

private:
    xccl_status_t finish(cudaError_t e)
    {
        in_flight_ = false;
        last_      = cuda_status(e);
        if (start_ != nullptr && e == cudaSuccess) {
            float ms = 0;
            if (cudaEventElapsedTime(&ms, start_, done_) == cudaSuccess) elapsed_us_ = ms * 1000.0;
        }
        return last_;
    }
    xccl_status_t start(cudaStream_t s);
    NcclTeam           *team_;
    xccl_coll_op_args_t args_;
    std::vector<uint32_t> sc_, sd_, dc_, dd_;
    cudaEvent_t         done_ = nullptr, start_ = nullptr;
    bool                in_flight_ = false;
    xccl_status_t       last_ = XCCL_OK;
    double              elapsed_us_ = -1.0;
    // scale / cast epilogue: NCCL reduces in the input datatype (into epi_tmp_ when the output datatype
    // differs, so that it never writes count * sizeof(dt) bytes into a destination sized for out_dt), then
    // one kernel on the same stream scales and converts into dst
    bool      epi_       = false;
    void     *epi_tmp_   = nullptr;
    size_t    epi_count_ = 0;
    xccl_dt_t epi_out_   = XCCL_DT_UNSUPPORTED;
};

class NcclTeam final : public TlTeam {
public:
    NcclTeam(TeamLib *tl, bool timing) : tl_(tl), timing(timing) {}
    ~NcclTeam() override
    {
        if (stream != nullptr) {
            cudaStreamSynchronize(stream);
            cudaStreamDestroy(stream);
        }
        if (comm != nullptr) api().CommDestroy(comm);
    }
    xccl_status_t init(const OobGroup &g)
    {
        rank = g.rank;
        size = g.size;
        ncclUniqueId id{};
        if (rank == 0) NCCL_TRY(tl_, api().GetUniqueId(&id));
        std::vector<ncclUniqueId> ids((size_t)size);
        xccl_status_t             st = g.allgather_blocking(&id, ids.data(), sizeof(id));
        if (st != XCCL_OK) return st;
        NCCL_TRY(tl_, api().CommInitRank(&comm, size, ids[0], rank));
        int lo = 0, hi = 0;
        cudaDeviceGetStreamPriorityRange(&lo, &hi);
        XCCL_CUDA_CHECK(cudaStreamCreateWithPriority(&stream, cudaStreamNonBlocking, hi));
        return XCCL_OK;
    }
    xccl_status_t create_test() override { return XCCL_OK; }
    xccl_status_t collective_init(const xccl_coll_op_args_t &args, xccl_memory_type_t, xccl_coll_req **req) override
    {
        auto         *r  = new NcclReq(this, args);
        xccl_status_t st = r->prepare();
        if (st != XCCL_OK) {
            delete r;
            return st;
        }
        *req = r;
        return XCCL_OK;
    }
    TeamLib     *tl_;
    bool         timing;
    ncclComm_t   comm   = nullptr;
    cudaStream_t stream = nullptr;
};

xccl_status_t NcclReq::prepare()
{
    const auto    &bi = args_.buffer_info;
    ncclDataType_t dt;
    ncclRedOp_t    op;
    switch (args_.coll_type) {
    case XCCL_ALLREDUCE:
    case XCCL_REDUCE:
    case XCCL_REDUCE_SCATTER:
        if (!to_nccl_dt(args_.reduce_info.dt, &dt) || !to_nccl_op(args_.reduce_info.op, &op)) return XCCL_ERR_UNSUPPORTED;
        if (args_.field_mask & XCCL_COLL_OP_ARGS_FIELD_EPILOGUE) {
            const xccl_dt_t in = args_.reduce_info.dt;
            epi_out_           = args_.epilogue.out_dt;
            if (epi_out_ == XCCL_DT_UNSUPPORTED || epi_out_ == XCCL_DT_LAST_PREDEFINED) epi_out_ = in;
            epi_       = (args_.epilogue.scale != 1.0f) || (epi_out_ != in);
            epi_count_ = args_.reduce_info.count;
            if (epi_count_ == 0) {
                epi_count_ = bi.len / xccl_dt_size(in) / (args_.coll_type == XCCL_REDUCE_SCATTER ? (size_t)team_->size : 1);
            }
            if (args_.coll_type == XCCL_REDUCE && args_.root != team_->rank) epi_ = false;  // no result here
            if (epi_) {
                char pin[16] = {0}, pout[16] = {0};
                if (host_scale_cast(pin, in, pout, epi_out_, 1, 1.0f) != XCCL_OK) return XCCL_ERR_UNSUPPORTED;
                if (epi_out_ != in) {
                    xccl_status_t st = cuda_alloc(&epi_tmp_, std::max<size_t>(epi_count_ * xccl_dt_size(in), 16));
                    if (st != XCCL_OK) return st;
                }
            }
        }
        break;
    case XCCL_ALLTOALLV:
        if (bi.src_counts == nullptr || bi.dst_counts == nullptr || bi.src_displacements == nullptr ||
            bi.dst_displacements == nullptr) {
            return XCCL_ERR_INVALID_PARAM;
        }
        sc_.assign(bi.src_counts, bi.src_counts + team_->size);
        sd_.assign(bi.src_displacements, bi.src_displacements + team_->size);
        dc_.assign(bi.dst_counts, bi.dst_counts + team_->size);
        dd_.assign(bi.dst_displacements, bi.dst_displacements + team_->size);
        break;
    case XCCL_ALLTOALL:
    case XCCL_ALLGATHER:
    case XCCL_BCAST: break;
    default: return XCCL_ERR_UNSUPPORTED;
    }
    XCCL_CUDA_CHECK(cudaEventCreateWithFlags(&done_, team_->timing ? cudaEventDefault : cudaEventDisableTiming));
    if (team_->timing) XCCL_CUDA_CHECK(cudaEventCreate(&start_));
    return XCCL_OK;
}

xccl_status_t NcclReq::start(cudaStream_t s)
{
    const auto &bi   = args_.buffer_info;
    const int   n    = team_->size;
    ncclComm_t  comm = team_->comm;
    void       *src = bi.src_buffer, *dst = bi.dst_buffer;
    if (src == XCCL_IN_PLACE || src == nullptr) src = dst;
    void *const user_dst = dst;
    if (epi_tmp_ != nullptr) dst = epi_tmp_;
    ncclDataType_t dt = ncclChar;
    ncclRedOp_t    op = ncclSum;
    switch (args_.coll_type) {
    case XCCL_ALLREDUCE:
        to_nccl_dt(args_.reduce_info.dt, &dt);
        to_nccl_op(args_.reduce_info.op, &op);
        NCCL_TRY(team_->tl_, api().AllReduce(src, dst, args_.reduce_info.count, dt, op, comm, s));
        break;
    case XCCL_REDUCE:
        to_nccl_dt(args_.reduce_info.dt, &dt);
        to_nccl_op(args_.reduce_info.op, &op);
        NCCL_TRY(team_->tl_, api().Reduce(src, dst, args_.reduce_info.count, dt, op, args_.root, comm, s));
        break;
    case XCCL_REDUCE_SCATTER: {
        to_nccl_dt(args_.reduce_info.dt, &dt);
        to_nccl_op(args_.reduce_info.op, &op);
        size_t cnt = args_.reduce_info.count;
        if (cnt == 0) cnt = bi.len / xccl_dt_size(args_.reduce_info.dt) / (size_t)n;
        NCCL_TRY(team_->tl_, api().ReduceScatter(src, dst, cnt, dt, op, comm, s));
        break;
    }
    case XCCL_ALLTOALL:
        NCCL_TRY(team_->tl_, api().GroupStart());
        for (int p = 0; p < n; p++) {
            NCCL_TRY(team_->tl_, api().Send((char *)src + (size_t)p * bi.len, bi.len, ncclChar, p, comm, s));
            NCCL_TRY(team_->tl_, api().Recv((char *)dst + (size_t)p * bi.len, bi.len, ncclChar, p, comm, s));
        }
        NCCL_TRY(team_->tl_, api().GroupEnd());
        break;
    case XCCL_ALLTOALLV: {
        const size_t ses = xccl_dt_size(bi.src_datatype), des = xccl_dt_size(bi.dst_datatype);
        NCCL_TRY(team_->tl_, api().GroupStart());
        for (int p = 0; p < n; p++) {
            NCCL_TRY(team_->tl_, api().Send((char *)src + (size_t)sd_[(size_t)p] * ses, (size_t)sc_[(size_t)p] * ses,
                                            ncclChar, p, comm, s));
            NCCL_TRY(team_->tl_, api().Recv((char *)dst + (size_t)dd_[(size_t)p] * des, (size_t)dc_[(size_t)p] * des,
                                            ncclChar, p, comm, s));
        }
        NCCL_TRY(team_->tl_, api().GroupEnd());
        break;
    }
    case XCCL_ALLGATHER:
        if (bi.src_buffer == XCCL_IN_PLACE) src = (char *)dst + (size_t)team_->rank * (bi.len / (size_t)n);
        NCCL_TRY(team_->tl_, api().AllGather(src, dst, bi.len / (size_t)n, ncclChar, comm, s));
        break;
    case XCCL_BCAST: NCCL_TRY(team_->tl_, api().Broadcast(src, dst, bi.len, ncclChar, args_.root, comm, s)); break;
    default: return XCCL_ERR_UNSUPPORTED;
    }
    if (epi_) {
        return cuda_reduce_multi(dst, nullptr, user_dst, 0, epi_count_, 0, args_.reduce_info.dt, XCCL_OP_SUM,
                                 args_.epilogue.scale, epi_out_, s);
    }
    return XCCL_OK;
}

xccl_status_t NcclReq::post()
{
    // re-posting a request that is still in flight is allowed: the stream orders the posts
    cudaStream_t s = team_->stream;
    if ((args_.field_mask & XCCL_COLL_OP_ARGS_FIELD_STREAM) && args_.stream.stream != nullptr) {
        s = *(cudaStream_t *)args_.stream.stream;
    }
    if (start_ != nullptr) XCCL_CUDA_CHECK(cudaEventRecord(start_, s));
    xccl_status_t st = start(s);
    if (st != XCCL_OK) return st;
    XCCL_CUDA_CHECK(cudaEventRecord(done_, s));
    in_flight_ = true;
    return XCCL_OK;
}

class NcclContext final : public TlContext {
public:
    NcclContext(const xccl_context_params_t &p, bool timing) : params_(p), timing_(timing) {}
    xccl_status_t team_create_post(const xccl_team_params_t &tp, TlTeam **team) override
    {
        OobGroup g = make_oob_group(tp, params_.oob);
        if (g.rank < 0) return XCCL_ERR_INVALID_PARAM;
        auto         *t  = new NcclTeam(tl, timing_);
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
    bool                  timing_;
};

class NcclLib final : public TeamLib {
public:
    NcclLib() : TeamLib(XCCL_TL_NCCL, 90)
    {
        caps.mem_types  = XCCL_BIT(XCCL_MEMORY_TYPE_CUDA);
        caps.team_usage = XCCL_LIB_PARAMS_TEAM_USAGE_SW_COLLECTIVES | XCCL_LIB_PARAMS_TEAM_USAGE_HW_COLLECTIVES;
        caps.epilogue   = true;  // one scale/cast kernel on the same stream after the library call
    }
    std::vector<OptField> lib_options() const override
    {
        return {
            {"ALLREDUCE", "1", "Serve allreduce", OptType::BOOL},   {"ALLTOALL", "1", "Serve alltoall", OptType::BOOL},
            {"ALLTOALLV", "1", "Serve alltoallv", OptType::BOOL},   {"ALLGATHER", "1", "Serve allgather", OptType::BOOL},
            {"BCAST", "1", "Serve bcast", OptType::BOOL},
            {"REDUCE", "1", "Serve reduce (extension: the reference leaves CUDA reduce to its UCX team)", OptType::BOOL},
            {"REDUCE_SCATTER", "1", "Serve reduce-scatter (extension)", OptType::BOOL},
        };
    }
    std::vector<OptField> context_options() const override
    {
        return {{"TIMING", "no", "Record CUDA events around each collective", OptType::BOOL}};
    }
    xccl_status_t open() override
    {
        if (!cuda_available() || !api().ok) return XCCL_ERR_NO_RESOURCE;
        caps.coll_types = 0;
        if (lib_cfg.flag("ALLREDUCE")) caps.coll_types |= XCCL_COLL_CAP_ALLREDUCE;
        if (lib_cfg.flag("ALLTOALL")) caps.coll_types |= XCCL_COLL_CAP_ALLTOALL;
        if (lib_cfg.flag("ALLTOALLV")) caps.coll_types |= XCCL_COLL_CAP_ALLTOALLV;
        if (lib_cfg.flag("ALLGATHER")) caps.coll_types |= XCCL_COLL_CAP_ALLGATHER;
        if (lib_cfg.flag("BCAST")) caps.coll_types |= XCCL_COLL_CAP_BCAST;
        if (lib_cfg.flag("REDUCE")) caps.coll_types |= XCCL_COLL_CAP_REDUCE;
        if (lib_cfg.flag("REDUCE_SCATTER")) caps.coll_types |= XCCL_COLL_CAP_REDUCE_SCATTER;
        return XCCL_OK;
    }
    xccl_status_t context_create(xccl_lib *, const xccl_context_params_t &params, const OptTable &cfg,
                                 TlContext **ctx) override
    {
        if (!cuda_available() || !api().ok) return XCCL_ERR_NO_RESOURCE;
        *ctx = new NcclContext(params, cfg.flag("TIMING"));
        return XCCL_OK;
    }
};

NcclLib          g_nccl_lib;
TeamLibRegistrar g_nccl_reg(&g_nccl_lib);

}  // namespace

bool nccl_available() { return cuda_available() && api().ok; }

}  // namespace nccltl
}  // namespace xccl

using namespace xccl;
using namespace xccl::nccltl;

extern "C" {

int xccl_nccl_version(void)
{
    int v = 0;
    if (api().ok && api().GetVersion != nullptr) api().GetVersion(&v);
    return v;
}

xccl_status_t xccl_p2p_comm_create(const xccl_oob_collectives_t *oob, void **comm_out)
{
    if (oob == nullptr || comm_out == nullptr) return XCCL_ERR_INVALID_PARAM;
    if (!nccl_available()) return XCCL_ERR_NO_RESOURCE;
    ncclUniqueId id{};
    if (oob->rank == 0 && api().GetUniqueId(&id) != ncclSuccess) return XCCL_ERR_NO_MESSAGE;
    std::vector<ncclUniqueId> ids((size_t)oob->size);
    xccl_status_t             st = oob_allgather_blocking(*oob, &id, ids.data(), sizeof(id));
    if (st != XCCL_OK) return st;
    ncclComm_t comm = nullptr;
    if (api().CommInitRank(&comm, oob->size, ids[0], oob->rank) != ncclSuccess) return XCCL_ERR_NO_MESSAGE;
    *comm_out = comm;
    return XCCL_OK;
}

void xccl_p2p_comm_destroy(void *comm)
{
    if (comm != nullptr && api().ok) api().CommDestroy((ncclComm_t)comm);
}

xccl_status_t xccl_p2p_send(void *comm, const void *buf, size_t bytes, int peer, void *stream)
{
    if (comm == nullptr || !api().ok) return XCCL_ERR_INVALID_PARAM;
    return api().Send(buf, bytes, ncclChar, peer, (ncclComm_t)comm, (cudaStream_t)stream) == ncclSuccess
               ? XCCL_OK
               : XCCL_ERR_NO_MESSAGE;
}

xccl_status_t xccl_p2p_recv(void *comm, void *buf, size_t bytes, int peer, void *stream)
{
    if (comm == nullptr || !api().ok) return XCCL_ERR_INVALID_PARAM;
    return api().Recv(buf, bytes, ncclChar, peer, (ncclComm_t)comm, (cudaStream_t)stream) == ncclSuccess
               ? XCCL_OK
               : XCCL_ERR_NO_MESSAGE;
}

xccl_status_t xccl_p2p_group_start(void) { return api().ok && api().GroupStart() == ncclSuccess ? XCCL_OK : XCCL_ERR_NO_MESSAGE; }
xccl_status_t xccl_p2p_group_end(void) { return api().ok && api().GroupEnd() == ncclSuccess ? XCCL_OK : XCCL_ERR_NO_MESSAGE; }

}  // extern "C"
