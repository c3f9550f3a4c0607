// Collective dispatch and global memory map fan-out.
// Reference behaviour: src/core/xccl_collective.c:16-92, src/core/xccl_mm.c:3-72.
#include <chrono>

#include <nvtx3/nvToolsExt.h>  // header-only: resolves to no-ops unless a profiler injects itself

#include "../cuda/mem_cuda.h"
#include "../utils/mem.h"
#include "core.h"

using namespace xccl;

namespace {
// XCCL_NVTX=y: ranges "xccl:<collective>:post" / ":wait" around the calls, so a timeline shows which
// collective a kernel or a host wait belongs to. Read once.
bool nvtx_on()
{
    static const bool on = global_state().opts.flag("NVTX");  // initialised once, also with several posting threads
    return on;
}
const char *coll_name(int t)
{
    static const char *names[] = {"barrier", "bcast", "allreduce", "reduce", "alltoall", "alltoallv", "allgather",
                                  "fanin", "fanout", "fanout_get", "reduce_scatter"};
    return (t >= 0 && t < (int)(sizeof(names) / sizeof(names[0]))) ? names[t] : "collective";
}
struct NvtxRange {
    bool on;
    NvtxRange(const xccl_coll_req *r, const char *what) : on(nvtx_on())
    {
        if (!on) return;
        char buf[64];
        std::snprintf(buf, sizeof(buf), "xccl:%s:%s", coll_name(r != nullptr ? r->coll_type : -1), what);
        nvtxRangePushA(buf);
    }
    ~NvtxRange()
    {
        if (on) nvtxRangePop();
    }
};
}  // namespace

xccl_status_t xccl_coll_req::wait()
{
    double        limit = global_state().opts.real("WAIT_TIMEOUT");
    auto          t0    = std::chrono::steady_clock::now();
    xccl_status_t st;
    unsigned      spins = 0;
    while ((st = test()) == XCCL_INPROGRESS) {
        if (core_team != nullptr) {
            xccl_status_t pst = xccl_context_progress(core_team->ctx);
            if (pst < 0) return pst;
        }
        if ((++spins & 0x3ff) == 0 && limit > 0) {
            double dt = std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
            if (dt > limit) {
                // the collective is still in flight inside its team library and cannot be matched with the peers'
                // any more: every later collective of that team fails at once instead of waiting again
                if (tl_team != nullptr) tl_team->poisoned = true;
                return XCCL_ERR_TIMED_OUT;
            }
        }
    }
    return st;
}

namespace {

// A region mapped through several team libraries: complete when each of them is.
struct FanoutMemHandle final : xccl_mem_handle {
    std::vector<xccl_mem_handle *> parts;
    xccl_status_t test() override
    {
        for (auto *p : parts) {
            xccl_status_t st = p->test();
            if (st != XCCL_OK) return st;
        }
        return XCCL_OK;
    }
    xccl_status_t unmap() override
    {
        for (auto *p : parts) {
            p->unmap();
            delete p;
        }
        parts.clear();
        return XCCL_OK;
    }
};

}  // namespace

namespace {

// The scale/cast epilogue for a team library that cannot fuse it: the library reduces in the input datatype
// (into the caller's dst when the output type is the same, else into a private buffer), and when its request
// completes the result is scaled and converted into dst as a last local step - on the host for host memory,
// with the reduction kernel (no vectors to add, only scale and cast) for device memory. The request reports
// completion only after that step. Such libraries complete through test(), so a caller already has to see
// XCCL_OK before it reads dst.
struct EpilogueReq final : xccl_coll_req {
    xccl_coll_req     *inner = nullptr;
    xccl_memory_type_t mem   = XCCL_MEMORY_TYPE_HOST;
    void              *tmp   = nullptr;   // owned; nullptr = scale in place in dst
    void              *dst   = nullptr;
    xccl_dt_t          dt = XCCL_DT_UNSUPPORTED, out_dt = XCCL_DT_UNSUPPORTED;
    size_t             count  = 0;
    float              scale  = 1.0f;
    void              *stream = nullptr;  // cudaStream_t value, may be null
    void              *event  = nullptr;
    bool               local_result = true;  // false on the non-root ranks of a reduce
    enum { IDLE, INNER, KERNEL, DONE } state = IDLE;

    ~EpilogueReq() override
    {
        if (event != nullptr) cuda_event_release(event);
        if (tmp != nullptr) mem_free(tmp, mem);
        delete inner;
    }
    xccl_status_t post() override
    {
        if (state == INNER || state == KERNEL) return XCCL_ERR_INVALID_PARAM;  // still in flight
        xccl_status_t st = inner->post();
        if (st == XCCL_OK) state = INNER;
        return st;
    }
    xccl_status_t test() override
    {
        if (state == INNER) {
            xccl_status_t st = inner->test();
            if (st != XCCL_OK) return st;
            if (!local_result || count == 0) {
                state = DONE;
            } else if (mem == XCCL_MEMORY_TYPE_CUDA) {
                st = cuda_reduce_multi(tmp != nullptr ? tmp : dst, nullptr, dst, 0, count, 0, dt, XCCL_OP_SUM, scale,
                                       out_dt, stream != nullptr ? stream : cuda_internal_stream());
                if (st != XCCL_OK) return st;
                st = cuda_event_record(stream != nullptr ? stream : cuda_internal_stream(), &event);
                if (st != XCCL_OK) return st;
                state = KERNEL;
            } else {
                st = host_scale_cast(tmp != nullptr ? tmp : dst, dt, dst, out_dt, count, scale);
                if (st != XCCL_OK) return st;
                state = DONE;
            }
        }
        if (state == KERNEL) {
            xccl_status_t st = cuda_event_query(event);
            if (st != XCCL_OK) return st;
            cuda_event_release(event);
            event = nullptr;
            state = DONE;
        }
        return state == DONE ? XCCL_OK : XCCL_ERR_INVALID_PARAM;  // IDLE: never posted
    }
    xccl_status_t finalize() override
    {
        if (state == INNER || state == KERNEL) return XCCL_INPROGRESS;
        return inner->finalize();
    }
    double elapsed_us() override { return inner->elapsed_us(); }
};

bool is_reduction(xccl_collective_type_t c) { return c == XCCL_ALLREDUCE || c == XCCL_REDUCE || c == XCCL_REDUCE_SCATTER; }

// Elements of dt that the reduction leaves in dst on this rank.
size_t result_count(const xccl_coll_op_args_t &a, int team_size)
{
    const size_t es = xccl_dt_size(a.reduce_info.dt);
    if (es == 0) return 0;
    if (a.coll_type == XCCL_REDUCE_SCATTER) {
        return a.buffer_info.len != 0 ? a.buffer_info.len / (size_t)team_size / es : a.reduce_info.count;
    }
    return a.buffer_info.len != 0 ? a.buffer_info.len / es : a.reduce_info.count;
}

}  // namespace

namespace xccl {
// A region handle returned by xccl_global_mem_map_start bundles one handle per team library;
// a team library finds its own part with this.
xccl_mem_handle *find_mem_part(xccl_mem_handle *h, bool (*match)(xccl_mem_handle *))
{
    if (h == nullptr) return nullptr;
    if (auto *f = dynamic_cast<FanoutMemHandle *>(h)) {
        for (auto *p : f->parts) {
            if (match(p)) return p;
        }
        return nullptr;
    }
    return match(h) ? h : nullptr;
}
}  // namespace xccl

namespace {

xccl_status_t init_with_local_epilogue(xccl_team *team, TlTeam *tt, const xccl_coll_op_args_t &args,
                                       xccl_memory_type_t mem, xccl_coll_req **out)
{
    const xccl_dt_t dt = args.reduce_info.dt;
    xccl_dt_t       od = args.epilogue.out_dt;
    if (od == XCCL_DT_UNSUPPORTED || od == XCCL_DT_LAST_PREDEFINED) od = dt;
    xccl_coll_op_args_t inner = args;
    inner.field_mask &= ~(uint64_t)XCCL_COLL_OP_ARGS_FIELD_EPILOGUE;
    if (args.epilogue.scale == 1.0f && od == dt) return tt->collective_init(inner, mem, out);

    // the conversion has to exist; probe it on the host, where both sides implement the same pairs
    char pin[16] = {0}, pout[16] = {0};
    if (host_scale_cast(pin, dt, pout, od, 1, 1.0f) != XCCL_OK) return XCCL_ERR_UNSUPPORTED;

    int rank = 0, size = 1;
    xccl_team_query(team, &rank, &size);
    auto *req         = new EpilogueReq;
    req->mem          = mem;
    req->dt           = dt;
    req->out_dt       = od;
    req->scale        = args.epilogue.scale;
    req->count        = result_count(args, size);
    req->dst          = args.buffer_info.dst_buffer;
    req->local_result = (args.coll_type != XCCL_REDUCE) || (args.root == rank);
    if ((args.field_mask & XCCL_COLL_OP_ARGS_FIELD_STREAM) && args.stream.stream != nullptr) {
        req->stream = *(void **)args.stream.stream;
    }
    if (od != dt && req->local_result) {
        xccl_status_t st = mem_alloc(&req->tmp, req->count * xccl_dt_size(dt), mem);
        if (st != XCCL_OK) {
            delete req;
            return st;
        }
        // in place: dst holds the input and receives the converted output; the library reads it, writes tmp
        if (inner.buffer_info.src_buffer == XCCL_IN_PLACE || inner.buffer_info.src_buffer == nullptr) {
            inner.buffer_info.src_buffer = args.buffer_info.dst_buffer;
        }
        inner.buffer_info.dst_buffer = req->tmp;
    }
    xccl_status_t st = tt->collective_init(inner, mem, &req->inner);
    if (st != XCCL_OK) {
        delete req;
        return st;
    }
    *out = req;
    return XCCL_OK;
}

}  // namespace

extern "C" {

xccl_status_t xccl_collective_init(xccl_coll_op_args_t *args, xccl_coll_req_h *request, xccl_team_h team)
{
    if (args == nullptr || request == nullptr || team == nullptr) return XCCL_ERR_INVALID_PARAM;
    if (!team->created) return XCCL_ERR_NO_RESOURCE;
    if ((int)args->coll_type < 0 || args->coll_type >= XCCL_COLL_LAST) return XCCL_ERR_INVALID_PARAM;
    // a root is a team rank: checked here once, so that no team library indexes its peers with it unchecked
    if (args->coll_type == XCCL_BCAST || args->coll_type == XCCL_REDUCE || args->coll_type == XCCL_FANIN ||
        args->coll_type == XCCL_FANOUT) {
        const xccl_team_params_t &tp = team->params;
        const int team_size = (tp.field_mask & XCCL_TEAM_PARAM_FIELD_OOB) ? tp.oob.size
                              : ((tp.field_mask & XCCL_TEAM_PARAM_FIELD_EP_RANGE) && tp.range.type != XCCL_EP_RANGE_UNDEFINED)
                                  ? tp.range.ep_num
                                  : team->ctx->params.oob.size;
        if (args->root < 0 || args->root >= team_size) {
            xccl_debug("root %d outside a team of %d ranks", args->root, team_size);
            return XCCL_ERR_INVALID_PARAM;
        }
    }

    // buffers and count arrays a collective cannot do without (an empty message may come without buffers)
    {
        const xccl_coll_buffer_info_t &bi = args->buffer_info;
        const bool empty = bi.len == 0 && args->reduce_info.count == 0;
        switch (args->coll_type) {
        case XCCL_ALLREDUCE:
        case XCCL_REDUCE_SCATTER:
        case XCCL_ALLTOALL:
            if (!empty && bi.dst_buffer == nullptr) return XCCL_ERR_INVALID_PARAM;
            break;
        case XCCL_ALLGATHER: {
            const xccl_team_params_t &tp = team->params;
            const int n = (tp.field_mask & XCCL_TEAM_PARAM_FIELD_OOB) ? tp.oob.size
                          : ((tp.field_mask & XCCL_TEAM_PARAM_FIELD_EP_RANGE) && tp.range.type != XCCL_EP_RANGE_UNDEFINED)
                              ? tp.range.ep_num
                              : team->ctx->params.oob.size;
            if (!empty && bi.dst_buffer == nullptr) return XCCL_ERR_INVALID_PARAM;
            if (n > 0 && bi.len % (size_t)n != 0) return XCCL_ERR_INVALID_PARAM;  // len is the gathered size
            break;
        }
        case XCCL_ALLTOALLV:
            if (bi.dst_buffer == nullptr || bi.src_counts == nullptr || bi.dst_counts == nullptr ||
                bi.src_displacements == nullptr || bi.dst_displacements == nullptr) {
                return XCCL_ERR_INVALID_PARAM;
            }
            break;
        case XCCL_BCAST:
            if (!empty && bi.dst_buffer == nullptr && (bi.src_buffer == nullptr || bi.src_buffer == XCCL_IN_PLACE)) {
                return XCCL_ERR_INVALID_PARAM;
            }
            break;
        default: break;
        }
    }

    // Synchronisation-only collectives carry no buffer and count as host memory.
    xccl_memory_type_t mem = XCCL_MEMORY_TYPE_HOST;
    switch (args->coll_type) {
    case XCCL_BARRIER:
    case XCCL_FANIN:
    case XCCL_FANOUT: break;
    case XCCL_FANOUT_GET: mem = mem_type_of(args->get_info.local_buffer); break;
    default: {
        const void *probe = args->buffer_info.src_buffer;
        if (probe == XCCL_IN_PLACE || probe == nullptr) probe = args->buffer_info.dst_buffer;
        mem = mem_type_of(probe);
    }
    }
    int id = team->coll_team_id[args->coll_type][mem];
    if (id < 0) {
        xccl_debug("no team library serves collective %d on memory type %d", (int)args->coll_type, (int)mem);
        return XCCL_ERR_UNSUPPORTED;
    }
    // The table names the first team library by priority. When that one answers XCCL_ERR_UNSUPPORTED for
    // these arguments (a datatype, operation or layout it does not handle - facts every rank sees alike),
    // the next one that serves the collective on this memory type is asked.
    const bool want_epi = is_reduction(args->coll_type) && (args->field_mask & XCCL_COLL_OP_ARGS_FIELD_EPILOGUE);
    xccl_status_t st = XCCL_ERR_UNSUPPORTED;
    for (size_t i = (size_t)id; i < team->tl_teams.size(); i++) {
        TlTeam       *tt   = team->tl_teams[i].get();
        const TlCaps &caps = tt->ctx->tl->caps;
        if (i != (size_t)id) {
            const bool     sync = (args->coll_type == XCCL_BARRIER || args->coll_type == XCCL_FANIN ||
                               args->coll_type == XCCL_FANOUT);
            const uint64_t mems = (sync && caps.sync_mem_types != ~0ull) ? caps.sync_mem_types : caps.mem_types;
            if (!(caps.coll_types & XCCL_BIT(args->coll_type)) || !(mems & XCCL_BIT(mem))) continue;
        }
        if (tt->poisoned) return XCCL_ERR_NO_PROGRESS;
        xccl_coll_req *req = nullptr;
        if (want_epi && !caps.epilogue) {
            st = init_with_local_epilogue(team, tt, *args, mem, &req);
        } else {
            st = tt->collective_init(*args, mem, &req);
        }
        if (st == XCCL_ERR_UNSUPPORTED) {
            xccl_debug("team library %s does not take this %s, trying the next one", tt->ctx->tl->name,
                       coll_name((int)args->coll_type));
            continue;
        }
        if (st != XCCL_OK) return st;
        req->core_team = team;
        req->coll_type = (int)args->coll_type;
        req->tl_team   = tt;
        *request       = req;
        return XCCL_OK;
    }
    return st;
}

xccl_status_t xccl_collective_post(xccl_coll_req_h request)
{
    if (request == nullptr) return XCCL_ERR_INVALID_PARAM;
    NvtxRange r(request, "post");
    return request->post();
}

xccl_status_t xccl_collective_wait(xccl_coll_req_h request)
{
    if (request == nullptr) return XCCL_ERR_INVALID_PARAM;
    NvtxRange r(request, "wait");
    return request->wait();
}

xccl_status_t xccl_collective_test(xccl_coll_req_h request)
{
    return request != nullptr ? request->test() : XCCL_ERR_INVALID_PARAM;
}

xccl_status_t xccl_collective_finalize(xccl_coll_req_h request)
{
    if (request == nullptr) return XCCL_ERR_INVALID_PARAM;
    xccl_status_t st = request->finalize();
    if (st != XCCL_OK) return st;  // still in flight: the caller keeps the request
    delete request;
    return XCCL_OK;
}

double xccl_collective_elapsed_us(xccl_coll_req_h request) { return request != nullptr ? request->elapsed_us() : -1.0; }

xccl_status_t xccl_global_mem_map_start(xccl_team_h team, xccl_mem_map_params_t params, xccl_mem_h *memh_p)
{
    if (team == nullptr || memh_p == nullptr || !team->created) return XCCL_ERR_INVALID_PARAM;
    auto *h = new FanoutMemHandle;
    for (auto &tt : team->tl_teams) {
        xccl_mem_handle *part = nullptr;
        xccl_status_t    st   = tt->mem_map_start(params, &part);
        if (st == XCCL_OK && part != nullptr) {
            h->parts.push_back(part);
        } else if (st != XCCL_ERR_NOT_IMPLEMENTED && st != XCCL_ERR_UNSUPPORTED) {
            h->unmap();
            delete h;
            return st;
        }
    }
    if (h->parts.empty()) {
        delete h;
        return XCCL_ERR_NOT_IMPLEMENTED;
    }
    *memh_p = h;
    return XCCL_OK;
}

xccl_status_t xccl_global_mem_map_test(xccl_mem_h memh) { return memh != nullptr ? memh->test() : XCCL_ERR_INVALID_PARAM; }

xccl_status_t xccl_global_mem_unmap(xccl_mem_h memh)
{
    if (memh == nullptr) return XCCL_ERR_INVALID_PARAM;
    xccl_status_t st = memh->unmap();
    delete memh;
    return st;
}

}  // extern "C"
