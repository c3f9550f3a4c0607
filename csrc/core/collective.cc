// Collective dispatch and global memory map fan-out.
// Reference behaviour: src/core/xccl_collective.c:16-92, src/core/xccl_mm.c:3-72.
#include <chrono>

#include <nvtx3/nvToolsExt.h>  // header-only: resolves to no-ops unless a profiler injects itself

#include "../utils/mem.h"
#include "core.h"

using namespace xccl;

namespace {
// XCCL_NVTX=y: ranges "xccl:<collective>:post" / ":wait" around the calls, so a timeline shows which
// collective a kernel or a host wait belongs to. Read once.
bool nvtx_on()
{
    static int on = -1;
    if (on < 0) on = global_state().opts.flag("NVTX") ? 1 : 0;
    return on == 1;
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
            if (dt > limit) return XCCL_ERR_TIMED_OUT;
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

extern "C" {

xccl_status_t xccl_collective_init(xccl_coll_op_args_t *args, xccl_coll_req_h *request, xccl_team_h team)
{
    if (args == nullptr || request == nullptr || team == nullptr) return XCCL_ERR_INVALID_PARAM;
    if (!team->created) return XCCL_ERR_NO_RESOURCE;
    if ((int)args->coll_type < 0 || args->coll_type >= XCCL_COLL_LAST) return XCCL_ERR_INVALID_PARAM;

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
    TlTeam *tt = team->tl_teams[(size_t)id].get();
    if (tt->poisoned) return XCCL_ERR_NO_PROGRESS;
    xccl_coll_req *req = nullptr;
    xccl_status_t  st  = tt->collective_init(*args, mem, &req);
    if (st != XCCL_OK) return st;
    req->core_team = team;
    req->coll_type = (int)args->coll_type;
    *request       = req;
    return XCCL_OK;
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
