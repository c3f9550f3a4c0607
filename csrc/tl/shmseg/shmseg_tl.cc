// Shared-segment team library: global memory map and FANOUT_GET for ranks of one host.
//
// The reference names a proprietary shared-memory team ("shmseg", src/api/xccl_tls.h:18) as the
// only implementation of xccl_global_mem_map_* and XCCL_FANOUT_GET; it is not in its tree. This
// is an implementation of that contract:
//   mem_map_start(address, length, root)  the root creates a POSIX shared-memory window of
//       `length` bytes and announces it out of band; everybody maps it
//   FANOUT_GET(memh, offset, local_buffer, len)  the root publishes bytes [offset, offset+len) of
//       its region into the window and raises the request's flag; every other rank waits for the
//       flag (bounded by XCCL_WAIT_TIMEOUT) and copies the bytes out. The root returns at once:
//       it is a fan-out, completion on the root says nothing about the readers (callers that
//       reuse the region follow it with a FANIN, as the reference's bcast schedule does).
//   Requests on one region are numbered in the order they are created (the same on every rank, as
//   for every collective) and each owns one of kSlots flags, so they may be POSTED in any order:
//   the fragments of a pipelined broadcast complete their upper levels in no fixed order.
// Host memory only.
#include <atomic>
#include <cerrno>
#include <chrono>
#include <cstring>
#include <fcntl.h>
#include <sys/mman.h>
#include <unistd.h>

#include "../../core/core.h"

namespace xccl {
namespace shmseg {

namespace {

constexpr int kSlots = 256;  // flags per region: requests in use at the same time must be fewer than this apart in creation order

struct WindowHdr {
    // flag of request k: slot k % kSlots holds (k << 24 | number of posts) of the newest publication
    std::atomic<uint64_t> published[kSlots];
};

struct Announce {
    char     name[48];
    uint64_t length;
};

std::atomic<int> g_counter{0};

class SegTeam;

class SegMem final : public xccl_mem_handle {
public:
    SegMem(SegTeam *t, const xccl_mem_map_params_t &p) : team(t), params(p) {}
    ~SegMem() override { release(); }
    xccl_status_t start();
    xccl_status_t test() override;
    xccl_status_t unmap() override
    {
        release();
        return XCCL_OK;
    }
    void release()
    {
        if (base != nullptr) munmap(base, bytes);
        base = nullptr;
        if (owner && name[0] != '\0') shm_unlink(name);
        name[0] = '\0';
    }
    SegTeam              *team;
    xccl_mem_map_params_t params;
    void                 *oob_req = nullptr;
    std::vector<Announce> all;
    Announce              mine{};
    char                  name[48] = {0};
    void                 *base  = nullptr;
    size_t                bytes = 0;
    bool                  owner = false, ready = false;
    uint64_t              n_reqs = 0;  // FANOUT_GET requests created on this handle by this rank
    WindowHdr            *hdr() const { return (WindowHdr *)base; }
    char                 *data() const { return (char *)base + sizeof(WindowHdr); }
};

class SegTeam final : public TlTeam {
public:
    SegTeam(TeamLib *tl, const OobGroup &g) : tl_(tl), oob(g)
    {
        rank = g.rank;
        size = g.size;
    }
    xccl_status_t create_test() override { return XCCL_OK; }
    xccl_status_t collective_init(const xccl_coll_op_args_t &args, xccl_memory_type_t mem, xccl_coll_req **req) override;
    xccl_status_t mem_map_start(const xccl_mem_map_params_t &p, xccl_mem_handle **h) override
    {
        if (!(p.field_mask & XCCL_MEM_MAP_PARAM_FIELD_ROOT) || !(p.field_mask & XCCL_MEM_MAP_PARAM_FIELD_LENGTH)) {
            return XCCL_ERR_INVALID_PARAM;
        }
        auto          m  = std::make_unique<SegMem>(this, p);
        xccl_status_t st = m->start();
        if (st != XCCL_OK) return st;
        *h = m.release();
        return XCCL_OK;
    }
    TeamLib *tl_;
    OobGroup oob;
};

xccl_status_t SegMem::start()
{
    all.resize((size_t)team->size);
    bytes = sizeof(WindowHdr) + params.length;
    if (team->rank == params.root) {
        std::snprintf(name, sizeof(name), "/xccl-seg-%d-%d", (int)getpid(), g_counter.fetch_add(1));
        int fd = shm_open(name, O_CREAT | O_EXCL | O_RDWR, 0600);
        if (fd < 0 && errno == EEXIST) {  // this process's id and a counter it has not used: left by a dead process
            shm_unlink(name);
            fd = shm_open(name, O_CREAT | O_EXCL | O_RDWR, 0600);
        }
        if (fd < 0) return XCCL_ERR_NO_RESOURCE;
        if (ftruncate(fd, (off_t)bytes) != 0) {
            close(fd);
            shm_unlink(name);
            return XCCL_ERR_NO_MEMORY;
        }
        base = mmap(nullptr, bytes, PROT_READ | PROT_WRITE, MAP_SHARED, fd, 0);
        close(fd);
        if (base == MAP_FAILED) {
            base = nullptr;
            return XCCL_ERR_NO_MEMORY;
        }
        owner = true;
        std::memcpy(mine.name, name, sizeof(mine.name));
        mine.length = params.length;
    }
    if (team->oob.allgather(&mine, all.data(), sizeof(Announce), &oob_req) != 0) return XCCL_ERR_NO_MESSAGE;
    return XCCL_OK;
}

xccl_status_t SegMem::test()
{
    if (ready) return XCCL_OK;
    xccl_status_t st = team->oob.test(oob_req);
    if (st != XCCL_OK) return st;
    team->oob.free(oob_req);
    oob_req = nullptr;
    if (!owner) {
        const Announce &a = all[(size_t)params.root];
        if (a.length != params.length) return XCCL_ERR_INVALID_PARAM;
        int fd = shm_open(a.name, O_RDWR, 0600);
        if (fd < 0) return XCCL_ERR_UNREACHABLE;
        base = mmap(nullptr, bytes, PROT_READ | PROT_WRITE, MAP_SHARED, fd, 0);
        close(fd);
        if (base == MAP_FAILED) {
            base = nullptr;
            return XCCL_ERR_NO_MEMORY;
        }
    }
    ready = true;
    return XCCL_OK;
}

class GetReq final : public xccl_coll_req {
public:
    GetReq(SegTeam *t, SegMem *m, const xccl_coll_get_info_t &g) : team_(t), mem_(m), get_(g), id_(m->n_reqs++) {}
    xccl_status_t post() override
    {
        if (!mem_->ready) return XCCL_ERR_NO_RESOURCE;
        if ((size_t)get_.offset + get_.len > mem_->params.length) return XCCL_ERR_INVALID_PARAM;
        seq_  = (id_ << 24) | (++posts_ & 0xffffffu);
        done_ = false;
        t0_   = std::chrono::steady_clock::now();
        if (team_->rank == mem_->params.root) {
            const char *src = (const char *)mem_->params.address + get_.offset;
            std::memcpy(mem_->data() + get_.offset, src, get_.len);
            if (get_.local_buffer != nullptr && get_.local_buffer != src) std::memcpy(get_.local_buffer, src, get_.len);
            // never lowered: a slot is shared by requests kSlots apart, the newer one has the larger value
            auto    &flag = mem_->hdr()->published[id_ % kSlots];
            uint64_t cur  = flag.load(std::memory_order_relaxed);
            while (cur < seq_ && !flag.compare_exchange_weak(cur, seq_, std::memory_order_release, std::memory_order_relaxed)) {
            }
            done_ = true;
        }
        return XCCL_OK;
    }
    xccl_status_t test() override
    {
        if (done_) return XCCL_OK;
        if (mem_->hdr()->published[id_ % kSlots].load(std::memory_order_acquire) >= seq_) {
            std::memcpy(get_.local_buffer, mem_->data() + get_.offset, get_.len);
            done_ = true;
            return XCCL_OK;
        }
        double limit = global_state().opts.real("WAIT_TIMEOUT");
        if (limit > 0 && std::chrono::duration<double>(std::chrono::steady_clock::now() - t0_).count() > limit) {
            done_ = true;
            return XCCL_ERR_TIMED_OUT;
        }
        return XCCL_INPROGRESS;
    }
    xccl_status_t finalize() override { return XCCL_OK; }

private:
    SegTeam                              *team_;
    SegMem                               *mem_;
    xccl_coll_get_info_t                  get_;
    uint64_t                              id_;         // creation index on the region, the same on every rank
    uint64_t                              posts_ = 0;
    uint64_t                              seq_  = 0;
    bool                                  done_ = true;
    std::chrono::steady_clock::time_point t0_;
};

}  // namespace

}  // namespace shmseg
}  // namespace xccl

// The core wraps the per-TL handles of one region; this finds the shared-segment part.
namespace xccl {
xccl_mem_handle *find_mem_part(xccl_mem_handle *h, bool (*match)(xccl_mem_handle *));
}

namespace xccl {
namespace shmseg {
namespace {

bool is_segmem(xccl_mem_handle *h) { return dynamic_cast<SegMem *>(h) != nullptr; }

xccl_status_t SegTeam::collective_init(const xccl_coll_op_args_t &args, xccl_memory_type_t mem, xccl_coll_req **req)
{
    if (args.coll_type != XCCL_FANOUT_GET || mem != XCCL_MEMORY_TYPE_HOST) return XCCL_ERR_UNSUPPORTED;
    auto *m = static_cast<SegMem *>(find_mem_part((xccl_mem_handle *)args.get_info.memh, is_segmem));
    if (m == nullptr || m->team != this) return XCCL_ERR_INVALID_PARAM;
    *req = new GetReq(this, m, args.get_info);
    return XCCL_OK;
}

class SegContext final : public TlContext {
public:
    explicit SegContext(const xccl_context_params_t &p) : params_(p) {}
    xccl_status_t team_create_post(const xccl_team_params_t &tp, TlTeam **team) override
    {
        OobGroup g = make_oob_group(tp, params_.oob);
        if (g.rank < 0) return XCCL_ERR_INVALID_PARAM;
        *team = new SegTeam(tl, g);
        return XCCL_OK;
    }

private:
    xccl_context_params_t params_;
};

class SegLib final : public TeamLib {
public:
    SegLib() : TeamLib(XCCL_TL_SHMSEG, 80)
    {
        caps.coll_types = XCCL_COLL_CAP_FANOUT_GET;
        caps.mem_types  = XCCL_BIT(XCCL_MEMORY_TYPE_HOST);
    }
    xccl_status_t context_create(xccl_lib *, const xccl_context_params_t &params, const OptTable &, TlContext **ctx) override
    {
        *ctx = new SegContext(params);
        return XCCL_OK;
    }
};

SegLib           g_seg_lib;
TeamLibRegistrar g_seg_reg(&g_seg_lib);

}  // namespace
}  // namespace shmseg
}  // namespace xccl
