// Shared-memory out-of-band provider and sub-group views. See include/xccl/xccl_oob.h.
#include <atomic>
#include <cerrno>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <fcntl.h>
#include <string>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>
#include <vector>

#include "../core/tl.h"
#include "xccl/xccl_oob.h"

namespace {

constexpr uint32_t kSlotBytes = 4032;  // mailbox payload; header + payload = 4096

struct alignas(64) Mailbox {
    std::atomic<uint32_t> wseq;  // messages written by the sender
    std::atomic<uint32_t> rseq;  // messages consumed by the receiver
    uint32_t              len;
    char                  pad[52];
    char                  data[kSlotBytes];
};
static_assert(sizeof(Mailbox) == 4096, "mailbox is one page");

struct SegHeader {
    std::atomic<uint32_t> attached;
    uint32_t              nranks;
    char                  pad[4088];
};

struct ShmOob {
    std::string name;
    int         rank = 0, size = 0;
    size_t      bytes = 0;
    SegHeader  *hdr   = nullptr;
    Mailbox    *boxes = nullptr;  // [dst][src]
    Mailbox    &box(int dst, int src) { return boxes[(size_t)dst * size + src]; }
};

struct AgReq {
    ShmOob             *oob;
    std::vector<int>    members;  // job ranks of the group
    int                 me;       // my index in members
    std::vector<char>   sbuf;
    char               *rbuf;
    size_t              size;
    std::vector<size_t> sent, rcvd;
};

bool ag_progress(AgReq *r)
{
    bool    done = true;
    ShmOob *o    = r->oob;
    for (size_t j = 0; j < r->members.size(); j++) {
        if ((int)j == r->me) continue;
        int peer = r->members[j];
        // push my bytes to the peer
        while (r->sent[j] < r->size) {
            Mailbox &b = o->box(peer, o->rank);
            uint32_t w = b.wseq.load(std::memory_order_relaxed);
            if (w != b.rseq.load(std::memory_order_acquire)) break;  // previous chunk not consumed
            uint32_t n = (uint32_t)std::min<size_t>(kSlotBytes, r->size - r->sent[j]);
            std::memcpy(b.data, r->sbuf.data() + r->sent[j], n);
            b.len = n;
            b.wseq.store(w + 1, std::memory_order_release);
            r->sent[j] += n;
        }
        // pull the peer's bytes
        while (r->rcvd[j] < r->size) {
            Mailbox &b  = o->box(o->rank, peer);
            uint32_t rd = b.rseq.load(std::memory_order_relaxed);
            if (b.wseq.load(std::memory_order_acquire) == rd) break;
            uint32_t n = b.len;
            if (n > r->size - r->rcvd[j]) n = (uint32_t)(r->size - r->rcvd[j]);  // size mismatch guard
            std::memcpy(r->rbuf + j * r->size + r->rcvd[j], b.data, n);
            b.rseq.store(rd + 1, std::memory_order_release);
            r->rcvd[j] += n;
        }
        if (r->sent[j] < r->size || r->rcvd[j] < r->size) done = false;
    }
    return done;
}

int shm_allgather(void *sbuf, void *rbuf, size_t size, int my_rank, xccl_ep_range_t range, void *coll_context,
                  void **request)
{
    auto *o = (ShmOob *)coll_context;
    auto *r = new AgReq;
    r->oob  = o;
    if (range.type == XCCL_EP_RANGE_UNDEFINED) {
        r->members.resize((size_t)o->size);
        for (int i = 0; i < o->size; i++) r->members[(size_t)i] = i;
        r->me = o->rank;
    } else {
        r->members.resize((size_t)range.ep_num);
        for (int i = 0; i < range.ep_num; i++) r->members[(size_t)i] = xccl_range_to_rank(range, i);
        r->me = my_rank;
    }
    if (r->me < 0 || r->me >= (int)r->members.size() || r->members[(size_t)r->me] != o->rank) {
        delete r;
        return -1;
    }
    r->sbuf.assign((char *)sbuf, (char *)sbuf + size);
    r->rbuf = (char *)rbuf;
    r->size = size;
    r->sent.assign(r->members.size(), 0);
    r->rcvd.assign(r->members.size(), 0);
    std::memcpy(r->rbuf + (size_t)r->me * size, sbuf, size);
    ag_progress(r);
    *request = r;
    return 0;
}

xccl_status_t shm_req_test(void *request) { return ag_progress((AgReq *)request) ? XCCL_OK : XCCL_INPROGRESS; }

xccl_status_t shm_req_free(void *request)
{
    delete (AgReq *)request;
    return XCCL_OK;
}

// ------------------------------------------------------------------ sub-group view

struct SubOob {
    xccl_oob_collectives_t parent;
    std::vector<int>       ranks;  // parent rank of member i
};

int sub_map_cb(int rank, void *ctx) { return ((SubOob *)ctx)->ranks[(size_t)rank]; }

int sub_allgather(void *sbuf, void *rbuf, size_t size, int my_rank, xccl_ep_range_t range, void *coll_context,
                  void **request)
{
    auto *s = (SubOob *)coll_context;
    if (range.type != XCCL_EP_RANGE_UNDEFINED) {
        // a range over a sub-group composes: member i of the range is sub rank range(i)
        auto *tmp  = new SubOob;
        tmp->parent = s->parent;
        tmp->ranks.resize((size_t)range.ep_num);
        for (int i = 0; i < range.ep_num; i++) tmp->ranks[(size_t)i] = s->ranks[(size_t)xccl_range_to_rank(range, i)];
        xccl_ep_range_t r2{};
        r2.type      = XCCL_EP_RANGE_CB;
        r2.ep_num    = range.ep_num;
        r2.cb.cb     = sub_map_cb;
        r2.cb.cb_ctx = tmp;
        int rc       = s->parent.allgather(sbuf, rbuf, size, my_rank, r2, s->parent.coll_context, request);
        delete tmp;  // the parent copies the member list inside allgather()
        return rc;
    }
    xccl_ep_range_t r{};
    r.type      = XCCL_EP_RANGE_CB;
    r.ep_num    = (int)s->ranks.size();
    r.cb.cb     = sub_map_cb;
    r.cb.cb_ctx = s;
    return s->parent.allgather(sbuf, rbuf, size, my_rank, r, s->parent.coll_context, request);
}

}  // namespace

extern "C" {

xccl_status_t xccl_oob_shm_create(const char *job_key, int rank, int size, xccl_oob_collectives_t *oob)
{
    if (job_key == nullptr || oob == nullptr || size < 1 || rank < 0 || rank >= size) return XCCL_ERR_INVALID_PARAM;
    auto *o  = new ShmOob;
    o->name  = std::string("/xccl-oob-") + job_key;
    o->rank  = rank;
    o->size  = size;
    o->bytes = sizeof(SegHeader) + sizeof(Mailbox) * (size_t)size * (size_t)size;
    int fd   = shm_open(o->name.c_str(), O_CREAT | O_RDWR, 0600);
    if (fd < 0) {
        xccl_error("shm_open(%s): %s", o->name.c_str(), std::strerror(errno));
        delete o;
        return XCCL_ERR_NO_RESOURCE;
    }
    if (ftruncate(fd, (off_t)o->bytes) != 0) {
        xccl_error("ftruncate(%s, %zu): %s", o->name.c_str(), o->bytes, std::strerror(errno));
        close(fd);
        delete o;
        return XCCL_ERR_NO_MEMORY;
    }
    void *p = mmap(nullptr, o->bytes, PROT_READ | PROT_WRITE, MAP_SHARED, fd, 0);
    close(fd);
    if (p == MAP_FAILED) {
        delete o;
        return XCCL_ERR_NO_MEMORY;
    }
    o->hdr   = (SegHeader *)p;
    o->boxes = (Mailbox *)((char *)p + sizeof(SegHeader));
    o->hdr->attached.fetch_add(1);
    oob->allgather    = shm_allgather;
    oob->req_test     = shm_req_test;
    oob->req_free     = shm_req_free;
    oob->coll_context = o;
    oob->rank         = rank;
    oob->size         = size;
    return XCCL_OK;
}

void xccl_oob_shm_destroy(xccl_oob_collectives_t *oob)
{
    if (oob == nullptr || oob->coll_context == nullptr) return;
    auto    *o    = (ShmOob *)oob->coll_context;
    uint32_t left = o->hdr->attached.fetch_sub(1) - 1;
    munmap((void *)o->hdr, o->bytes);
    if (left == 0) shm_unlink(o->name.c_str());
    delete o;
    oob->coll_context = nullptr;
}

xccl_status_t xccl_oob_sub_create(const xccl_oob_collectives_t *parent, const int *parent_ranks, int n,
                                  xccl_oob_collectives_t *sub)
{
    if (parent == nullptr || parent_ranks == nullptr || sub == nullptr || n < 1) return XCCL_ERR_INVALID_PARAM;
    auto *s   = new SubOob;
    s->parent = *parent;
    s->ranks.assign(parent_ranks, parent_ranks + n);
    int me = -1;
    for (int i = 0; i < n; i++) {
        if (parent_ranks[i] == parent->rank) me = i;
    }
    if (me < 0) {
        delete s;
        return XCCL_ERR_INVALID_PARAM;
    }
    sub->allgather    = sub_allgather;
    sub->req_test     = parent->req_test;
    sub->req_free     = parent->req_free;
    sub->coll_context = s;
    sub->rank         = me;
    sub->size         = n;
    return XCCL_OK;
}

void xccl_oob_sub_destroy(xccl_oob_collectives_t *sub)
{
    if (sub == nullptr) return;
    delete (SubOob *)sub->coll_context;
    sub->coll_context = nullptr;
}

xccl_status_t xccl_oob_allgather(const xccl_oob_collectives_t *oob, void *sbuf, void *rbuf, size_t size)
{
    if (oob == nullptr) return XCCL_ERR_INVALID_PARAM;
    return xccl::oob_allgather_blocking(*oob, sbuf, rbuf, size);
}

}  // extern "C"
