#include "transport.h"

#include <algorithm>
#include <cerrno>
#include <cstdio>
#include <cstring>
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include "../../core/core.h"

namespace xccl {
namespace host {

namespace {

struct WireHeader {
    uint32_t tag;
    uint32_t magic;
    uint64_t len;
};
static_assert(sizeof(WireHeader) == 16, "header is 16 bytes");
constexpr uint32_t kMagic = 0x58434c31;  // "XCL1"

inline size_t wire_len(size_t len) { return (len + 15) & ~(size_t)15; }

void ring_write(char *ring, size_t ring_bytes, uint64_t pos, const void *src, size_t n)
{
    size_t off   = (size_t)(pos % ring_bytes);
    size_t first = std::min(n, ring_bytes - off);
    std::memcpy(ring + off, src, first);
    if (first < n) std::memcpy(ring, (const char *)src + first, n - first);
}

void ring_read(const char *ring, size_t ring_bytes, uint64_t pos, void *dst, size_t n)
{
    size_t off   = (size_t)(pos % ring_bytes);
    size_t first = std::min(n, ring_bytes - off);
    std::memcpy(dst, ring + off, first);
    if (first < n) std::memcpy((char *)dst + first, ring, n - first);
}

std::atomic<int> g_seg_counter{0};

}  // namespace

Transport::Transport(int rank, int size, size_t ring_bytes)
    : rank_(rank), size_(size), ring_bytes_(std::max<size_t>(4096, ring_bytes & ~(size_t)15)), peers_((size_t)size),
      outq_((size_t)size), in_((size_t)size)
{
}

Transport::~Transport()
{
    for (int p = 0; p < size_; p++) {
        if (p != rank_ && peers_[(size_t)p].base != nullptr) munmap(peers_[(size_t)p].base, peers_[(size_t)p].bytes);
        for (auto &u : in_[(size_t)p].unexpected) delete u->claimed;
    }
    if (mine_.base != nullptr) {
        munmap(mine_.base, mine_.bytes);
        if (!unlinked_) shm_unlink(my_name_.c_str());
    }
}

// The name of a segment is needed only until every peer has mapped it. Dropping it then means that a process which
// exits without destroying its team (or is killed) leaves nothing behind under /dev/shm.
void Transport::unlink_when_attached()
{
    if (unlinked_ || mine_.base == nullptr) return;
    for (int p = 0; p < size_; p++) {
        if (p != rank_ && ctl_of(mine_, p)->attached.load(std::memory_order_acquire) == 0) return;
    }
    shm_unlink(my_name_.c_str());
    unlinked_ = true;
}

RingCtl *Transport::ctl_of(const Segment &s, int src) const
{
    return (RingCtl *)((char *)s.base + (size_t)src * (sizeof(RingCtl) + ring_bytes_));
}

char *Transport::data_of(const Segment &s, int src) const { return (char *)ctl_of(s, src) + sizeof(RingCtl); }

xccl_status_t Transport::create_local(PeerInfo *mine)
{
    char name[64];
    std::snprintf(name, sizeof(name), "/xccl-h-%d-%d", (int)getpid(), g_seg_counter.fetch_add(1));
    my_name_    = name;
    mine_.bytes = (size_t)size_ * (sizeof(RingCtl) + ring_bytes_);
    int fd      = shm_open(name, O_CREAT | O_EXCL | O_RDWR, 0600);
    if (fd < 0 && errno == EEXIST) {
        // the name carries this process's id and a counter it has not used yet: a leftover of a dead process
        shm_unlink(name);
        fd = shm_open(name, O_CREAT | O_EXCL | O_RDWR, 0600);
    }
    if (fd < 0) {
        xccl_error("shm_open(%s): %s", name, std::strerror(errno));
        return XCCL_ERR_NO_RESOURCE;
    }
    if (ftruncate(fd, (off_t)mine_.bytes) != 0) {
        xccl_error("ftruncate(%s, %zu): %s", name, mine_.bytes, std::strerror(errno));
        close(fd);
        shm_unlink(name);
        return XCCL_ERR_NO_MEMORY;
    }
    mine_.base = mmap(nullptr, mine_.bytes, PROT_READ | PROT_WRITE, MAP_SHARED, fd, 0);
    close(fd);
    if (mine_.base == MAP_FAILED) {
        mine_.base = nullptr;
        shm_unlink(name);
        return XCCL_ERR_NO_MEMORY;
    }
    std::memset(mine, 0, sizeof(*mine));
    std::snprintf(mine->seg_name, sizeof(mine->seg_name), "%s", name);
    mine->host_hash  = global_state().host_hash;
    mine->ring_bytes = ring_bytes_;
    mine->pid        = (int32_t)getpid();
    return XCCL_OK;
}

xccl_status_t Transport::connect(const PeerInfo *all)
{
    for (int p = 0; p < size_; p++) {
        if (p == rank_) {
            peers_[(size_t)p] = mine_;
            continue;
        }
        if (all[p].host_hash != global_state().host_hash) {
            xccl_error("host team: rank %d is on another host; the shared-memory transport cannot reach it", p);
            return XCCL_ERR_UNREACHABLE;
        }
        if (all[p].ring_bytes != ring_bytes_) {
            xccl_error("host team: rank %d uses a ring of %llu bytes, this rank %zu", p,
                       (unsigned long long)all[p].ring_bytes, ring_bytes_);
            return XCCL_ERR_INVALID_PARAM;
        }
        int fd = shm_open(all[p].seg_name, O_RDWR, 0600);
        if (fd < 0) {
            xccl_error("shm_open(%s): %s", all[p].seg_name, std::strerror(errno));
            return XCCL_ERR_UNREACHABLE;
        }
        Segment s;
        s.bytes = (size_t)size_ * (sizeof(RingCtl) + ring_bytes_);
        s.base  = mmap(nullptr, s.bytes, PROT_READ | PROT_WRITE, MAP_SHARED, fd, 0);
        close(fd);
        if (s.base == MAP_FAILED) return XCCL_ERR_NO_MEMORY;
        peers_[(size_t)p] = s;
        ctl_of(s, rank_)->attached.store(1, std::memory_order_release);
    }
    unlink_when_attached();
    return XCCL_OK;
}

void Transport::send_nb(int peer, const void *buf, size_t len, uint32_t tag, P2pReq *req)
{
    req->done   = false;
    req->status = XCCL_OK;
    outq_[(size_t)peer].push_back(SendOp{(const char *)buf, len, 0, tag, false, req});
    push(peer);
}

void Transport::recv_nb(int peer, void *buf, size_t len, uint32_t tag, P2pReq *req)
{
    req->done   = false;
    req->status = XCCL_OK;
    Inbound &in = in_[(size_t)peer];
    RecvOp   op{(char *)buf, len, tag, req};
    for (auto it = in.unexpected.begin(); it != in.unexpected.end(); ++it) {
        Unexpected *u = it->get();
        if (u->tag != tag || u->claimed != nullptr) continue;
        if (u->complete) {
            if (u->data.size() > len) {
                req->status = XCCL_ERR_MESSAGE_TRUNCATED;
            } else {
                std::memcpy(buf, u->data.data(), u->data.size());
            }
            req->done = true;
            in.unexpected.erase(it);
        } else {
            u->claimed = new RecvOp(op);
        }
        return;
    }
    in.posted.push_back(op);
}

void Transport::push(int peer)
{
    auto    &q    = outq_[(size_t)peer];
    RingCtl *ctl  = ctl_of(peers_[(size_t)peer], rank_);
    char    *ring = data_of(peers_[(size_t)peer], rank_);
    uint64_t tail = ctl->tail.load(std::memory_order_relaxed);
    bool     moved = false;
    while (!q.empty()) {
        SendOp  &op   = q.front();
        uint64_t head = ctl->head.load(std::memory_order_acquire);
        size_t   free_bytes = ring_bytes_ - (size_t)(tail - head);
        if (!op.header_sent) {
            if (free_bytes < sizeof(WireHeader)) break;
            WireHeader h{op.tag, kMagic, (uint64_t)op.len};
            ring_write(ring, ring_bytes_, tail, &h, sizeof(h));
            tail += sizeof(h);
            free_bytes -= sizeof(h);
            op.header_sent = true;
            moved          = true;
        }
        size_t total = wire_len(op.len);
        size_t n     = std::min(free_bytes, total - op.off);
        if (n > 0) {
            if (op.off < op.len) {
                size_t payload = std::min(n, op.len - op.off);
                ring_write(ring, ring_bytes_, tail, op.buf + op.off, payload);
            }
            tail += n;
            op.off += n;
            moved = true;
        }
        if (op.off < total) {
            break;  // ring full
        }
        ctl->tail.store(tail, std::memory_order_release);
        op.req->done = true;
        q.pop_front();
    }
    if (moved) ctl->tail.store(tail, std::memory_order_release);
}

void Transport::finish_message(int peer)
{
    Inbound &in = in_[(size_t)peer];
    if (in.recv != nullptr) {
        in.recv->req->status = in.truncated ? XCCL_ERR_MESSAGE_TRUNCATED : XCCL_OK;
        in.recv->req->done   = true;
        delete in.recv;
        in.recv = nullptr;
    } else if (in.unexp != nullptr) {
        Unexpected *u = in.unexp;
        u->complete   = true;
        if (u->claimed != nullptr) {
            RecvOp *r = u->claimed;
            if (u->data.size() > r->cap) {
                r->req->status = XCCL_ERR_MESSAGE_TRUNCATED;
            } else {
                std::memcpy(r->buf, u->data.data(), u->data.size());
            }
            r->req->done = true;
            delete r;
            u->claimed = nullptr;
            in.unexpected.remove_if([u](const std::unique_ptr<Unexpected> &x) { return x.get() == u; });
        }
        in.unexp = nullptr;
    }
    in.in_msg    = false;
    in.truncated = false;
    in.dest      = nullptr;
}

void Transport::pull(int peer)
{
    Inbound    &in   = in_[(size_t)peer];
    RingCtl    *ctl  = ctl_of(mine_, peer);
    const char *ring = data_of(mine_, peer);
    uint64_t    head = ctl->head.load(std::memory_order_relaxed);
    bool        moved = false;
    for (;;) {
        uint64_t tail  = ctl->tail.load(std::memory_order_acquire);
        size_t   avail = (size_t)(tail - head);
        if (!in.in_msg) {
            if (avail < sizeof(WireHeader)) break;
            WireHeader h;
            ring_read(ring, ring_bytes_, head, &h, sizeof(h));
            head += sizeof(h);
            moved = true;
            if (h.magic != kMagic) {
                xccl_error("host transport: corrupt message header from rank %d", peer);
                break;
            }
            in.in_msg    = true;
            in.msg_len   = (size_t)h.len;
            in.remaining = (size_t)h.len;
            in.pad       = wire_len((size_t)h.len) - (size_t)h.len;
            in.recv      = nullptr;
            in.unexp     = nullptr;
            for (auto it = in.posted.begin(); it != in.posted.end(); ++it) {
                if (it->tag == h.tag) {
                    in.recv = new RecvOp(*it);
                    in.posted.erase(it);
                    break;
                }
            }
            if (in.recv != nullptr) {
                in.truncated = in.msg_len > in.recv->cap;
                in.dest      = in.truncated ? nullptr : in.recv->buf;
            } else {
                auto u = std::make_unique<Unexpected>();
                u->tag = h.tag;
                u->data.resize(in.msg_len);
                in.unexp = u.get();
                in.dest  = u->data.data();
                in.unexpected.push_back(std::move(u));
            }
            continue;
        }
        if (in.remaining > 0) {
            if (avail == 0) break;
            size_t n = std::min(avail, in.remaining);
            if (in.dest != nullptr) {
                ring_read(ring, ring_bytes_, head, in.dest, n);
                in.dest += n;
            }
            head += n;
            in.remaining -= n;
            moved = true;
            ctl->head.store(head, std::memory_order_release);  // free space early for long messages
        }
        if (in.remaining == 0 && in.pad > 0) {
            tail  = ctl->tail.load(std::memory_order_acquire);
            avail = (size_t)(tail - head);
            if (avail == 0) break;
            size_t n = std::min(avail, in.pad);
            head += n;
            in.pad -= n;
            moved = true;
        }
        if (in.remaining == 0 && in.pad == 0) {
            finish_message(peer);
        }
    }
    if (moved) ctl->head.store(head, std::memory_order_release);
}

void Transport::progress()
{
    if (!unlinked_) unlink_when_attached();
    for (int p = 0; p < size_; p++) {
        if (!outq_[(size_t)p].empty()) push(p);
        pull(p);
    }
}

}  // namespace host
}  // namespace xccl
