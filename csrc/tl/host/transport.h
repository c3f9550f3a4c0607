// Tagged point-to-point messages between the members of one team over POSIX shared memory.
//
// Every member owns a segment with one single-producer / single-consumer byte ring per peer.
// A message is a 16-byte header {tag, length} followed by the payload, streamed through the
// ring in as many pieces as its free space allows, so messages of any size pass through a
// ring of fixed size. The receiver matches (source, tag) against posted receives in posting
// order; a message that arrives before its receive is kept in an "unexpected" buffer.
// This plays the role UCX tag matching plays for the reference's host team
// (src/team_lib/ucx/xccl_ucx_sendrecv.h:99-239), for ranks of one node.
#pragma once
#include <atomic>
#include <cstdint>
#include <deque>
#include <list>
#include <memory>
#include <string>
#include <vector>

#include "xccl/xccl.h"

namespace xccl {
namespace host {

struct P2pReq {
    bool          done   = true;
    xccl_status_t status = XCCL_OK;
};

struct alignas(64) RingCtl {
    std::atomic<uint64_t> head;  // bytes consumed (receiver writes)
    char                  pad0[56];
    std::atomic<uint64_t> tail;  // bytes produced (sender writes)
    std::atomic<uint32_t> attached;  // the sender has mapped this segment (sender writes, once)
    char                  pad1[52];
};
static_assert(sizeof(RingCtl) == 128, "two cache lines");

struct PeerInfo {  // what members exchange out of band
    char     seg_name[64];
    uint64_t host_hash;
    uint64_t ring_bytes;
    int32_t  pid;
    int32_t  pad;
};

class Transport {
public:
    Transport(int rank, int size, size_t ring_bytes);
    ~Transport();

    xccl_status_t create_local(PeerInfo *mine);          // allocate my segment
    xccl_status_t connect(const PeerInfo *all);          // map every peer's segment

    void send_nb(int peer, const void *buf, size_t len, uint32_t tag, P2pReq *req);
    void recv_nb(int peer, void *buf, size_t len, uint32_t tag, P2pReq *req);
    void progress();

    int rank() const { return rank_; }
    int size() const { return size_; }

private:
    struct Segment {
        void  *base  = nullptr;
        size_t bytes = 0;
    };
    struct SendOp {
        const char *buf;
        size_t      len, off;
        uint32_t    tag;
        bool        header_sent;
        P2pReq     *req;
    };
    struct RecvOp {
        char    *buf;
        size_t   cap;
        uint32_t tag;
        P2pReq  *req;
    };
    struct Unexpected {
        uint32_t          tag;
        std::vector<char> data;
        bool              complete = false;
        RecvOp           *claimed  = nullptr;  // a receive posted while the message was still arriving
    };
    struct Inbound {  // consumer state of the ring that peer p writes into my segment
        bool        in_msg    = false;
        size_t      remaining = 0, pad = 0, msg_len = 0;
        char       *dest      = nullptr;
        RecvOp     *recv      = nullptr;
        Unexpected *unexp     = nullptr;
        bool        truncated = false;
        std::list<RecvOp>                        posted;
        std::list<std::unique_ptr<Unexpected>>   unexpected;
    };

    RingCtl *ctl_of(const Segment &s, int src) const;
    char    *data_of(const Segment &s, int src) const;
    void     push(int peer);
    void     pull(int peer);
    void     finish_message(int peer);

    int                          rank_, size_;
    size_t                       ring_bytes_;
    std::string                  my_name_;
    bool                         unlinked_ = false;  // the segment's name is gone: every peer has it mapped
    void                         unlink_when_attached();
    Segment                      mine_;
    std::vector<Segment>         peers_;     // peers_[p] = p's segment (mine for p == rank)
    std::vector<std::deque<SendOp>> outq_;   // per destination
    std::vector<Inbound>         in_;        // per source
};

}  // namespace host
}  // namespace xccl
