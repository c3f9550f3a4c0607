// Host collectives as coroutines over the tagged transport.
//
// Algorithm definitions follow the behaviour of the reference's UCX team:
//   recursive k-nomial exchange   src/team_lib/ucx/allreduce/allreduce_knomial.{c,h}
//   scatter-reduce + allgather    src/team_lib/ucx/allreduce/allreduce_sra.c
//   k-nomial trees                src/team_lib/ucx/bcast/bcast_knomial.c, reduce/reduce_knomial.c
//   ring allgather                src/team_lib/ucx/allgather/allgather_ring.c
//   pairwise exchange             src/team_lib/ucx/alltoall/alltoall_pairwise.c, alltoallv/
//   linear variants               bcast_linear.c, reduce_linear.c, fanin_linear.c, fanout_linear.c,
//                                 alltoall_linear_shift.c
// They are re-derived here from those definitions, not transcribed: one function per
// algorithm, written in program order, suspending at XCCL_CO_WAIT.
#include <algorithm>
#include <cstring>

#include "host_tl.h"

namespace xccl {
namespace host {

// ------------------------------------------------------------------ k-nomial layout

KnomialLayout knomial_layout(int rank, int size, int radix)
{
    KnomialLayout l{};
    l.radix = std::max(2, std::min(radix, std::max(size, 2)));
    l.size  = size;
    int p = 0, pw = 1;  // smallest p with radix^p >= size
    while (pw < size) {
        pw *= l.radix;
        p++;
    }
    int full_tree = (pw == size) ? pw : pw / l.radix;
    if (full_tree < 1) full_tree = 1;
    int n_full  = size / full_tree;
    l.full_size = n_full * full_tree;
    l.n_rounds  = p;
    if (pw != size && n_full == 1) l.n_rounds = p - 1;
    l.partner = -1;
    if (rank >= l.full_size) {
        l.role    = KnomialLayout::EXTRA;
        l.partner = rank - l.full_size;
    } else if (rank + l.full_size < size) {
        l.role    = KnomialLayout::PROXY;
        l.partner = rank + l.full_size;
    } else {
        l.role = KnomialLayout::BASE;
    }
    return l;
}

std::vector<int> knomial_peers(const KnomialLayout &l, int rank, int round)
{
    std::vector<int> peers;
    long radix_pow = 1;
    for (int i = 0; i < round; i++) radix_pow *= l.radix;
    long step = radix_pow * l.radix;
    long base = rank - rank % step;
    for (int k = 1; k < l.radix; k++) {
        long peer = (rank + k * radix_pow) % step + base;
        if (peer < l.full_size) peers.push_back((int)peer);
    }
    return peers;
}

namespace {

struct Seg {
    size_t off, cnt;
};
// segment s of a block of B elements cut into n nearly equal parts
inline Seg segment(size_t B, size_t n, size_t s)
{
    size_t q = B / n, rem = B % n;
    return Seg{q * s + std::min(s, rem), q + (s < rem ? 1 : 0)};
}

inline long ipow(int b, int e)
{
    long v = 1;
    while (e-- > 0) v *= b;
    return v;
}

}  // namespace

// ------------------------------------------------------------------ allreduce

Coro allreduce_knomial(HostReq &r)
{
    Bufs         &b = r.b;
    const int     rank = r.team->rank, size = r.team->size;
    KnomialLayout l = knomial_layout(rank, size, r.team->cfg.allreduce_radix);
    if (b.src != b.dst) std::memcpy(b.dst, b.src, b.len);
    if (size == 1) co_return XCCL_OK;

    if (l.role == KnomialLayout::EXTRA) {
        r.send(l.partner, b.dst, b.len);
        r.recv(l.partner, b.dst, b.len);
        XCCL_CO_WAIT(r.all_done());
        co_return XCCL_OK;
    }
    char *tmp = r.scratch((size_t)(l.radix - 1) * b.len);
    if (l.role == KnomialLayout::PROXY) {
        r.recv(l.partner, tmp, b.len);
        XCCL_CO_WAIT(r.all_done());
        xccl_status_t st = r.reduce_multi(b.dst, tmp, b.dst, 1, b.count, b.len);
        if (st != XCCL_OK) co_return st;
    }
    for (int round = 0; round < l.n_rounds; round++) {
        std::vector<int> peers = knomial_peers(l, rank, round);
        if (peers.empty()) continue;
        for (size_t j = 0; j < peers.size(); j++) {
            r.send(peers[j], b.dst, b.len);
            r.recv(peers[j], tmp + j * b.len, b.len);
        }
        XCCL_CO_WAIT(r.all_done());
        xccl_status_t st = r.reduce_multi(b.dst, tmp, b.dst, peers.size(), b.count, b.len);
        if (st != XCCL_OK) co_return st;
    }
    if (l.role == KnomialLayout::PROXY) {
        r.send(l.partner, b.dst, b.len);
        XCCL_CO_WAIT(r.all_done());
    }
    co_return XCCL_OK;
}

Coro allreduce_sra(HostReq &r)
{
    Bufs         &b = r.b;
    const int     rank = r.team->rank, size = r.team->size;
    const size_t  es = xccl_dt_size(b.dt);
    KnomialLayout l  = knomial_layout(rank, size, r.team->cfg.allreduce_radix);
    if (b.src != b.dst) std::memcpy(b.dst, b.src, b.len);
    if (size == 1) co_return XCCL_OK;

    if (l.role == KnomialLayout::EXTRA) {
        r.send(l.partner, b.dst, b.len);
        r.recv(l.partner, b.dst, b.len);
        XCCL_CO_WAIT(r.all_done());
        co_return XCCL_OK;
    }
    char *tmp = r.scratch(b.len + (size_t)(l.radix + 1) * es + 16);
    if (l.role == KnomialLayout::PROXY) {
        r.recv(l.partner, tmp, b.len);
        XCCL_CO_WAIT(r.all_done());
        xccl_status_t st = r.reduce_multi(b.dst, tmp, b.dst, 1, b.count, b.len);
        if (st != XCCL_OK) co_return st;
    }

    struct Frame {
        size_t off, cnt;  // the block this round started from (elements)
        int    round;
    };
    std::vector<Frame> frames;
    size_t             off = 0, cnt = b.count;

    // scatter-reduce: each round keeps 1/step_radix of the current block
    for (int round = 0; round < l.n_rounds; round++) {
        std::vector<int> peers = knomial_peers(l, rank, round);
        if (peers.empty()) continue;
        const long   rp = ipow(l.radix, round), step = rp * l.radix;
        const size_t sr = peers.size() + 1;
        const size_t my_pos = (size_t)((rank % step) / rp);
        const Seg    mine   = segment(cnt, sr, my_pos);
        const size_t slot   = (cnt / sr + 1) * es;  // room for the largest segment
        for (size_t j = 0; j < peers.size(); j++) {
            size_t pos = (size_t)((peers[j] % step) / rp);
            Seg    s   = segment(cnt, sr, pos);
            r.send(peers[j], b.dst + (off + s.off) * es, s.cnt * es);
            r.recv(peers[j], tmp + j * slot, mine.cnt * es);
        }
        XCCL_CO_WAIT(r.all_done());
        char         *seg = b.dst + (off + mine.off) * es;
        xccl_status_t st  = r.reduce_multi(seg, tmp, seg, peers.size(), mine.cnt, slot);
        if (st != XCCL_OK) co_return st;
        frames.push_back(Frame{off, cnt, round});
        off += mine.off;
        cnt = mine.cnt;
    }
    // allgather: replay the rounds backwards, every member returns its reduced segment
    while (!frames.empty()) {
        Frame            f     = frames.back();
        std::vector<int> peers = knomial_peers(l, rank, f.round);
        const long       rp = ipow(l.radix, f.round), step = rp * l.radix;
        const size_t     sr = peers.size() + 1;
        frames.pop_back();
        for (size_t j = 0; j < peers.size(); j++) {
            size_t pos = (size_t)((peers[j] % step) / rp);
            Seg    s   = segment(f.cnt, sr, pos);
            r.send(peers[j], b.dst + off * es, cnt * es);
            r.recv(peers[j], b.dst + (f.off + s.off) * es, s.cnt * es);
        }
        XCCL_CO_WAIT(r.all_done());
        off = f.off;
        cnt = f.cnt;
    }
    if (l.role == KnomialLayout::PROXY) {
        r.send(l.partner, b.dst, b.len);
        XCCL_CO_WAIT(r.all_done());
    }
    co_return XCCL_OK;
}

// ------------------------------------------------------------------ reduce

Coro reduce_knomial(HostReq &r)
{
    Bufs     &b = r.b;
    const int rank = r.team->rank, size = r.team->size;
    const int radix = std::max(2, std::min(r.team->cfg.reduce_radix, std::max(size, 2)));
    const int vrank = (rank - b.root + size) % size;
    // non-roots accumulate in scratch: dst is only significant at the root
    char *tmp  = r.scratch((size_t)radix * b.len);
    char *work = (rank == b.root) ? b.dst : tmp + (size_t)(radix - 1) * b.len;
    if (work != b.src) std::memcpy(work, b.src, b.len);
    for (long dist = 1; dist < size; dist *= radix) {
        if (vrank % dist != 0) break;
        int pos = (int)((vrank / dist) % radix);
        if (pos > 0) {
            int parent = (int)((vrank - pos * dist + b.root) % size);
            r.send(parent, work, b.len);
            XCCL_CO_WAIT(r.all_done());
            break;
        }
        size_t n = 0;
        for (int i = radix - 1; i >= 1; i--) {
            long child = vrank + i * dist;
            if (child >= size) continue;
            r.recv((int)((child + b.root) % size), tmp + n * b.len, b.len);
            n++;
        }
        if (n == 0) continue;
        XCCL_CO_WAIT(r.all_done());
        xccl_status_t st = r.reduce_multi(work, tmp, work, n, b.count, b.len);
        if (st != XCCL_OK) co_return st;
    }
    co_return XCCL_OK;
}

Coro reduce_linear(HostReq &r)
{
    Bufs     &b = r.b;
    const int rank = r.team->rank, size = r.team->size;
    if (rank != b.root) {
        r.send(b.root, b.src, b.len);
        XCCL_CO_WAIT(r.all_done());
        co_return XCCL_OK;
    }
    if (b.src != b.dst) std::memcpy(b.dst, b.src, b.len);
    char *tmp = r.scratch(b.len);
    for (int p = 0; p < size; p++) {
        if (p == rank) continue;
        r.recv(p, tmp, b.len);
        XCCL_CO_WAIT(r.all_done());
        xccl_status_t st = r.reduce_multi(b.dst, tmp, b.dst, 1, b.count, b.len);
        if (st != XCCL_OK) co_return st;
    }
    co_return XCCL_OK;
}

// ------------------------------------------------------------------ bcast

Coro bcast_knomial(HostReq &r)
{
    Bufs     &b = r.b;
    const int rank = r.team->rank, size = r.team->size;
    const int radix = std::max(2, std::min(r.team->cfg.bcast_radix, std::max(size, 2)));
    const int vrank = (rank - b.root + size) % size;
    if (rank == b.root && b.src != b.dst) std::memcpy(b.dst, b.src, b.len);
    long dist_max = 1;
    while (dist_max * radix < size) dist_max *= radix;
    for (long dist = dist_max; dist >= 1; dist /= radix) {
        if (vrank % dist != 0) continue;
        int pos = (int)((vrank / dist) % radix);
        if (pos > 0) {
            r.recv((int)((vrank - pos * dist + b.root) % size), b.dst, b.len);
            XCCL_CO_WAIT(r.all_done());
        } else {
            for (int i = radix - 1; i >= 1; i--) {
                long child = vrank + i * dist;
                if (child < size) r.send((int)((child + b.root) % size), b.dst, b.len);
            }
        }
    }
    XCCL_CO_WAIT(r.all_done());
    co_return XCCL_OK;
}

Coro bcast_linear(HostReq &r)
{
    Bufs     &b = r.b;
    const int rank = r.team->rank, size = r.team->size;
    if (rank == b.root) {
        if (b.src != b.dst) std::memcpy(b.dst, b.src, b.len);
        for (int p = 0; p < size; p++) {
            if (p != rank) r.send(p, b.dst, b.len);
        }
    } else {
        r.recv(b.root, b.dst, b.len);
    }
    XCCL_CO_WAIT(r.all_done());
    co_return XCCL_OK;
}

// ------------------------------------------------------------------ barrier, fanin, fanout

Coro barrier_knomial(HostReq &r)
{
    const int     rank = r.team->rank, size = r.team->size;
    KnomialLayout l = knomial_layout(rank, size, r.team->cfg.barrier_radix);
    if (size == 1) co_return XCCL_OK;
    if (l.role == KnomialLayout::EXTRA) {
        r.send(l.partner, nullptr, 0);
        r.recv(l.partner, nullptr, 0);
        XCCL_CO_WAIT(r.all_done());
        co_return XCCL_OK;
    }
    if (l.role == KnomialLayout::PROXY) {
        r.recv(l.partner, nullptr, 0);
        XCCL_CO_WAIT(r.all_done());
    }
    for (int round = 0; round < l.n_rounds; round++) {
        for (int peer : knomial_peers(l, rank, round)) {
            r.send(peer, nullptr, 0);
            r.recv(peer, nullptr, 0);
        }
        XCCL_CO_WAIT(r.all_done());
    }
    if (l.role == KnomialLayout::PROXY) {
        r.send(l.partner, nullptr, 0);
        XCCL_CO_WAIT(r.all_done());
    }
    co_return XCCL_OK;
}

Coro fanin_linear(HostReq &r)
{
    const int rank = r.team->rank, size = r.team->size, root = r.b.root;
    if (rank == root) {
        for (int p = 0; p < size; p++) {
            if (p != root) r.recv(p, nullptr, 0);
        }
    } else {
        r.send(root, nullptr, 0);
    }
    XCCL_CO_WAIT(r.all_done());
    co_return XCCL_OK;
}

Coro fanout_linear(HostReq &r)
{
    const int rank = r.team->rank, size = r.team->size, root = r.b.root;
    if (rank == root) {
        for (int p = 0; p < size; p++) {
            if (p != root) r.send(p, nullptr, 0);
        }
    } else {
        r.recv(root, nullptr, 0);
    }
    XCCL_CO_WAIT(r.all_done());
    co_return XCCL_OK;
}

// ------------------------------------------------------------------ allgather

Coro allgather_ring(HostReq &r)
{
    Bufs        &b = r.b;
    const int    rank = r.team->rank, size = r.team->size;
    const size_t block = b.len / (size_t)size;
    char        *mine  = b.dst + (size_t)rank * block;
    if (b.src != mine && r.args.buffer_info.src_buffer != XCCL_IN_PLACE) std::memcpy(mine, b.src, block);
    const int next = (rank + 1) % size, prev = (rank - 1 + size) % size;
    for (int s = 0; s < size - 1; s++) {
        int sblock = (rank - s + size) % size;
        int rblock = (rank - s - 1 + 2 * size) % size;
        r.send(next, b.dst + (size_t)sblock * block, block);
        r.recv(prev, b.dst + (size_t)rblock * block, block);
        XCCL_CO_WAIT(r.all_done());
        r.drop_completed();
    }
    co_return XCCL_OK;
}

// ------------------------------------------------------------------ alltoall(v)

namespace {

// Shared body of alltoall and alltoallv: `sbuf_of(p)`/`rbuf_of(p)` give address and byte count.
template <typename SendOf, typename RecvOf>
Coro pairwise_exchange(HostReq &r, SendOf sbuf_of, RecvOf rbuf_of)
{
    const int  rank = r.team->rank, size = r.team->size;
    const auto &cfg = r.team->cfg;
    {
        auto [sp, sn] = sbuf_of(rank);
        auto [rp, rn] = rbuf_of(rank);
        if (sp != rp) std::memcpy(rp, sp, std::min(sn, rn));
    }
    const int window = (cfg.a2a_chunk > 0 && cfg.a2a_chunk <= size - 1) ? cfg.a2a_chunk : size - 1;
    std::deque<std::pair<P2pReq *, P2pReq *>> inflight;
    for (int s = 0; s < size - 1; s++) {
        while ((int)inflight.size() >= window) {
            XCCL_CO_WAIT((r.progress(), inflight.front().first->done && inflight.front().second->done));
            if (inflight.front().first->status != XCCL_OK) co_return inflight.front().first->status;
            if (inflight.front().second->status != XCCL_OK) co_return inflight.front().second->status;
            inflight.pop_front();
        }
        int rpeer = (rank + 1 + s) % size;
        int speer = (rank - 1 - s + 2 * size) % size;
        if (cfg.a2a_reverse) std::swap(rpeer, speer);
        auto [sp, sn] = sbuf_of(speer);
        auto [rp, rn] = rbuf_of(rpeer);
        P2pReq *rq    = r.recv(rpeer, rp, rn);
        P2pReq *sq    = r.send(speer, sp, sn);
        inflight.emplace_back(sq, rq);
        if (cfg.a2a_barrier > 0 && (s + 1) % cfg.a2a_barrier == 0 && s + 1 < size - 1) {
            XCCL_CO_WAIT(r.all_done());
            inflight.clear();
            XCCL_CO_CALL(barrier_knomial(r));
        }
    }
    XCCL_CO_WAIT(r.all_done());
    co_return XCCL_OK;
}

}  // namespace

Coro alltoall_pairwise(HostReq &r)
{
    Bufs &b = r.b;
    auto  s = [&b](int p) { return std::pair<char *, size_t>(b.src + (size_t)p * b.len, b.len); };
    auto  d = [&b](int p) { return std::pair<char *, size_t>(b.dst + (size_t)p * b.len, b.len); };
    return pairwise_exchange(r, s, d);
}

Coro alltoallv_pairwise(HostReq &r)
{
    Bufs &b = r.b;
    auto  s = [&b](int p) {
        return std::pair<char *, size_t>(b.src + (size_t)b.src_displs[(size_t)p] * b.src_dt_size,
                                         (size_t)b.src_counts[(size_t)p] * b.src_dt_size);
    };
    auto d = [&b](int p) {
        return std::pair<char *, size_t>(b.dst + (size_t)b.dst_displs[(size_t)p] * b.dst_dt_size,
                                         (size_t)b.dst_counts[(size_t)p] * b.dst_dt_size);
    };
    return pairwise_exchange(r, s, d);
}

// In-place alltoall: in step s rank i is paired with (s - i) mod N; the outgoing block is
// staged in scratch so the incoming one can land in its place.
Coro alltoall_linear_shift(HostReq &r)
{
    Bufs     &b = r.b;
    const int rank = r.team->rank, size = r.team->size;
    char     *tmp  = r.scratch(b.len);
    if (b.src != b.dst) std::memcpy(b.dst, b.src, b.len * (size_t)size);
    for (int s = 0; s < size; s++) {
        int peer = (s - rank + 2 * size) % size;
        if (peer == rank) continue;
        char *blk = b.dst + (size_t)peer * b.len;
        std::memcpy(tmp, blk, b.len);
        r.send(peer, tmp, b.len);
        r.recv(peer, blk, b.len);
        XCCL_CO_WAIT(r.all_done());
        r.drop_completed();
    }
    co_return XCCL_OK;
}

// ------------------------------------------------------------------ reduce-scatter (extension)

Coro reduce_scatter_pairwise(HostReq &r)
{
    Bufs        &b = r.b;
    const int    rank = r.team->rank, size = r.team->size;
    const size_t block = b.len / (size_t)size, cnt = b.count;
    char        *tmp   = r.scratch(block * (size_t)size);
    size_t       n     = 0;
    for (int s = 1; s < size; s++) {
        int to = (rank + s) % size, from = (rank - s + size) % size;
        r.send(to, b.src + (size_t)to * block, block);
        r.recv(from, tmp + n * block, block);
        n++;
    }
    XCCL_CO_WAIT(r.all_done());
    xccl_status_t st = r.reduce_multi(b.src + (size_t)rank * block, tmp, b.dst, n, cnt, block);
    co_return st;
}

}  // namespace host
}  // namespace xccl

extern "C" int xccl_host_knomial_peers(int rank, int size, int radix, int round, int *out, int *role, int *n_rounds,
                                       int *partner)
{
    auto l = xccl::host::knomial_layout(rank, size, radix);
    if (role != nullptr) *role = (int)l.role;
    if (n_rounds != nullptr) *n_rounds = l.n_rounds;
    if (partner != nullptr) *partner = l.partner;
    if (round < 0 || round >= l.n_rounds || l.role == xccl::host::KnomialLayout::EXTRA) return 0;
    auto peers = xccl::host::knomial_peers(l, rank, round);
    for (size_t i = 0; i < peers.size(); i++) out[i] = peers[i];
    return (int)peers.size();
}
