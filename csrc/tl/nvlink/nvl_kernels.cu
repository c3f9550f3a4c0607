// NVLink-team collectives for sm_100a: kernels that move and reduce data by loading and
// storing peer GPUs' memory directly (and, for NVLS, through NVSwitch multimem instructions).
//
// Shared structure. Every rank owns a workspace split into two halves that alternate between
// consecutive uses, so a rank may start the next collective while a slower peer still reads the
// previous one. Data is cut into 16-byte packs; block b of every rank works on the same range of
// packs ("piece"), which makes a barrier among the b-th blocks of all ranks sufficient.
//
//   one-shot allreduce   push my vector into slot[my rank] of every peer's workspace, barrier,
//                        reduce the N slots locally                    (latency-bound sizes)
//   two-shot allreduce   copy in, barrier, reduce my 1/N of each piece from all peers' workspaces
//                        in place, barrier, gather the reduced parts   (bandwidth-bound sizes)
//   NVLS allreduce       as two-shot, but the reduction is one multimem.ld_reduce (done in the
//                        switch) and the result is broadcast with multimem.st
//   reduce / reduce-scatter / bcast / allgather / alltoall / alltoallv: copy in, barrier, pull.
//   barrier / fanin / fanout: flag traffic only.
//
// The post-scale and the output cast of xccl_coll_epilogue_t are applied where the reduced value
// is produced, so gradient averaging and fp32->bf16 casting cost no extra pass over memory.
// Baseline these replace: the reference's NCCL team, src/team_lib/nccl/xccl_nccl_collective.c:40-231.
#include <algorithm>

#include "../../cuda/cuda_common.h"
#include "../../cuda/dev_types.cuh"
#include "nvl_kernels.cuh"

namespace xccl {
namespace nvl {

namespace {

using dev::Pack;
using dev::Traits;

#ifdef XCCL_DEBUG_BOUNDS
// Bounds-checking build (python -m xccl_b200.build --debug-bounds -> libxccl_bounds.so). Every 16-byte access of the
// kernels in this file to a workspace, to the multicast mapping or to a peer's registered buffer is checked against
// the address ranges the launch is entitled to (the host writes them into g_dbg before the launch). An access outside
// them is NOT made: it is recorded (how many, the first address, its kind, the block) and skipped, so a wrong index
// shows up as a report and wrong data, never as a fault. xccl_nvlink_debug_bounds_report reads the record.
struct DbgRanges {
    const char *lo[3 * kMaxRanks + 2];
    const char *hi[3 * kMaxRanks + 2];
    int         n;
};
__device__ DbgRanges          g_dbg;
__device__ unsigned long long g_dbg_violation[4];  // count, first address, kind (1 store, 2 load, 3 mc store, 4 mc load), block

__device__ __forceinline__ bool dbg_ok(const void *p, int kind)
{
    const char *a = (const char *)p;
    for (int i = 0; i < g_dbg.n; i++) {
        if (a >= g_dbg.lo[i] && a + 16 <= g_dbg.hi[i]) return true;
    }
    if (atomicAdd(&g_dbg_violation[0], 1ull) == 0ull) {
        g_dbg_violation[1] = (unsigned long long)(uintptr_t)p;
        g_dbg_violation[2] = (unsigned long long)kind;
        g_dbg_violation[3] = ((unsigned long long)blockIdx.y << 32) | blockIdx.x;
    }
    return false;
}
// the unqualified names used by the kernels below resolve to these checked forms
#define st_16(p, v)                                  \
    do {                                             \
        if (dbg_ok((p), 1)) ::xccl::nvl::st_16((p), (v)); \
    } while (0)
#define ld_nc16(p) (dbg_ok((p), 2) ? ::xccl::nvl::ld_nc16(p) : make_uint4(0, 0, 0, 0))
#define mm_st_16(p, v)                                  \
    do {                                                \
        if (dbg_ok((p), 3)) ::xccl::nvl::mm_st_16((p), (v)); \
    } while (0)
#define XCCL_DBG_MC_LOAD_OK(p) dbg_ok((p), 4)
#else
#define XCCL_DBG_MC_LOAD_OK(p) true
#endif

template <typename T> struct Epp {
    static constexpr int value = 16 / (int)sizeof(T);
};

struct Range {
    size_t lo, hi;
};

__device__ __forceinline__ Range block_range(size_t npacks)
{
    size_t per = (npacks + gridDim.x - 1) / gridDim.x;
    size_t lo  = min((size_t)blockIdx.x * per, npacks);
    return Range{lo, min(lo + per, npacks)};
}

// Range of block b in chunk number `chunk` of a chunked kernel that alternates between the two workspace halves.
// Blocks of different index are not ordered with one another, and a half is reused two chunks later: from the third
// chunk on the block ranges are cut from the chunk capacity (the same pack ranges of the half in every chunk), not
// from what the chunk holds, so a block that runs ahead never writes where a block that lags still reads.
__device__ __forceinline__ Range chunk_range(size_t n, size_t cap, size_t chunk)
{
    if (chunk < 2) return block_range(n);
    const Range r = block_range(cap);
    return Range{min(r.lo, n), min(r.hi, n)};
}

__device__ __forceinline__ Range sub_range(Range r, int n, int k)
{
    size_t len = r.hi - r.lo;
    size_t per = (len + n - 1) / n;
    size_t lo  = min(r.lo + (size_t)k * per, r.hi);
    return Range{lo, min(lo + per, r.hi)};
}

template <typename T> __device__ __forceinline__ uint4 as_raw(const Pack<T, Epp<T>::value> &p)
{
    return *reinterpret_cast<const uint4 *>(&p);
}
template <typename T> __device__ __forceinline__ Pack<T, Epp<T>::value> from_raw(uint4 v)
{
    return *reinterpret_cast<Pack<T, Epp<T>::value> *>(&v);
}

// Pack i of an array of `count` elements that may be unaligned or end inside the pack.
template <typename T>
__device__ __forceinline__ uint4 load_pack(const T *p, size_t i, size_t count, bool aligned)
{
    constexpr int E  = Epp<T>::value;
    const size_t  e0 = i * E;
    if (aligned && e0 + E <= count) {
        return *reinterpret_cast<const uint4 *>(p + e0);
    }
    uint4 raw = make_uint4(0, 0, 0, 0);
    T    *v   = reinterpret_cast<T *>(&raw);
#pragma unroll
    for (int e = 0; e < E; e++) {
        if (e0 + e < count) v[e] = p[e0 + e];
    }
    return raw;
}

// Stores E output elements (converted from accumulators) as pack i of `dst`.
template <typename O, int E, typename A>
__device__ __forceinline__ void store_out(O *dst, size_t i, size_t count, bool aligned, const A (&acc)[E])
{
    const size_t e0 = i * E;
    if (aligned && e0 + E <= count) {
        Pack<O, E> out;
#pragma unroll
        for (int e = 0; e < E; e++) out.v[e] = dev::to_out<O>(acc[e]);
        *reinterpret_cast<Pack<O, E> *>(dst + e0) = out;
        return;
    }
#pragma unroll
    for (int e = 0; e < E; e++) {
        if (e0 + e < count) dst[e0 + e] = dev::to_out<O>(acc[e]);
    }
}

template <typename O, int E> __device__ __forceinline__ bool out_aligned(const O *dst)
{
    constexpr size_t a = sizeof(Pack<O, E>) >= 16 ? 16 : sizeof(Pack<O, E>);
    return ((uintptr_t)dst % a) == 0;
}


// Memory-level parallelism. One 16-byte access per thread per iteration keeps only ~8 KB per SM
// in flight, far too little to cover NVLink latency, so every streaming loop issues U loads
// before the first dependent store.
template <int U, typename LoadFn, typename StoreFn>
__device__ __forceinline__ void stream_packs(size_t lo, size_t hi, LoadFn ld, StoreFn st)
{
    const size_t bd = blockDim.x;
    size_t       i  = lo + threadIdx.x;
    for (; i + (U - 1) * bd < hi; i += U * bd) {
        uint4 v[U];
#pragma unroll
        for (int u = 0; u < U; u++) v[u] = ld(i + u * bd);
#pragma unroll
        for (int u = 0; u < U; u++) st(i + u * bd, v[u]);
    }
    for (; i < hi; i += bd) st(i, ld(i));
}

// Reduces pack i of n source arrays (src_of(q) + i * 16) and hands the accumulators to out(i, acc).
// The combination order is q = 0, 1, ... on every rank, so all ranks compute identical bits.
template <typename T, bool kSum, int U, typename SrcFn, typename OutFn>
__device__ __forceinline__ void reduce_packs(SrcFn src_of, int n, size_t lo, size_t hi, int op, OutFn out)
{
    using A         = typename Traits<T>::acc;
    constexpr int E = Epp<T>::value;
    const size_t  bd = blockDim.x;
    size_t        i  = lo + threadIdx.x;
    constexpr int kN = 8;  // sources loaded per batch
    auto one = [&](size_t idx) {
        A acc[E];
        for (int q0 = 0; q0 < n; q0 += kN) {
            uint4 raw[kN];
#pragma unroll
            for (int q = 0; q < kN; q++) {
                if (q0 + q < n) raw[q] = ld_nc16(src_of(q0 + q) + idx * 16);
            }
#pragma unroll
            for (int q = 0; q < kN; q++) {
                if (q0 + q < n) {
                    auto y = from_raw<T>(raw[q]);
                    if (q0 + q == 0) {
#pragma unroll
                        for (int e = 0; e < E; e++) acc[e] = Traits<T>::up(y.v[e]);
                    } else {
#pragma unroll
                        for (int e = 0; e < E; e++) acc[e] = dev::combine<T, kSum>(op, acc[e], Traits<T>::up(y.v[e]));
                    }
                }
            }
        }
        out(idx, acc);
    };
    if (U == 2 && E <= 8 && n <= 4) {
        // few sources: two packs per thread in flight
        for (; i + bd < hi; i += 2 * bd) {
            uint4 ra[4], rb[4];
#pragma unroll
            for (int q = 0; q < 4; q++) {
                if (q < n) {
                    const char *sq = src_of(q);
                    ra[q] = ld_nc16(sq + i * 16);
                    rb[q] = ld_nc16(sq + (i + bd) * 16);
                }
            }
            A acc_a[E], acc_b[E];
#pragma unroll
            for (int q = 0; q < 4; q++) {
                if (q < n) {
                    auto ya = from_raw<T>(ra[q]);
                    auto yb = from_raw<T>(rb[q]);
#pragma unroll
                    for (int e = 0; e < E; e++) {
                        acc_a[e] = (q == 0) ? Traits<T>::up(ya.v[e]) : dev::combine<T, kSum>(op, acc_a[e], Traits<T>::up(ya.v[e]));
                        acc_b[e] = (q == 0) ? Traits<T>::up(yb.v[e]) : dev::combine<T, kSum>(op, acc_b[e], Traits<T>::up(yb.v[e]));
                    }
                }
            }
            out(i, acc_a);
            out(i + bd, acc_b);
        }
    }
    for (; i < hi; i += bd) one(i);
}

// ------------------------------------------------------------------ allreduce: one-shot

template <typename T, typename O, bool kSum>
__global__ void __launch_bounds__(512) allreduce_one_shot_kernel(World w, Call c)
{
    using A          = typename Traits<T>::acc;
    constexpr int E  = Epp<T>::value;
    Self          s  = self_begin(w);
    const T      *src = (const T *)c.src[s.local];
    O            *dst = (O *)c.dst[s.local];
    const size_t  npacks = (c.count + E - 1) / E;
    const size_t  slot   = npacks * 16;
    const size_t  hoff   = (size_t)c.parity * (w.ws_bytes / 2);
    const bool    src_al = ((uintptr_t)src & 15) == 0;
    const bool    dst_al = out_aligned<O, E>(dst);
    const Range   r      = block_range(npacks);

    stream_packs<4>(
        r.lo, r.hi, [&](size_t i) { return load_pack<T>(src, i, c.count, src_al); },
        [&](size_t i, uint4 v) {
            for (int p = 0; p < w.size; p++) st_16(w.ws[p] + hoff + (size_t)s.rank * slot + i * 16, v);
        });
    block_barrier(w, s);
    if (!s.failed) {
        const char *mine = w.ws[s.rank] + hoff;
        reduce_packs<T, kSum, 2>([&](int q) { return mine + (size_t)q * slot; }, w.size, r.lo, r.hi, c.op, [&](size_t i, A(&acc)[E]) {
#pragma unroll
            for (int e = 0; e < E; e++) acc[e] = dev::scaled(acc[e], c.scale, c.do_scale != 0);
            store_out<O, E>(dst, i, c.count, dst_al, acc);
        });
    }
    self_end(w, s);
}

// ------------------------------------------------------------------ allreduce: two-shot and NVLS

template <typename T> __device__ __forceinline__ uint4 nvls_reduce(const void *mc);
template <> __device__ __forceinline__ uint4 nvls_reduce<float>(const void *mc) { return mm_ld_reduce_add_f32x4(mc); }
template <> __device__ __forceinline__ uint4 nvls_reduce<__nv_bfloat16>(const void *mc) { return mm_ld_reduce_add_bf16x8(mc); }
template <> __device__ __forceinline__ uint4 nvls_reduce<__half>(const void *mc) { return mm_ld_reduce_add_f16x8(mc); }
template <typename T> __device__ __forceinline__ uint4 nvls_reduce(const void *) { return make_uint4(0, 0, 0, 0); }

template <typename T, typename O, bool kSum, bool kNvls>
__global__ void __launch_bounds__(512) allreduce_two_shot_kernel(World w, Call c)
{
    using A           = typename Traits<T>::acc;
    constexpr int E   = Epp<T>::value;
    Self          s   = self_begin(w);
    const T      *src = (const T *)c.src[s.local];
    O            *dst = (O *)c.dst[s.local];
    const size_t  npacks = (c.count + E - 1) / E;
    const size_t  half   = w.ws_bytes / 2;
    const size_t  cap    = half / 16;  // packs per chunk
    const bool    src_al = ((uintptr_t)src & 15) == 0;
    const bool    dst_al = out_aligned<O, E>(dst);
    int           parity = c.parity;

    for (size_t c0 = 0; c0 < npacks; c0 += cap, parity ^= 1) {
        const size_t n     = min(cap, npacks - c0);
        const size_t hoff  = (size_t)parity * half;
        const size_t e_off = c0 * E;
        const size_t cnt   = c.count - e_off;  // elements from this chunk's start to the end
        const Range  r     = chunk_range(n, cap, c0 / cap);
        char        *mine  = w.ws[s.rank] + hoff;

        // 1. my input piece -> my workspace
        stream_packs<4>(
            r.lo, r.hi, [&](size_t i) { return load_pack<T>(src + e_off, i, cnt, src_al); },
            [&](size_t i, uint4 v) { st_16(mine + i * 16, v); });
        block_barrier(w, s);
        if (s.failed) break;

        // 2. reduce my share of the piece across all ranks, result in place
        const Range m = sub_range(r, w.size, s.rank);
        if (kNvls) {
            char *mc = w.mc_ws + hoff;
            stream_packs<4>(
                m.lo, m.hi, [&](size_t i) { return XCCL_DBG_MC_LOAD_OK(mc + i * 16) ? nvls_reduce<T>(mc + i * 16) : make_uint4(0, 0, 0, 0); },
                [&](size_t i, uint4 v) {
                    if (c.do_scale) {
                        auto x = from_raw<T>(v);
#pragma unroll
                        for (int e = 0; e < E; e++) x.v[e] = Traits<T>::down(dev::scaled(Traits<T>::up(x.v[e]), c.scale, true));
                        v = as_raw<T>(x);
                    }
                    mm_st_16(mc + i * 16, v);
                });
        } else {
            reduce_packs<T, kSum, 2>([&](int q) { return (const char *)w.ws[q] + hoff; }, w.size, m.lo, m.hi, c.op, [&](size_t i, A(&acc)[E]) {
                Pack<T, E> out;
#pragma unroll
                for (int e = 0; e < E; e++) out.v[e] = Traits<T>::down(dev::scaled(acc[e], c.scale, c.do_scale != 0));
                st_16(mine + i * 16, as_raw<T>(out));
            });
        }
        block_barrier(w, s);
        if (s.failed) break;

        // 3. gather the reduced shares. NVLS already broadcast them into my workspace.
        for (int q = 0; q < w.size; q++) {
            const int   p    = (s.rank + q) % w.size;  // start with my own share, spread the peers
            const Range g    = sub_range(r, w.size, p);
            const char *from = (kNvls ? mine : w.ws[p] + hoff);
            stream_packs<4>(
                g.lo, g.hi, [&](size_t i) { return ld_nc16(from + i * 16); },
                [&](size_t i, uint4 v) {
                    auto x = from_raw<T>(v);
                    A    acc[E];
#pragma unroll
                    for (int e = 0; e < E; e++) acc[e] = Traits<T>::up(x.v[e]);
                    store_out<O, E>(dst + e_off, i, cnt, dst_al, acc);
                });
        }
    }
    self_end(w, s);
}

// ------------------------------------------------------------------ reduce (to root), reduce-scatter

// kNvls: the reducing rank reads each pack once through the multicast mapping (multimem.ld_reduce): the switch fetches
// and adds the N workspaces' copies, so a root takes in S bytes instead of (N - 1) x S.
template <typename T, typename O, bool kSum, bool kScatter, bool kNvls>
__global__ void __launch_bounds__(512) reduce_kernel(World w, Call c)
{
    using A           = typename Traits<T>::acc;
    constexpr int E   = Epp<T>::value;
    Self          s   = self_begin(w);
    const T      *src = (const T *)c.src[s.local];
    O            *dst = (O *)c.dst[s.local];
    const int     nseg   = kScatter ? w.size : 1;  // segments each rank contributes
    const size_t  npacks = (c.count + E - 1) / E;  // packs per segment
    const size_t  half   = w.ws_bytes / 2;
    const size_t  cap    = half / 16 / nseg;
    const bool    dst_al = out_aligned<O, E>(dst);
    const int     my_seg = kScatter ? s.rank : 0;
    const bool    i_reduce = kScatter || s.rank == c.root;
    int           parity = c.parity;

    for (size_t c0 = 0; c0 < npacks; c0 += cap, parity ^= 1) {
        const size_t n     = min(cap, npacks - c0);
        const size_t hoff  = (size_t)parity * half;
        const size_t e_off = c0 * E;
        const size_t cnt   = c.count - e_off;
        const Range  r     = chunk_range(n, cap, c0 / cap);
        const size_t stride = (c0 / cap < 2) ? n : cap;  // packs between segments in the half: fixed once halves are reused
        char        *mine  = w.ws[s.rank] + hoff;
        for (int q = 0; q < nseg; q++) {
            const T   *seg = src + (size_t)q * c.count + e_off;
            const bool al  = ((uintptr_t)seg & 15) == 0;
            stream_packs<4>(
                r.lo, r.hi, [&](size_t i) { return load_pack<T>(seg, i, cnt, al); },
                [&](size_t i, uint4 v) { st_16(mine + ((size_t)q * stride + i) * 16, v); });
        }
        block_barrier(w, s);
        if (s.failed) break;
        if (i_reduce && kNvls) {
            const char *mc = w.mc_ws + hoff + (size_t)my_seg * stride * 16;
            stream_packs<8>(
                r.lo, r.hi, [&](size_t i) { return XCCL_DBG_MC_LOAD_OK(mc + i * 16) ? nvls_reduce<T>(mc + i * 16) : make_uint4(0, 0, 0, 0); },
                [&](size_t i, uint4 v) {
                    auto x = from_raw<T>(v);
                    A    acc[E];
#pragma unroll
                    for (int e = 0; e < E; e++) acc[e] = dev::scaled(Traits<T>::up(x.v[e]), c.scale, c.do_scale != 0);
                    store_out<O, E>(dst + e_off, i, cnt, dst_al, acc);
                });
        } else if (i_reduce) {
            const size_t seg_off = hoff + (size_t)my_seg * stride * 16;
            reduce_packs<T, kSum, 2>([&](int q) { return (const char *)w.ws[q] + seg_off; }, w.size, r.lo, r.hi, c.op, [&](size_t i, A(&acc)[E]) {
#pragma unroll
                for (int e = 0; e < E; e++) acc[e] = dev::scaled(acc[e], c.scale, c.do_scale != 0);
                store_out<O, E>(dst + e_off, i, cnt, dst_al, acc);
            });
        }
    }
    self_end(w, s);
}

// ------------------------------------------------------------------ byte movers

enum MoveKind { MV_BCAST = 0, MV_ALLGATHER = 1, MV_ALLTOALL = 2 };

using Byte = unsigned char;

__device__ __forceinline__ void store_bytes(Byte *dst, size_t i, size_t bytes, bool aligned, uint4 v)
{
    const size_t b0 = i * 16;
    if (aligned && b0 + 16 <= bytes) {
        *reinterpret_cast<uint4 *>(dst + b0) = v;
        return;
    }
    const Byte *s = reinterpret_cast<const Byte *>(&v);
    for (int e = 0; e < 16; e++) {
        if (b0 + e < bytes) dst[b0 + e] = s[e];
    }
}

// kMc (bcast only): the root stores through the multicast mapping, so one store lands in every
// rank's workspace (the switch replicates it) and the others copy out of their OWN workspace.
template <int KIND, bool kMc> __global__ void __launch_bounds__(512) mover_kernel(World w, Call c)
{
    Self          s   = self_begin(w);
    const Byte   *src = (const Byte *)c.src[s.local];
    Byte         *dst = (Byte *)c.dst[s.local];
    const size_t  seg_bytes = (KIND == MV_ALLGATHER) ? c.len / w.size : c.len;
    const int     nseg_ws   = (KIND == MV_ALLTOALL) ? w.size : 1;
    const size_t  npacks    = (seg_bytes + 15) / 16;
    const size_t  half      = w.ws_bytes / 2;
    size_t        cap       = half / 16 / nseg_ws;
    if (KIND == MV_BCAST && kMc && w.mc_bcast_cap != 0) cap = min(cap, w.mc_bcast_cap);  // same rule as chunks_used()
    int           parity    = c.parity;

    for (size_t c0 = 0; c0 < npacks; c0 += cap, parity ^= 1) {
        const size_t n     = min(cap, npacks - c0);
        const size_t hoff  = (size_t)parity * half;
        const size_t b_off = c0 * 16;
        const size_t left  = seg_bytes - b_off;
        const Range  r     = chunk_range(n, cap, c0 / cap);
        const size_t stride = (c0 / cap < 2) ? n : cap;  // packs between segments in the half: fixed once halves are reused
        char        *mine  = w.ws[s.rank] + hoff;

        if (KIND != MV_BCAST || s.rank == c.root) {
            const size_t cnt = r.hi - r.lo;
            if (KIND == MV_ALLTOALL && cnt <= 4 * (size_t)blockDim.x) {
                // short segments: one flat loop over (destination, pack) keeps every load in flight at once
                const bool al = (((uintptr_t)src | seg_bytes) & 15) == 0;
                stream_packs<4>(
                    0, cnt * (size_t)w.size,
                    [&](size_t it) {
                        const uint32_t q = (uint32_t)it / (uint32_t)cnt;
                        return load_pack<Byte>(src + (size_t)q * seg_bytes + b_off, r.lo + (it - q * cnt), left, al);
                    },
                    [&](size_t it, uint4 v) {
                        const uint32_t q = (uint32_t)it / (uint32_t)cnt;
                        st_16(mine + ((size_t)q * stride + r.lo + (it - q * cnt)) * 16, v);
                    });
            } else
            for (int q = 0; q < nseg_ws; q++) {
                const Byte *seg = src + (size_t)q * seg_bytes + b_off;
                const bool  al  = ((uintptr_t)seg & 15) == 0;
                Byte       *own = nullptr;  // bcast root with a separate dst keeps a local copy too
                if (KIND == MV_BCAST && dst != src) own = dst + b_off;
                const bool own_al = ((uintptr_t)own & 15) == 0;
                stream_packs<4>(
                    r.lo, r.hi, [&](size_t i) { return load_pack<Byte>(seg, i, left, al); },
                    [&](size_t i, uint4 v) {
                        if (kMc) {
                            mm_st_16(w.mc_ws + hoff + i * 16, v);
                        } else {
                            st_16(mine + ((size_t)q * stride + i) * 16, v);
                        }
                        if (own != nullptr) store_bytes(own, i, left, own_al, v);
                    });
            }
        }
        block_barrier(w, s);
        if (s.failed) break;

        if (KIND == MV_BCAST) {
            if (s.rank != c.root) {
                Byte      *out = dst + b_off;
                const bool al  = ((uintptr_t)out & 15) == 0;
                const char *from = kMc ? mine : w.ws[c.root] + hoff;
                stream_packs<4>(
                    r.lo, r.hi, [&](size_t i) { return ld_nc16(from + i * 16); },
                    [&](size_t i, uint4 v) { store_bytes(out, i, left, al, v); });
            }
        } else if (r.hi - r.lo <= 4 * (size_t)blockDim.x) {
            // short segments: pull from all peers in one flat loop, so the round trips overlap
            const size_t cnt = r.hi - r.lo;
            const int    seg = (KIND == MV_ALLTOALL) ? s.rank : 0;
            const bool   al  = (((uintptr_t)dst | seg_bytes) & 15) == 0;
            stream_packs<4>(
                0, cnt * (size_t)w.size,
                [&](size_t it) {
                    const uint32_t q = (uint32_t)it / (uint32_t)cnt;
                    const int      p = (s.rank + (int)q) % w.size;
                    return ld_nc16(w.ws[p] + hoff + ((size_t)seg * stride + r.lo + (it - q * cnt)) * 16);
                },
                [&](size_t it, uint4 v) {
                    const uint32_t q = (uint32_t)it / (uint32_t)cnt;
                    const int      p = (s.rank + (int)q) % w.size;
                    store_bytes(dst + (size_t)p * seg_bytes + b_off, r.lo + (it - q * cnt), left, al, v);
                });
        } else {
            for (int q = 0; q < w.size; q++) {
                const int   p    = (s.rank + q) % w.size;
                const int   seg  = (KIND == MV_ALLTOALL) ? s.rank : 0;
                const char *from = w.ws[p] + hoff + (size_t)seg * stride * 16;
                Byte       *out  = dst + (size_t)p * seg_bytes + b_off;
                const bool  al   = ((uintptr_t)out & 15) == 0;
                stream_packs<4>(
                    r.lo, r.hi, [&](size_t i) { return ld_nc16(from + i * 16); },
                    [&](size_t i, uint4 v) { store_bytes(out, i, left, al, v); });
            }
        }
    }
    self_end(w, s);
}

// Push form of allgather / alltoall for messages that fit one workspace half: every rank stores its segments
// straight into slot [its rank] of the DESTINATION ranks' workspaces, the ranks meet at the barrier, and each
// copies its own workspace out. Against the pull form (copy in, barrier, load from the peers) the loads after the
// barrier are local, which takes one NVLink round trip off the latency.
template <int KIND> __global__ void __launch_bounds__(512) push_mover_kernel(World w, Call c)
{
    Self         s   = self_begin(w);
    const Byte  *src = (const Byte *)c.src[s.local];
    Byte        *dst = (Byte *)c.dst[s.local];
    const size_t seg_bytes = (KIND == MV_ALLGATHER) ? c.len / w.size : c.len;
    const size_t n    = (seg_bytes + 15) / 16;
    const size_t hoff = (size_t)c.parity * (w.ws_bytes / 2);
    const Range  r    = block_range(n);
    const size_t cnt  = r.hi - r.lo;
    const bool   src_al = (((uintptr_t)src | seg_bytes) & 15) == 0;
    const bool   dst_al = (((uintptr_t)dst | seg_bytes) & 15) == 0;
    stream_packs<4>(
        0, cnt * (size_t)w.size,
        [&](size_t it) {
            const uint32_t q = (uint32_t)(it / cnt);
            const int      p = (s.rank + (int)q) % w.size;
            return load_pack<Byte>(src + (KIND == MV_ALLTOALL ? (size_t)p * seg_bytes : 0), r.lo + (it - q * cnt), seg_bytes, src_al);
        },
        [&](size_t it, uint4 v) {
            const uint32_t q = (uint32_t)(it / cnt);
            const int      p = (s.rank + (int)q) % w.size;
            st_16(w.ws[p] + hoff + ((size_t)s.rank * n + r.lo + (it - q * cnt)) * 16, v);
        });
    block_barrier(w, s);
    if (!s.failed) {
        const char *mine = w.ws[s.rank] + hoff;
        stream_packs<4>(
            0, cnt * (size_t)w.size,
            [&](size_t it) {
                const uint32_t q = (uint32_t)(it / cnt);
                return ld_nc16(mine + ((size_t)q * n + r.lo + (it - q * cnt)) * 16);
            },
            [&](size_t it, uint4 v) {
                const uint32_t q = (uint32_t)(it / cnt);
                store_bytes(dst + (size_t)q * seg_bytes, r.lo + (it - q * cnt), seg_bytes, dst_al, v);
            });
    }
    self_end(w, s);
}

// alltoallv: any counts. A rank's outgoing segments, each rounded up to a 16-byte pack and laid end to end in
// destination order, form its "stream". Round k stages window k of that stream (cap bytes) in the workspace half
// of alternating parity, the ranks meet at a barrier, and every receiver pulls the part of its segment that lies
// inside the window. A header per block index, written in round 0, publishes the sender's per-destination bytes;
// after the first barrier every block reads all N headers and so knows every stream's length: the number of
// rounds (the longest stream divided by the window) is the same on all ranks without any host exchange.
//
// Who moves what: block b of a sender stages slice b of the window, block b of a receiver pulls what slice b holds
// for it, so the barrier among the b-th blocks orders every byte. Blocks of different index are NOT ordered with one
// another and may drift apart by more than a round; a half is reused two rounds later, so from the third round on the
// slices are the same byte ranges of the half in every round (window / blocks), whatever the window holds. Only the
// first use of each half (rounds 0 and 1) may cut its slices to the bytes actually present, which keeps all blocks
// busy for exchanges smaller than a window.
//
// Whatever the number of rounds, the launch counts as ONE workspace half for the caller's parity bookkeeping: a
// closing barrier after a multi-round exchange makes sure no peer still reads either half when the next
// collective begins.
constexpr size_t kVHeaderBytes = (size_t)kMaxBlocks * kMaxRanks * 4;

// Slice of window k (stream offsets) that block b handles, for a stream of `total` bytes.
__device__ __forceinline__ Range v_slice(size_t total, size_t cap, size_t k, int b, int nblocks)
{
    const size_t w0 = k * cap;
    if (total <= w0) return Range{w0, w0};
    const size_t len   = min(cap, total - w0);
    const size_t basis = (k < 2) ? len : cap;  // bytes the slices are cut from
    const size_t per   = ((basis / 16 + nblocks - 1) / nblocks) * 16;
    const size_t lo    = min(w0 + (size_t)b * per, w0 + len);
    return Range{lo, min(lo + per, w0 + len)};
}

__global__ void __launch_bounds__(512) alltoallv_kernel(World w, Call c)
{
    __shared__ uint32_t sh_hdr[kMaxRanks * kMaxRanks];  // [sender][destination] bytes
    Self            s    = self_begin(w);
    const Byte     *src  = (const Byte *)c.src[s.local];
    Byte           *dst  = (Byte *)c.dst[s.local];
    const uint32_t *meta = c.vmeta[s.local];
    const uint32_t *sc = meta, *sd = meta + w.size, *dc = meta + 2 * w.size, *dd = meta + 3 * w.size;
    const size_t    half = w.ws_bytes / 2;
    const size_t    cap  = (half - kVHeaderBytes) & ~(size_t)15;  // stream bytes per round
    int             parity = c.parity;
    size_t          rounds = 1;
    size_t          my_total = 0;
    for (int q = 0; q < w.size; q++) my_total += (((size_t)sc[q] * c.src_es + 15) / 16) * 16;

    for (size_t k = 0; k < rounds; k++, parity ^= 1) {
        const size_t hoff = (size_t)parity * half;
        char        *mine = w.ws[s.rank] + hoff;
        const size_t w0   = k * cap;
        if (k == 0) {
            uint32_t *hdr = reinterpret_cast<uint32_t *>(mine) + (size_t)blockIdx.x * kMaxRanks;
            if ((int)threadIdx.x < w.size) hdr[threadIdx.x] = sc[threadIdx.x] * (uint32_t)c.src_es;
        }
        // stage my slice of the window: the parts of the outgoing segments that lie inside it
        const Range sl = v_slice(my_total, cap, k, blockIdx.x, gridDim.x);
        size_t      off = 0;
        for (int q = 0; q < w.size && sl.lo < sl.hi; q++) {
            const size_t bytes = (size_t)sc[q] * c.src_es;
            const size_t n     = (bytes + 15) / 16;
            const size_t lo = max(off, sl.lo), hi = min(off + n * 16, sl.hi);
            if (lo < hi) {
                const Byte *seg = src + (size_t)sd[q] * c.src_es;
                const bool  al  = ((uintptr_t)seg & 15) == 0;
                char       *to  = mine + kVHeaderBytes + (off - w0);  // may point before the data area; indexed from lo on
                stream_packs<4>(
                    (lo - off) / 16, (hi - off) / 16, [&](size_t i) { return load_pack<Byte>(seg, i, bytes, al); },
                    [&](size_t i, uint4 v) { st_16(to + i * 16, v); });
            }
            off += n * 16;
        }
        block_barrier(w, s);
        if (s.failed) break;
        if (k == 0) {
            // every sender's header -> shared memory; the longest stream fixes the number of rounds
            for (int t = threadIdx.x; t < w.size * w.size; t += blockDim.x) {
                const int       p  = t / w.size, j = t % w.size;
                const uint32_t *ph = reinterpret_cast<const uint32_t *>(w.ws[p] + hoff) + (size_t)blockIdx.x * kMaxRanks;
                sh_hdr[p * kMaxRanks + j] = ld_relaxed_sys(ph + j);
            }
            __syncthreads();
            size_t longest = 0;
            for (int p = 0; p < w.size; p++) {
                size_t tot = 0;
                for (int j = 0; j < w.size; j++) tot += (((size_t)sh_hdr[p * kMaxRanks + j] + 15) / 16) * 16;
                longest = max(longest, tot);
            }
            rounds = max((size_t)1, (longest + cap - 1) / cap);
        }
        for (int q = 0; q < w.size; q++) {
            const int       p    = (s.rank + q) % w.size;
            const char     *peer = w.ws[p] + hoff;
            const uint32_t *ph   = sh_hdr + p * kMaxRanks;
            size_t          poff = 0, ptotal = 0;
            for (int j = 0; j < w.size; j++) {
                const size_t padded = (((size_t)ph[j] + 15) / 16) * 16;
                if (j < s.rank) poff += padded;
                ptotal += padded;
            }
            const Range  psl   = v_slice(ptotal, cap, k, blockIdx.x, gridDim.x);  // what the sender's block staged
            const size_t sent  = ph[s.rank];
            const size_t want  = (size_t)dc[p] * c.dst_es;
            const size_t bytes = min(sent, want);
            const size_t n     = (sent + 15) / 16;  // the sender's partition
            const size_t lo = max(poff, psl.lo), hi = min(poff + n * 16, psl.hi);
            if (lo >= hi) continue;
            Byte        *out  = dst + (size_t)dd[p] * c.dst_es;
            const bool   al   = ((uintptr_t)out & 15) == 0;
            const char  *from = peer + kVHeaderBytes + (poff - w0);
            stream_packs<4>(
                (lo - poff) / 16, (hi - poff) / 16, [&](size_t i) { return ld_nc16(from + i * 16); },
                [&](size_t i, uint4 v) { store_bytes(out, i, bytes, al, v); });
        }
    }
    if (rounds > 1) block_barrier(w, s);
    self_end(w, s);
}

// ------------------------------------------------------------------ direct (zero-copy) algorithms
// No workspace: the kernels read peers' user buffers and write peers' user buffers. The opening
// barrier tells a block that the same block of every peer has started, hence that the peer's stream
// has produced its source; the closing barrier tells it that every peer has finished reading from and
// writing to this rank's buffers.

// allreduce: rank r owns 1/N of the packs: it loads that share from all N sources, reduces (scale and
// cast fused) and stores the result into all N destinations. In place is safe: a pack is read and
// written by one thread only. reduce-scatter (kScatter): segment r of every source -> local dst.
template <typename T, typename O, bool kSum, bool kScatter>
__global__ void __launch_bounds__(512) direct_reduce_kernel(World w, Call c)
{
    using A           = typename Traits<T>::acc;
    constexpr int E   = Epp<T>::value;
    Self          s   = self_begin(w);
    const size_t  npacks = (c.count + E - 1) / E;
    block_barrier(w, s);
    if (!s.failed) {
        if (kScatter) {
            // count = elements per segment; my segment of every peer
            const Range r   = block_range(npacks);
            O          *dst = (O *)c.dst[s.local];
            const size_t seg_bytes = c.count * sizeof(T);
            reduce_packs<T, kSum, 2>([&](int q) { return (const char *)c.peer_src[q] + (size_t)s.rank * seg_bytes; }, w.size, r.lo,
                                     r.hi, c.op, [&](size_t i, A(&acc)[E]) {
#pragma unroll
                                         for (int e = 0; e < E; e++) acc[e] = dev::scaled(acc[e], c.scale, c.do_scale != 0);
                                         store_out<O, E>(dst, i, c.count, true, acc);
                                     });
        } else {
            const size_t per = (npacks + w.size - 1) / w.size;
            const size_t lo  = min((size_t)s.rank * per, npacks), hi = min(lo + per, npacks);
            const Range  r   = sub_range(Range{lo, hi}, gridDim.x, blockIdx.x);
            reduce_packs<T, kSum, 2>([&](int q) { return (const char *)c.peer_src[q]; }, w.size, r.lo, r.hi, c.op,
                                     [&](size_t i, A(&acc)[E]) {
#pragma unroll
                                         for (int e = 0; e < E; e++) acc[e] = dev::scaled(acc[e], c.scale, c.do_scale != 0);
                                         for (int q = 0; q < w.size; q++) {
                                             const int p = (s.rank + q) % w.size;
                                             store_out<O, E>((O *)c.peer_dst[p], i, c.count, true, acc);
                                         }
                                     });
        }
        block_barrier(w, s);
    }
    self_end(w, s);
}

// allgather / alltoall: pull every peer's contribution straight into the local destination.
template <int KIND> __global__ void __launch_bounds__(512) direct_mover_kernel(World w, Call c)
{
    Self         s   = self_begin(w);
    Byte        *dst = (Byte *)c.dst[s.local];
    const size_t seg_bytes = (KIND == MV_ALLGATHER) ? c.len / w.size : c.len;
    const size_t npacks    = seg_bytes / 16;
    block_barrier(w, s);
    if (!s.failed) {
        const Range r = block_range(npacks);
        for (int q = 0; q < w.size; q++) {
            const int   p    = (s.rank + q) % w.size;
            const char *from = (const char *)c.peer_src[p] + ((KIND == MV_ALLTOALL) ? (size_t)s.rank * seg_bytes : 0);
            char       *out  = (char *)dst + (size_t)p * seg_bytes;
            if (from == out) continue;  // in-place allgather: my own segment is where it belongs
            stream_packs<4>(
                r.lo, r.hi, [&](size_t i) { return ld_nc16(from + i * 16); }, [&](size_t i, uint4 v) { st_16(out + i * 16, v); });
        }
        block_barrier(w, s);
    }
    self_end(w, s);
}

// ------------------------------------------------------------------ symmetric memory: NVLS in place
// The buffers live in allocations of xccl_team_mem_alloc, at the same offset on every rank, and are addressed
// through the multicast mapping. allreduce: rank r owns 1/N of the packs; one multimem.ld_reduce per pack makes the
// switch fetch and add that pack from all N source buffers, one multimem.st writes the (scaled) sum into all N
// destination buffers. Every byte crosses each GPU's links once in each direction and nothing is staged. In place is
// safe: a pack is read and written by one thread of one rank. bcast: the root streams its source through
// multimem.st into every destination.
template <typename T> __global__ void __launch_bounds__(512) symmetric_allreduce_kernel(World w, Call c)
{
    constexpr int E = Epp<T>::value;
    Self          s = self_begin(w);
    const size_t  npacks = c.count / E;
    const char   *src = (const char *)c.mc_src[s.local];
    char         *dst = (char *)c.mc_dst[s.local];
    block_barrier(w, s);  // the same block of every peer has started: the peers' streams have produced their sources
    if (!s.failed) {
        const size_t per = (npacks + w.size - 1) / w.size;
        const size_t lo  = min((size_t)s.rank * per, npacks), hi = min(lo + per, npacks);
        const Range  r   = sub_range(Range{lo, hi}, gridDim.x, blockIdx.x);
        stream_packs<8>(
            r.lo, r.hi, [&](size_t i) { return XCCL_DBG_MC_LOAD_OK(src + i * 16) ? nvls_reduce<T>(src + i * 16) : make_uint4(0, 0, 0, 0); },
            [&](size_t i, uint4 v) {
                if (c.do_scale) {
                    auto x = from_raw<T>(v);
#pragma unroll
                    for (int e = 0; e < E; e++) x.v[e] = Traits<T>::down(dev::scaled(Traits<T>::up(x.v[e]), c.scale, true));
                    v = as_raw<T>(x);
                }
                mm_st_16(dst + i * 16, v);
            });
        block_barrier(w, s);  // every share has been written everywhere; nobody reads a source any more
    }
    self_end(w, s);
}

__global__ void __launch_bounds__(512) symmetric_bcast_kernel(World w, Call c)
{
    Self         s = self_begin(w);
    const size_t npacks = c.len / 16;
    block_barrier(w, s);  // the destinations may be overwritten: every peer has reached this call
    if (!s.failed) {
        if (s.rank == c.root) {
            const char *src = (const char *)c.src[s.local];
            char       *dst = (char *)c.mc_dst[s.local];
            const Range r   = block_range(npacks);
            stream_packs<8>(
                r.lo, r.hi, [&](size_t i) { return *reinterpret_cast<const uint4 *>(src + i * 16); },
                [&](size_t i, uint4 v) { mm_st_16(dst + i * 16, v); });
        }
        block_barrier(w, s);
    }
    self_end(w, s);
}

// ------------------------------------------------------------------ synchronisation only

__global__ void sync_kernel(World w, Call c, int kind)
{
    Self s = self_begin(w);
    if (kind == XCCL_BARRIER) {
        block_barrier(w, s);
    } else {
        s.epoch++;
        int bad = 0;
        const bool to_root = (kind == XCCL_FANIN);
        if (s.rank == c.root) {
            if ((int)threadIdx.x < w.size && (int)threadIdx.x != c.root) {
                if (to_root) {
                    if (!wait_rank(w, s, threadIdx.x, s.epoch)) {
                        record_failure(w, s, NVL_TIMEOUT, threadIdx.x, s.epoch);
                        bad = 1;
                    }
                } else {
                    signal_rank(w, s, threadIdx.x, s.epoch);
                }
            }
        } else if (threadIdx.x == 0) {
            if (to_root) {
                signal_rank(w, s, c.root, s.epoch);
            } else if (!wait_rank(w, s, c.root, s.epoch)) {
                record_failure(w, s, NVL_TIMEOUT, c.root, s.epoch);
                bad = 1;
            }
        }
        s.failed = __syncthreads_or(bad) != 0;
    }
    self_end(w, s);
}

__global__ void timeout_probe_kernel(World w, unsigned long long budget_ns)
{
    Self s = self_begin(w);
    if (threadIdx.x == 0) {
        // the last general counter is reserved for this probe and is never written
        const uint32_t *never = w.pad[s.rank] + kPadCounterOff + kPadCounterWords - 1;
        if (!wait_flag(never, 1u, budget_ns)) record_failure(w, s, NVL_TIMEOUT, s.rank, 1u);
    }
    self_end(w, s);
}

// ------------------------------------------------------------------ launch helpers

#ifdef XCCL_DEBUG_BOUNDS
// Ranges a launch may touch with its 16-byte accesses: every rank's workspace, the multicast mapping, and what the call
// names (registered peer buffers, symmetric buffers through the multicast mapping) with generous but finite extents.
void dbg_set_ranges(const World &w, const Call &c, cudaStream_t stream)
{
    DbgRanges r{};
    auto add = [&](const void *p, size_t bytes) {
        if (p == nullptr || bytes == 0 || r.n >= (int)(sizeof(r.lo) / sizeof(r.lo[0]))) return;
        r.lo[r.n] = (const char *)p;
        r.hi[r.n] = (const char *)p + bytes;
        r.n++;
    };
    for (int p = 0; p < w.size; p++) add(w.ws[p], w.ws_bytes);
    add(w.mc_ws, w.ws_bytes);
    const size_t span = std::max<size_t>(std::max(c.len * (size_t)w.size, c.count * 16 * (size_t)w.size), 16);
    for (int p = 0; p < w.size; p++) {
        add(c.peer_src[p], span);
        add(c.peer_dst[p], span);
    }
    add(c.mc_src[0], span);
    add(c.mc_dst[0], span);
    cudaMemcpyToSymbolAsync(g_dbg, &r, sizeof(r), 0, cudaMemcpyHostToDevice, stream);
}
template <typename... R> void dbg_prepare(cudaStream_t s, World w, Call c, R...) { dbg_set_ranges(w, c, s); }
inline void dbg_prepare(cudaStream_t, World, unsigned long long) {}  // the timeout probe touches no data
#endif

template <typename... Args>
xccl_status_t launch(void (*kernel)(Args...), dim3 grid, dim3 block, bool cooperative, cudaStream_t stream, Args... args)
{
    cudaLaunchConfig_t cfg{};
    cfg.gridDim          = grid;
    cfg.blockDim         = block;
    cfg.dynamicSmemBytes = 0;
    cfg.stream           = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id              = cudaLaunchAttributeCooperative;
    attr[0].val.cooperative = cooperative ? 1 : 0;
    cfg.attrs               = attr;
    cfg.numAttrs            = 1;
#ifdef XCCL_DEBUG_BOUNDS
    dbg_prepare(stream, args...);
#endif
    XCCL_CUDA_CHECK(cudaLaunchKernelEx(&cfg, kernel, args...));
    return XCCL_OK;
}

// How many blocks (per rank) may run: bounded by the pad layout, the work, and - when all ranks
// share one cooperative launch - by what fits on the device at once.
template <typename K>
int pick_blocks(K kernel, const World &w, const LaunchCfg &cfg, size_t packs, int packs_per_thread)
{
    int blocks = cfg.blocks;
    if (blocks <= 0) {
        size_t per_block = (size_t)cfg.threads * (size_t)packs_per_thread;
        blocks           = (int)std::min<size_t>((packs + per_block - 1) / per_block, (size_t)cfg.max_blocks);
    }
    blocks = std::max(1, std::min(blocks, std::min(cfg.max_blocks, kMaxBlocks)));
    if (cfg.cooperative) {
        int dev = 0, sms = 0, per_sm = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, cfg.threads, 0);
        int fit = std::max(1, (sms * std::max(per_sm, 1)) / std::max(w.n_local, 1));
        blocks  = std::min(blocks, fit);
    }
    return blocks;
}

bool reduce_op_ok(xccl_dt_t dt, xccl_op_t op)
{
    bool arith = (op == XCCL_OP_MAX || op == XCCL_OP_MIN || op == XCCL_OP_SUM || op == XCCL_OP_PROD);
    bool logic = (op >= XCCL_OP_AND && op <= XCCL_OP_BXOR);
    bool is_f  = (dt == XCCL_DT_FLOAT16 || dt == XCCL_DT_FLOAT32 || dt == XCCL_DT_FLOAT64 || dt == XCCL_DT_BFLOAT16);
    return is_f ? arith : (arith || logic);
}

template <typename T, typename O>
xccl_status_t allreduce_typed(const World &w, const Call &c, Alg alg, const LaunchCfg &cfg, cudaStream_t stream)
{
    constexpr int E      = Epp<T>::value;
    const size_t  npacks = (c.count + E - 1) / E;
    const bool    sum    = (c.op == XCCL_OP_SUM);
    dim3          block((unsigned)cfg.threads);
    if (alg == ALG_ONE_SHOT) {
        if (npacks * 16 * (size_t)w.size > w.ws_bytes / 2) return XCCL_ERR_BUFFER_TOO_SMALL;
        auto k      = sum ? allreduce_one_shot_kernel<T, O, true> : allreduce_one_shot_kernel<T, O, false>;
        int  blocks = pick_blocks(k, w, cfg, npacks, 1);
        return launch(k, dim3((unsigned)blocks, (unsigned)w.n_local), block, cfg.cooperative, stream, w, c);
    }
    if (alg == ALG_NVLS) {
        constexpr bool can = std::is_same<T, float>::value || std::is_same<T, __half>::value ||
                             std::is_same<T, __nv_bfloat16>::value;
        if (!can || !sum || w.mc_ws == nullptr) return XCCL_ERR_UNSUPPORTED;
        auto k      = allreduce_two_shot_kernel<T, O, true, true>;
        int  blocks = pick_blocks(k, w, cfg, npacks, 2);
        return launch(k, dim3((unsigned)blocks, (unsigned)w.n_local), block, cfg.cooperative, stream, w, c);
    }
    auto k      = sum ? allreduce_two_shot_kernel<T, O, true, false> : allreduce_two_shot_kernel<T, O, false, false>;
    int  blocks = pick_blocks(k, w, cfg, npacks, 2);
    return launch(k, dim3((unsigned)blocks, (unsigned)w.n_local), block, cfg.cooperative, stream, w, c);
}

template <typename T, typename O, bool kScatter>
xccl_status_t reduce_typed(const World &w, const Call &c, const LaunchCfg &cfg, cudaStream_t stream, bool nvls)
{
    constexpr int  E      = Epp<T>::value;
    constexpr bool can    = std::is_same<T, float>::value || std::is_same<T, __half>::value ||
                            std::is_same<T, __nv_bfloat16>::value;
    const size_t   npacks = (c.count + E - 1) / E;
    const bool     sum    = (c.op == XCCL_OP_SUM);
    if (nvls && (!can || !sum || w.mc_ws == nullptr)) return XCCL_ERR_UNSUPPORTED;
    auto k = nvls ? reduce_kernel<T, O, true, kScatter, can>
                  : sum ? reduce_kernel<T, O, true, kScatter, false> : reduce_kernel<T, O, false, kScatter, false>;
    int           blocks = pick_blocks(k, w, cfg, npacks * (kScatter ? w.size : 1), 2);
    return launch(k, dim3((unsigned)blocks, (unsigned)w.n_local), dim3((unsigned)cfg.threads), cfg.cooperative, stream,
                  w, c);
}

}  // namespace

bool direct_shape_ok(int coll, const Call &c, xccl_dt_t dt, int team_size)
{
    auto al = [](const void *p) { return ((uintptr_t)p & 15) == 0; };
    for (int r = 0; r < team_size; r++) {
        if (c.peer_src[r] == nullptr || !al(c.peer_src[r])) return false;
        if (coll == XCCL_ALLREDUCE && (c.peer_dst[r] == nullptr || !al(c.peer_dst[r]))) return false;
    }
    switch (coll) {
    case XCCL_ALLREDUCE:
    case XCCL_REDUCE_SCATTER: return (c.count * xccl_dt_size(dt)) % 16 == 0 && c.count > 0;
    case XCCL_ALLGATHER: return c.len % ((size_t)team_size * 16) == 0 && c.len > 0;
    case XCCL_ALLTOALL: return c.len % 16 == 0 && c.len > 0;
    default: return false;
    }
}

namespace {
template <typename T, typename O, bool kScatter>
xccl_status_t direct_reduce_typed(const World &w, const Call &c, const LaunchCfg &cfg, cudaStream_t stream)
{
    constexpr int E      = Epp<T>::value;
    const size_t  npacks = (c.count + E - 1) / E;
    const bool    sum    = (c.op == XCCL_OP_SUM);
    auto          k      = sum ? direct_reduce_kernel<T, O, true, kScatter> : direct_reduce_kernel<T, O, false, kScatter>;
    const size_t  mine   = kScatter ? npacks : (npacks + w.size - 1) / w.size;
    int           blocks = pick_blocks(k, w, cfg, mine, 2);
    return launch(k, dim3((unsigned)blocks, (unsigned)w.n_local), dim3((unsigned)cfg.threads), cfg.cooperative, stream, w, c);
}
template <bool kScatter>
xccl_status_t direct_reduce_dispatch(const World &w, const Call &c, xccl_dt_t dt, xccl_dt_t out_dt, const LaunchCfg &cfg,
                                     cudaStream_t stream)
{
    if (out_dt == XCCL_DT_UNSUPPORTED || out_dt == XCCL_DT_LAST_PREDEFINED) out_dt = dt;
    if (!reduce_op_ok(dt, (xccl_op_t)c.op)) return XCCL_ERR_UNSUPPORTED;
    // the direct kernels cover the gradient types; everything else keeps the staged kernels
    if (dt == XCCL_DT_FLOAT32 && out_dt == XCCL_DT_FLOAT32) return direct_reduce_typed<float, float, kScatter>(w, c, cfg, stream);
    if (dt == XCCL_DT_FLOAT32 && out_dt == XCCL_DT_BFLOAT16) return direct_reduce_typed<float, __nv_bfloat16, kScatter>(w, c, cfg, stream);
    if (dt == XCCL_DT_BFLOAT16 && out_dt == XCCL_DT_BFLOAT16) return direct_reduce_typed<__nv_bfloat16, __nv_bfloat16, kScatter>(w, c, cfg, stream);
    if (dt == XCCL_DT_FLOAT16 && out_dt == XCCL_DT_FLOAT16) return direct_reduce_typed<__half, __half, kScatter>(w, c, cfg, stream);
    return XCCL_ERR_UNSUPPORTED;
}
}  // namespace

xccl_status_t launch_direct(const World &w, const Call &c, int coll, xccl_dt_t dt, xccl_dt_t out_dt, const LaunchCfg &cfg,
                            cudaStream_t stream)
{
    if (!direct_shape_ok(coll, c, dt, w.size)) return XCCL_ERR_INVALID_PARAM;
    switch (coll) {
    case XCCL_ALLREDUCE: return direct_reduce_dispatch<false>(w, c, dt, out_dt, cfg, stream);
    case XCCL_REDUCE_SCATTER: return direct_reduce_dispatch<true>(w, c, dt, out_dt, cfg, stream);
    case XCCL_ALLGATHER: {
        auto k      = direct_mover_kernel<MV_ALLGATHER>;
        int  blocks = pick_blocks(k, w, cfg, c.len / 16, 4);
        return launch(k, dim3((unsigned)blocks, (unsigned)w.n_local), dim3((unsigned)cfg.threads), cfg.cooperative, stream, w, c);
    }
    case XCCL_ALLTOALL: {
        auto k      = direct_mover_kernel<MV_ALLTOALL>;
        int  blocks = pick_blocks(k, w, cfg, c.len * (size_t)w.size / 16, 4);
        return launch(k, dim3((unsigned)blocks, (unsigned)w.n_local), dim3((unsigned)cfg.threads), cfg.cooperative, stream, w, c);
    }
    default: return XCCL_ERR_UNSUPPORTED;
    }
}

xccl_status_t launch_symmetric(const World &w, const Call &c, int coll, xccl_dt_t dt, const LaunchCfg &cfg, cudaStream_t stream)
{
    auto al = [](const void *p) { return ((uintptr_t)p & 15) == 0; };
    dim3 block((unsigned)cfg.threads);
    if (coll == XCCL_BCAST) {
        if (c.len == 0) return XCCL_OK;
        if (c.len % 16 != 0) return XCCL_ERR_INVALID_PARAM;
        for (int i = 0; i < w.n_local; i++) {
            if (c.mc_dst[i] == nullptr || !al(c.mc_dst[i]) || !al(c.src[i])) return XCCL_ERR_INVALID_PARAM;
        }
        auto k      = symmetric_bcast_kernel;
        int  blocks = pick_blocks(k, w, cfg, c.len / 16, 8);
        return launch(k, dim3((unsigned)blocks, (unsigned)w.n_local), block, cfg.cooperative, stream, w, c);
    }
    if (coll != XCCL_ALLREDUCE || !nvls_supported(dt, (xccl_op_t)c.op)) return XCCL_ERR_UNSUPPORTED;
    if (c.count == 0) return XCCL_OK;
    if ((c.count * xccl_dt_size(dt)) % 16 != 0) return XCCL_ERR_INVALID_PARAM;
    for (int i = 0; i < w.n_local; i++) {
        if (c.mc_src[i] == nullptr || c.mc_dst[i] == nullptr || !al(c.mc_src[i]) || !al(c.mc_dst[i])) return XCCL_ERR_INVALID_PARAM;
    }
    const size_t mine = (c.count * xccl_dt_size(dt) / 16 + w.size - 1) / w.size;
    if (dt == XCCL_DT_FLOAT32) {
        auto k = symmetric_allreduce_kernel<float>;
        return launch(k, dim3((unsigned)pick_blocks(k, w, cfg, mine, 8), (unsigned)w.n_local), block, cfg.cooperative, stream, w, c);
    }
    if (dt == XCCL_DT_BFLOAT16) {
        auto k = symmetric_allreduce_kernel<__nv_bfloat16>;
        return launch(k, dim3((unsigned)pick_blocks(k, w, cfg, mine, 8), (unsigned)w.n_local), block, cfg.cooperative, stream, w, c);
    }
    auto k = symmetric_allreduce_kernel<__half>;
    return launch(k, dim3((unsigned)pick_blocks(k, w, cfg, mine, 8), (unsigned)w.n_local), block, cfg.cooperative, stream, w, c);
}

bool nvls_supported(xccl_dt_t dt, xccl_op_t op)
{
    return op == XCCL_OP_SUM && (dt == XCCL_DT_FLOAT32 || dt == XCCL_DT_FLOAT16 || dt == XCCL_DT_BFLOAT16);
}

size_t one_shot_limit(const World &w) { return w.ws_bytes / 2 / (size_t)std::max(w.size, 1); }

xccl_status_t launch_allreduce(const World &w, const Call &c, xccl_dt_t dt, xccl_dt_t out_dt, Alg alg,
                               const LaunchCfg &cfg, cudaStream_t stream)
{
    if (!reduce_op_ok(dt, (xccl_op_t)c.op)) return XCCL_ERR_UNSUPPORTED;
    if (c.count == 0) return XCCL_OK;
    return XCCL_DISPATCH_IO(dt, out_dt, return (allreduce_typed<T, O>(w, c, alg, cfg, stream)););
}

xccl_status_t launch_reduce(const World &w, const Call &c, xccl_dt_t dt, xccl_dt_t out_dt, const LaunchCfg &cfg,
                            cudaStream_t stream, bool nvls)
{
    if (!reduce_op_ok(dt, (xccl_op_t)c.op)) return XCCL_ERR_UNSUPPORTED;
    if (c.count == 0) return XCCL_OK;
    return XCCL_DISPATCH_IO(dt, out_dt, return (reduce_typed<T, O, false>(w, c, cfg, stream, nvls)););
}

xccl_status_t launch_reduce_scatter(const World &w, const Call &c, xccl_dt_t dt, xccl_dt_t out_dt,
                                    const LaunchCfg &cfg, cudaStream_t stream, bool nvls)
{
    if (!reduce_op_ok(dt, (xccl_op_t)c.op)) return XCCL_ERR_UNSUPPORTED;
    if (c.count == 0) return XCCL_OK;
    return XCCL_DISPATCH_IO(dt, out_dt, return (reduce_typed<T, O, true>(w, c, cfg, stream, nvls)););
}

bool push_fits(const World &w, int coll, size_t len)
{
    const size_t seg = (coll == XCCL_ALLGATHER) ? len / (size_t)w.size : len;
    return ((seg + 15) / 16) * 16 * (size_t)w.size <= w.ws_bytes / 2;
}

template <int KIND, bool kMc = false>
static xccl_status_t mover(const World &w, const Call &c, const LaunchCfg &cfg, cudaStream_t stream)
{
    size_t seg    = (KIND == MV_ALLGATHER) ? c.len / (size_t)w.size : c.len;
    size_t npacks = (seg + 15) / 16;
    if (npacks == 0) return XCCL_OK;
    if (KIND != MV_BCAST && c.push && npacks * 16 * (size_t)w.size <= w.ws_bytes / 2) {
        auto k      = push_mover_kernel<KIND == MV_BCAST ? MV_ALLGATHER : KIND>;
        int  blocks = pick_blocks(k, w, cfg, npacks * (size_t)w.size, 2);
        return launch(k, dim3((unsigned)blocks, (unsigned)w.n_local), dim3((unsigned)cfg.threads), cfg.cooperative, stream,
                      w, c);
    }
    auto k      = mover_kernel<KIND, kMc>;
    int  blocks = pick_blocks(k, w, cfg, npacks * (KIND == MV_BCAST ? 1 : (size_t)w.size), 2);
    return launch(k, dim3((unsigned)blocks, (unsigned)w.n_local), dim3((unsigned)cfg.threads), cfg.cooperative, stream,
                  w, c);
}

xccl_status_t launch_bcast(const World &w, const Call &c, const LaunchCfg &cfg, cudaStream_t stream, bool multicast)
{
    if (multicast) {
        if (w.mc_ws == nullptr) return XCCL_ERR_UNSUPPORTED;
        return mover<MV_BCAST, true>(w, c, cfg, stream);
    }
    return mover<MV_BCAST>(w, c, cfg, stream);
}
xccl_status_t launch_allgather(const World &w, const Call &c, const LaunchCfg &cfg, cudaStream_t stream)
{
    return mover<MV_ALLGATHER>(w, c, cfg, stream);
}
xccl_status_t launch_alltoall(const World &w, const Call &c, const LaunchCfg &cfg, cudaStream_t stream)
{
    return mover<MV_ALLTOALL>(w, c, cfg, stream);
}

xccl_status_t launch_alltoallv(const World &w, const Call &c, size_t max_src_bytes, const LaunchCfg &cfg,
                               cudaStream_t stream)
{
    // The kernel walks the exchange in windows of one workspace half, so any counts are served. Block b of a rank
    // meets block b of every peer, so all ranks must launch the same grid although their byte counts differ:
    // the grid never depends on the counts.
    (void)max_src_bytes;
    if (w.ws_bytes / 2 < kVHeaderBytes + 4096) return XCCL_ERR_BUFFER_TOO_SMALL;
    auto      k = alltoallv_kernel;
    LaunchCfg fixed = cfg;
    if (fixed.blocks <= 0) fixed.blocks = cfg.max_blocks;
    int blocks = pick_blocks(k, w, fixed, 0, 2);
    return launch(k, dim3((unsigned)blocks, (unsigned)w.n_local), dim3((unsigned)cfg.threads), cfg.cooperative, stream,
                  w, c);
}

xccl_status_t launch_sync(const World &w, const Call &c, int kind, const LaunchCfg &cfg, cudaStream_t stream)
{
    return launch(sync_kernel, dim3(1, (unsigned)w.n_local), dim3(32), cfg.cooperative, stream, w, c, kind);
}

xccl_status_t launch_timeout_probe(const World &w, unsigned long long budget_ns, cudaStream_t stream)
{
    return launch(timeout_probe_kernel, dim3(1, (unsigned)w.n_local), dim3(32), false, stream, w, budget_ns);
}

}  // namespace nvl
}  // namespace xccl

// Record of the bounds-checking build: out[0] = accesses that were refused since the last call, out[1] = the first
// refused address, out[2] = its kind (1 store, 2 load, 3 multicast store, 4 multicast load), out[3] = (rank << 32) |
// block. Clears the record. Returns XCCL_ERR_NOT_IMPLEMENTED in a library built without XCCL_DEBUG_BOUNDS.
extern "C" xccl_status_t xccl_nvlink_debug_bounds_report(unsigned long long *out)
{
#ifdef XCCL_DEBUG_BOUNDS
    if (out == nullptr) return XCCL_ERR_INVALID_PARAM;
    XCCL_CUDA_CHECK(cudaDeviceSynchronize());
    XCCL_CUDA_CHECK(cudaMemcpyFromSymbol(out, xccl::nvl::g_dbg_violation, 4 * sizeof(unsigned long long)));
    unsigned long long zero[4] = {0, 0, 0, 0};
    XCCL_CUDA_CHECK(cudaMemcpyToSymbol(xccl::nvl::g_dbg_violation, zero, sizeof(zero)));
    return XCCL_OK;
#else
    (void)out;
    return XCCL_ERR_NOT_IMPLEMENTED;
#endif
}
