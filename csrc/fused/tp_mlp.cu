// Host side of the fused tensor-parallel MLP operations: owns the symmetric buffers the
// allgather->GEMM and GEMM->reduce-scatter kernels communicate through, builds the TMA
// descriptors and launches tp_gemm_kernel in the matching mode.
//
// Buffers per rank (all in one symmetric region, or plain device memory when emulated):
//   pad    signal pad: barrier flags for the copy CTAs, arrival counters for reduce-scatter
//   xg     [M, K]  gathered activations; rows [r*M/tp, (r+1)*M/tp) are rank r's own shard and are
//          the only rows other ranks ever read
//   part   [2][tp][M/tp][N_rs]  partial output tiles written by every rank, two parities
#include <algorithm>
#include <cstring>
#include <vector>

#include "../core/core.h"
#include "../cuda/cuda_common.h"
#include "../tl/nvlink/nvl_shm.h"
#include "tp_gemm.cuh"
#include "tp_mlp.h"

namespace xccl {
namespace tp {

struct TpWorkspace {
    int  tp = 1, n_local = 1, rank_base = 0;
    int  M = 0, K = 0, N_rs = 0;
    bool emulated = false;
    nvl::SymmetricRegion *region = nullptr;
    std::vector<void *>   allocs;     // emulated buffers
    char     *base[kMaxTpRanks]  = {nullptr};  // per TEAM rank: start of that rank's buffers as mapped here
    uint32_t *ready[kMaxTpRanks] = {nullptr};  // per LOCAL rank
    uint32_t *error = nullptr;
    size_t    off_xg = 0, off_part = 0, total = 0;
    uint32_t  seq_ag = 0, seq_rs = 0, rs_count[2] = {0, 0};
    int       copy_ctas = 16;

    uint32_t      *pad(int r) const { return (uint32_t *)base[r]; }
    __nv_bfloat16 *xg(int r) const { return (__nv_bfloat16 *)(base[r] + off_xg); }
    __nv_bfloat16 *part(int r) const { return (__nv_bfloat16 *)(base[r] + off_part); }
};

namespace {

size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

void layout(TpWorkspace *w)
{
    w->off_xg   = align_up(nvl::kPadBytes, 4096);
    w->off_part = align_up(w->off_xg + (size_t)w->M * w->K * 2, 4096);
    w->total    = align_up(w->off_part + (size_t)2 * w->M * w->N_rs * 2, 4096);
}

}  // namespace

}  // namespace tp
}  // namespace xccl

using namespace xccl;
using namespace xccl::tp;

extern "C" {

xccl_status_t xccl_tp_ws_create(const xccl_oob_collectives_t *oob, int emu_ranks, int M, int K, int N_rs,
                                xccl_tp_ws_h *out)
{
    if (out == nullptr || M <= 0 || K <= 0 || N_rs <= 0) return XCCL_ERR_INVALID_PARAM;
    if (!cuda_available()) return XCCL_ERR_NO_RESOURCE;
    auto *w = new TpWorkspace;
    w->M = M;
    w->K = K;
    w->N_rs = N_rs;
    const char *cc = std::getenv("XCCL_TP_COPY_CTAS");
    if (cc != nullptr && std::atoi(cc) > 0) w->copy_ctas = std::atoi(cc);
    layout(w);
    xccl_status_t st = XCCL_OK;
    if (oob == nullptr) {
        w->emulated  = true;
        w->tp        = std::max(emu_ranks, 1);
        w->n_local   = w->tp;
        w->rank_base = 0;
        if (w->tp > kMaxTpRanks) st = XCCL_ERR_INVALID_PARAM;
        for (int r = 0; r < w->tp && st == XCCL_OK; r++) {
            void *p = nullptr;
            if (cudaMalloc(&p, w->total) != cudaSuccess) {
                (void)cudaGetLastError();
                st = XCCL_ERR_NO_MEMORY;
                break;
            }
            w->allocs.push_back(p);
            cudaMemset(p, 0, nvl::kPadBytes);
            w->base[r] = (char *)p;
        }
    } else {
        w->tp        = oob->size;
        w->n_local   = 1;
        w->rank_base = oob->rank;
        if (w->tp > kMaxTpRanks) {
            st = XCCL_ERR_INVALID_PARAM;
        } else {
            OobGroup g;
            g.oob        = *oob;
            g.range.type = XCCL_EP_RANGE_UNDEFINED;
            g.rank       = oob->rank;
            g.size       = oob->size;
            st           = nvl::SymmetricRegion::create(g, w->total, false, &w->region);
            if (st == XCCL_OK) {
                for (int r = 0; r < w->tp; r++) w->base[r] = w->region->base[(size_t)r];
            }
        }
    }
    int tiles_m = (M + kBM - 1) / kBM;
    if (st == XCCL_OK && (M % kBM != 0 || tiles_m % w->tp != 0)) st = XCCL_ERR_INVALID_PARAM;
    for (int l = 0; l < w->n_local && st == XCCL_OK; l++) {
        void *p = nullptr;
        if (cudaMalloc(&p, (size_t)tiles_m * 4) != cudaSuccess) {
            st = XCCL_ERR_NO_MEMORY;
            break;
        }
        cudaMemset(p, 0, (size_t)tiles_m * 4);
        w->allocs.push_back(p);
        w->ready[l] = (uint32_t *)p;
    }
    if (st == XCCL_OK) {
        void *p = nullptr;
        if (cudaMalloc(&p, 4) != cudaSuccess) {
            st = XCCL_ERR_NO_MEMORY;
        } else {
            cudaMemset(p, 0, 4);
            w->allocs.push_back(p);
            w->error = (uint32_t *)p;
        }
    }
    cudaDeviceSynchronize();
    if (st != XCCL_OK) {
        xccl_tp_ws_destroy(w);
        return st;
    }
    *out = w;
    return XCCL_OK;
}

void xccl_tp_ws_destroy(xccl_tp_ws_h w)
{
    if (w == nullptr) return;
    cudaDeviceSynchronize();
    for (void *p : w->allocs) cudaFree(p);
    delete w->region;
    delete w;
}

void *xccl_tp_ws_x_shard(xccl_tp_ws_h w, int local_rank)
{
    if (w == nullptr || local_rank < 0 || local_rank >= w->n_local) return nullptr;
    int r = w->rank_base + local_rank;
    return w->xg(r) + (size_t)r * (w->M / w->tp) * w->K;
}

void *xccl_tp_ws_x_full(xccl_tp_ws_h w, int local_rank)
{
    if (w == nullptr || local_rank < 0 || local_rank >= w->n_local) return nullptr;
    return w->xg(w->rank_base + local_rank);
}

uint32_t xccl_tp_ws_error(xccl_tp_ws_h w)
{
    uint32_t v = 0;
    if (w == nullptr) return 0xffffffffu;
    cudaMemcpy(&v, w->error, 4, cudaMemcpyDeviceToHost);
    return v;
}

xccl_status_t xccl_tp_ag_gemm_swiglu(xccl_tp_ws_h w, const void *const *Wg, const void *const *Wu, void *const *Hout,
                                     int F_local, void *stream)
{
    if (w == nullptr || Wg == nullptr || Wu == nullptr || Hout == nullptr || F_local % (kBN / 2) != 0) {
        return XCCL_ERR_INVALID_PARAM;
    }
    GemmParams p{};
    GemmLaunch l{};
    p.M = w->M;
    p.N = 2 * F_local;
    p.K = w->K;
    p.epilogue  = EPI_SWIGLU;
    p.comm      = w->tp > 1 ? COMM_ALLGATHER_A : COMM_NONE;
    p.tp_size   = w->tp;
    p.rank_base = w->rank_base;
    p.seq       = ++w->seq_ag;
    p.error     = w->error;
    p.ldc       = F_local;
    int dev = 0, sms = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    int ctas      = sms / w->n_local;
    int copy_ctas = w->tp > 1 ? std::max(1, std::min(w->copy_ctas, ctas / 4)) : 0;
    l.n_local     = w->n_local;
    l.ctas        = ctas;
    l.cooperative = w->tp > 1;
    p.n_gemm_ctas = ctas - copy_ctas;
    for (int r = 0; r < w->tp; r++) {
        p.xg[r]  = w->xg(r);
        p.pad[r] = w->pad(r);
    }
    for (int i = 0; i < w->n_local; i++) {
        p.C[i]     = (__nv_bfloat16 *)Hout[i];
        p.ready[i] = w->ready[i];
        xccl_status_t st = make_tensor_map_2d(&l.tmA[i], w->xg(w->rank_base + i), (uint64_t)w->M, (uint64_t)w->K,
                                              (uint64_t)w->K, kBM);
        if (st != XCCL_OK) return st;
        st = make_tensor_map_2d(&l.tmB0[i], Wg[i], (uint64_t)F_local, (uint64_t)w->K, (uint64_t)w->K, kBN / 2);
        if (st != XCCL_OK) return st;
        st = make_tensor_map_2d(&l.tmB1[i], Wu[i], (uint64_t)F_local, (uint64_t)w->K, (uint64_t)w->K, kBN / 2);
        if (st != XCCL_OK) return st;
    }
    return launch_gemm(p, l, (cudaStream_t)stream);
}

xccl_status_t xccl_tp_gemm_rs(xccl_tp_ws_h w, const void *const *Hin, const void *const *Wd, void *const *Yout,
                              int F_local, void *stream)
{
    if (w == nullptr || Hin == nullptr || Wd == nullptr || Yout == nullptr || F_local % 8 != 0) return XCCL_ERR_INVALID_PARAM;
    GemmParams p{};
    GemmLaunch l{};
    p.M = w->M;
    p.N = w->N_rs;
    p.K = F_local;
    p.epilogue  = EPI_STORE;
    p.comm      = w->tp > 1 ? COMM_REDUCE_SCATTER_C : COMM_NONE;
    p.tp_size   = w->tp;
    p.rank_base = w->rank_base;
    p.seq       = ++w->seq_rs;
    p.error     = w->error;
    p.ldc       = w->N_rs;
    const int tiles_n = (p.N + kBN - 1) / kBN;
    w->rs_count[p.seq & 1] += (uint32_t)tiles_n;
    p.rs_target = w->rs_count[p.seq & 1];
    int dev = 0, sms = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    l.n_local     = w->n_local;
    l.ctas        = sms / w->n_local;
    l.cooperative = w->emulated && w->tp > 1;  // emulated ranks wait on one another inside one launch
    p.n_gemm_ctas = l.ctas;
    for (int r = 0; r < w->tp; r++) {
        p.part[r] = w->part(r);
        p.pad[r]  = w->pad(r);
    }
    for (int i = 0; i < w->n_local; i++) {
        p.C[i] = (__nv_bfloat16 *)Yout[i];
        xccl_status_t st = make_tensor_map_2d(&l.tmA[i], Hin[i], (uint64_t)w->M, (uint64_t)F_local, (uint64_t)F_local, kBM);
        if (st != XCCL_OK) return st;
        st = make_tensor_map_2d(&l.tmB0[i], Wd[i], (uint64_t)w->N_rs, (uint64_t)F_local, (uint64_t)F_local, kBN / 2);
        if (st != XCCL_OK) return st;
        l.tmB1[i] = l.tmB0[i];
    }
    return launch_gemm(p, l, (cudaStream_t)stream);
}

}  // extern "C"
