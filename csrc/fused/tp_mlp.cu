// Host side of the fused tensor-parallel MLP operations: owns the symmetric buffers the
// allgather->GEMM and GEMM->reduce-scatter kernels communicate through, builds the TMA
// descriptors and launches tp_gemm_kernel in the matching mode.
//
// Buffers per rank (all in one symmetric region, or plain device memory when emulated):
//   pad    signal pad: barrier flags for the copy CTAs, arrival counters for reduce-scatter
//   xg     [M, K]  gathered activations; rows [r*M/tp, (r+1)*M/tp) are rank r's own shard and are
//          the only rows other ranks ever read
//   part   [2][tp][M/tp][N_rs]  partial output tiles written by every rank, two parities
#include <cuda_fp8.h>

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
    int       copy_ctas = 0;      // CTAs of the allgather->GEMM kernel that pull the remote shards; 0 = by team size
    int       copy_mode = 1;      // 1: copier warps in every CTA, 0: whole copy CTAs
    bool      rs_debug_local = false;
    bool      rs_fused  = true;   // XCCL_TP_RS_FUSED=0: separate reduce phase after the last tile
    // input rows arriving from the host while the allgather->GEMM kernel already runs
    uint32_t   *in_flags[kMaxTpRanks] = {nullptr};  // per LOCAL rank: one word per chunk of in_rows rows
    uint32_t    in_seq = 0;
    bool        in_active = false;
    int         in_ramp   = 0;      // 1: walk the local rows in growing groups (the kernel starts before the rows are there); 2: phases over all shards
    int         in_rows = 256;
    cudaEvent_t in_consumed = nullptr;

    uint32_t      *pad(int r) const { return (uint32_t *)base[r]; }
    __nv_bfloat16 *xg(int r) const { return (__nv_bfloat16 *)(base[r] + off_xg); }
    __nv_bfloat16 *part(int r) const { return (__nv_bfloat16 *)(base[r] + off_part); }
    // fp8 view of the gathered buffer: [M, K] e4m3 rows, then their [M, K/128] fp32 scales
    float *sx(int r) const { return (float *)(base[r] + off_xg + (size_t)M * K); }
};

namespace {

size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

// One warp per (row, 128-column block): amax by shuffles, four values per lane.
__global__ void __launch_bounds__(256) quantize_rows_1x128_kernel(const __nv_bfloat16 *x, int rows, int K, uint8_t *out,
                                                                  float *scales)
{
    const int    kb_per_row = K / 128;
    const size_t warp  = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) / 32;
    const int    lane  = threadIdx.x % 32;
    const size_t total = (size_t)rows * kb_per_row;
    if (warp >= total) return;
    const size_t row = warp / kb_per_row;
    const int    kb  = (int)(warp % kb_per_row);
    const uint2  raw = *reinterpret_cast<const uint2 *>(x + row * (size_t)K + (size_t)kb * 128 + lane * 4);
    const __nv_bfloat162 *h = reinterpret_cast<const __nv_bfloat162 *>(&raw);
    const float2 a = __bfloat1622float2(h[0]), b = __bfloat1622float2(h[1]);
    float amax = fmaxf(fmaxf(fabsf(a.x), fabsf(a.y)), fmaxf(fabsf(b.x), fabsf(b.y)));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    const float s = fmaxf(amax, 1e-12f) / 448.0f, inv = 1.0f / s;
    uint32_t q = (uint32_t)__nv_cvt_float_to_fp8(a.x * inv, __NV_SATFINITE, __NV_E4M3) |
                 ((uint32_t)__nv_cvt_float_to_fp8(a.y * inv, __NV_SATFINITE, __NV_E4M3) << 8) |
                 ((uint32_t)__nv_cvt_float_to_fp8(b.x * inv, __NV_SATFINITE, __NV_E4M3) << 16) |
                 ((uint32_t)__nv_cvt_float_to_fp8(b.y * inv, __NV_SATFINITE, __NV_E4M3) << 24);
    *reinterpret_cast<uint32_t *>(out + row * (size_t)K + (size_t)kb * 128 + lane * 4) = q;
    if (lane == 0) scales[row * kb_per_row + kb] = s;
}

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
    w->copy_ctas = (int)tp_options().num("COPY_CTAS");
    w->copy_mode = (int)tp_options().num("COPY_MODE");
    w->rs_debug_local = tp_options().flag("RS_DEBUG_LOCAL");
    w->rs_fused  = tp_options().flag("RS_FUSED");
    w->in_rows   = std::max(1, (int)tp_options().num("H2D_CHUNK_ROWS"));
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
    // Copy mode 0 (whole copy CTAs, bulk copies through shared memory): one SM pulls only 16-20 GB/s over NVLink
    // (measured on 8 GPUs: 4 copy CTAs 1.52 ms, 8: 0.92 ms, 16: 0.76 ms for the 8192 x 7168 x 8192 projection whose MMAs
    // take 0.68 ms), so 16 of them are needed to stay ahead of the tile walk, and each costs tensor throughput.
    // Copy mode 1 (two copier warps in every CTA, plain loads) costs no tensor throughput but moves only about
    // 120 GB/s per GPU however many loads it keeps in flight (8 GPUs: 1.12 ms), enough for two ranks (67 MB in 2.5 ms:
    // 4.16 ms per block step against 4.41 ms with copy CTAs), not for eight.
    if (w->copy_ctas <= 0) w->copy_ctas = 16;
    if (w->copy_mode < 0) w->copy_mode = w->tp <= 2 ? 1 : 0;
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
        void  *f = nullptr;
        size_t chunks = (size_t)(M / w->tp + w->in_rows - 1) / w->in_rows;
        if (cudaMalloc(&f, chunks * 4) != cudaSuccess) {
            st = XCCL_ERR_NO_MEMORY;
            break;
        }
        cudaMemset(f, 0, chunks * 4);
        w->allocs.push_back(f);
        w->in_flags[l] = (uint32_t *)f;
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
    if (w->in_consumed != nullptr) cudaEventDestroy(w->in_consumed);
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
    int copy_ctas = (w->tp > 1 && w->copy_mode == 0) ? std::max(1, std::min(w->copy_ctas, ctas / 4)) : 0;
    l.n_local     = w->n_local;
    l.ctas        = ctas;
    l.cooperative = w->tp > 1;
    p.n_gemm_ctas = ctas - copy_ctas;
    p.copy_mode   = w->copy_mode;
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
        if (w->in_active) p.in_ready[i] = w->in_flags[i];
    }
    if (w->in_active) {
        p.in_target        = w->in_seq;
        p.in_rows_per_flag = w->in_rows;
        // H2D_PHASES (with copy CTAs; every rank of the team must run with the same setting): every rank reports its
        // rows block by block and the walk takes row block c of every shard before c + 1. Otherwise the peers' shards
        // are read whole and only the local rows ramp.
        const bool phases  = w->tp > 1 && w->copy_mode == 0 && w->in_ramp == 2;
        p.group_ramp       = w->in_ramp == 0 ? 0 : phases ? 2 : 1;
    }
    xccl_status_t lst = launch_gemm(p, l, (cudaStream_t)stream);
    if (w->in_active && lst == XCCL_OK) {
        // the next host->device copy into the shard may start once this kernel has consumed it
        if (w->in_consumed == nullptr) XCCL_CUDA_CHECK(cudaEventCreateWithFlags(&w->in_consumed, cudaEventDisableTiming));
        XCCL_CUDA_CHECK(cudaEventRecord(w->in_consumed, (cudaStream_t)stream));
    }
    w->in_active = false;
    return lst;
}

// The overlapped input copy in two halves, so that the caller can launch the consuming kernel BETWEEN them: the kernel
// then starts at once and waits for rows, and the host time of issuing the chunks (two driver calls per chunk) is spent
// while the GPU already works. `expect` fixes the sequence number the next allgather->GEMM waits for and orders the copy
// stream after the kernel that read the shard last; `issue` enqueues the chunks and their flag writes. ramp != 0: the
// kernel walks the local rows in groups of 1, 1, 2, 4, ... row blocks, so its first wave needs the first chunk only
// (for a step that starts with an idle GPU; a pipelined caller, whose copy runs under the previous step's second
// kernel, passes 0 and keeps the full groups). ramp == 2 (or the option H2D_PHASES): with copy CTAs, phases over all
// shards as described at GemmParams::group_ramp; every rank of the team must ask for the same.
xccl_status_t xccl_tp_h2d_expect(xccl_tp_ws_h w, void *copy_stream, int ramp)
{
    if (w == nullptr) return XCCL_ERR_INVALID_PARAM;
    if (w->in_active) return XCCL_ERR_NO_RESOURCE;  // one copy per allgather->GEMM
    if (w->in_consumed != nullptr) XCCL_CUDA_CHECK(cudaStreamWaitEvent((cudaStream_t)copy_stream, w->in_consumed, 0));
    w->in_seq++;
    w->in_active = true;
    w->in_ramp   = (ramp == 0 || !tp_options().flag("H2D_RAMP")) ? 0 : (ramp == 2 || tp_options().flag("H2D_PHASES")) ? 2 : 1;
    return XCCL_OK;
}

xccl_status_t xccl_tp_h2d_issue(xccl_tp_ws_h w, const void *const *host_x, void *copy_stream)
{
    if (w == nullptr || host_x == nullptr) return XCCL_ERR_INVALID_PARAM;
    XCCL_DRIVER_FN(cuStreamWriteValue32);
    cudaStream_t cs = (cudaStream_t)copy_stream;
    const size_t rows = (size_t)w->M / w->tp, row_bytes = (size_t)w->K * 2;
    for (int i = 0; i < w->n_local; i++) {
        char       *dst = (char *)xccl_tp_ws_x_shard(w, i);
        const char *src = (const char *)host_x[i];
        size_t      c   = 0;
        for (size_t r0 = 0; r0 < rows; r0 += (size_t)w->in_rows, c++) {
            const size_t n = std::min((size_t)w->in_rows, rows - r0);
            XCCL_CUDA_CHECK(cudaMemcpyAsync(dst + r0 * row_bytes, src + r0 * row_bytes, n * row_bytes, cudaMemcpyHostToDevice, cs));
            XCCL_CU_CHECK(cuStreamWriteValue32((CUstream)cs, (CUdeviceptr)(w->in_flags[i] + c), w->in_seq, 0));
        }
    }
    return XCCL_OK;
}

xccl_status_t xccl_tp_h2d_begin(xccl_tp_ws_h w, const void *const *host_x, void *copy_stream)
{
    xccl_status_t st = xccl_tp_h2d_expect(w, copy_stream, 1);
    return st != XCCL_OK ? st : xccl_tp_h2d_issue(w, host_x, copy_stream);
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
    p.rs_fused  = w->rs_fused ? 1 : 0;
    p.rs_debug_local = w->rs_debug_local ? 1 : 0;
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


xccl_status_t xccl_tp_quantize_rows(const void *x_bf16, int rows, int K, void *out8, float *scales, void *stream)
{
    if (x_bf16 == nullptr || out8 == nullptr || scales == nullptr || rows <= 0 || K <= 0 || K % 128 != 0) {
        return XCCL_ERR_INVALID_PARAM;
    }
    const size_t warps  = (size_t)rows * (K / 128);
    const size_t blocks = (warps * 32 + 255) / 256;
    quantize_rows_1x128_kernel<<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16 *)x_bf16, rows, K,
                                                                                   (uint8_t *)out8, scales);
    XCCL_CUDA_CHECK(cudaGetLastError());
    return XCCL_OK;
}

void *xccl_tp_ws_x8_shard(xccl_tp_ws_h w, int local_rank)
{
    if (w == nullptr || local_rank < 0 || local_rank >= w->n_local) return nullptr;
    int r = w->rank_base + local_rank;
    return (uint8_t *)w->xg(r) + (size_t)r * (w->M / w->tp) * w->K;
}

float *xccl_tp_ws_sx_shard(xccl_tp_ws_h w, int local_rank)
{
    if (w == nullptr || local_rank < 0 || local_rank >= w->n_local || w->K % 128 != 0) return nullptr;
    int r = w->rank_base + local_rank;
    return w->sx(r) + (size_t)r * (w->M / w->tp) * (w->K / 128);
}

xccl_status_t xccl_tp_ag_gemm_swiglu_fp8(xccl_tp_ws_h w, const void *const *Wg8, const float *const *sWg,
                                         const void *const *Wu8, const float *const *sWu, void *const *Hout, int F_local,
                                         void *stream)
{
    return xccl_tp_ag_gemm_swiglu_fp8q(w, Wg8, sWg, Wu8, sWu, Hout, nullptr, F_local, stream);
}

xccl_status_t xccl_tp_ag_gemm_swiglu_fp8q(xccl_tp_ws_h w, const void *const *Wg8, const float *const *sWg,
                                          const void *const *Wu8, const float *const *sWu, void *const *Hout,
                                          float *const *out_scales, int F_local, void *stream)
{
    if (w == nullptr || Wg8 == nullptr || sWg == nullptr || Wu8 == nullptr || sWu == nullptr || Hout == nullptr ||
        F_local % 128 != 0 || w->K % 128 != 0) {
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
    p.ldc       = F_local;   // elements of the output row: bf16 values, or e4m3 bytes with out_scales
    int dev = 0, sms = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    int ctas      = sms / w->n_local;
    int copy_ctas = (w->tp > 1 && w->copy_mode == 0) ? std::max(1, std::min(w->copy_ctas, ctas / 4)) : 0;
    l.n_local     = w->n_local;
    l.ctas        = ctas;
    l.cooperative = w->tp > 1;
    p.n_gemm_ctas = ctas - copy_ctas;
    p.copy_mode   = w->copy_mode;
    if (out_scales != nullptr) p.out_fp8 = 1;
    for (int r = 0; r < w->tp; r++) {
        p.xg[r]  = w->xg(r);
        p.sg[r]  = w->sx(r);
        p.pad[r] = w->pad(r);
    }
    for (int i = 0; i < w->n_local; i++) {
        p.C[i]     = (__nv_bfloat16 *)Hout[i];
        p.ready[i] = w->ready[i];
        p.sb0[i]   = sWg[i];
        p.sb1[i]   = sWu[i];
        xccl_status_t st = make_tensor_map_u8(&l.tmA[i], w->xg(w->rank_base + i), (uint64_t)w->M, (uint64_t)w->K, 128);
        if (st != XCCL_OK) return st;
        st = make_tensor_map_u8(&l.tmB0[i], Wg8[i], (uint64_t)F_local, (uint64_t)w->K, kBN / 2);
        if (st != XCCL_OK) return st;
        st = make_tensor_map_u8(&l.tmB1[i], Wu8[i], (uint64_t)F_local, (uint64_t)w->K, kBN / 2);
        if (st != XCCL_OK) return st;
        if (out_scales != nullptr) p.out_scale[i] = out_scales[i];
    }
    return launch_gemm_fp8(p, l, (cudaStream_t)stream);
}

xccl_status_t xccl_tp_gemm_rs_fp8(xccl_tp_ws_h w, const void *const *H8, const float *const *sH, const void *const *Wd8,
                                  const float *const *sWd, void *const *Yout, int F_local, void *stream)
{
    if (w == nullptr || H8 == nullptr || sH == nullptr || Wd8 == nullptr || sWd == nullptr || Yout == nullptr ||
        F_local % 128 != 0 || w->N_rs % 128 != 0) {
        return XCCL_ERR_INVALID_PARAM;
    }
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
    w->rs_count[p.seq & 1] += (uint32_t)((p.N + kBN - 1) / kBN);  // tiles per row block
    p.rs_target = w->rs_count[p.seq & 1];
    p.rs_fused  = w->rs_fused ? 1 : 0;
    p.rs_debug_local = w->rs_debug_local ? 1 : 0;
    int dev = 0, sms = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    l.n_local     = w->n_local;
    l.ctas        = sms / w->n_local;
    l.cooperative = w->emulated && w->tp > 1;
    p.n_gemm_ctas = l.ctas;
    for (int r = 0; r < w->tp; r++) {
        p.part[r] = w->part(r);
        p.pad[r]  = w->pad(r);
    }
    for (int i = 0; i < w->n_local; i++) {
        p.C[i]   = (__nv_bfloat16 *)Yout[i];
        p.sb0[i] = sWd[i];
        // activation scales are local here: the kernel reads them through the TEAM-rank slot of this local rank
        p.sg[w->rank_base + i] = const_cast<float *>(sH[i]);
        xccl_status_t st = make_tensor_map_u8(&l.tmA[i], H8[i], (uint64_t)w->M, (uint64_t)F_local, 128);
        if (st != XCCL_OK) return st;
        st = make_tensor_map_u8(&l.tmB0[i], Wd8[i], (uint64_t)w->N_rs, (uint64_t)F_local, kBN / 2);
        if (st != XCCL_OK) return st;
        l.tmB1[i] = l.tmB0[i];
    }
    return launch_gemm_fp8(p, l, (cudaStream_t)stream);
}

}  // extern "C"
