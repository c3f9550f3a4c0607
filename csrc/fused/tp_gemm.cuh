// Interface of the tensor-parallel GEMM kernels (implemented in tp_gemm.cu).
//
// One persistent, warp-specialised tcgen05 kernel serves four operations:
//   GEMM             C[M,N]   = A[M,K] * B[N,K]^T                         (bf16 in, fp32 accumulate in TMEM)
//   GEMM + SwiGLU    H[M,F]   = silu(A * Wg^T) .* (A * Wu^T)              (gate and up tiles share one accumulator)
//   allgather->GEMM  the A operand is the concatenation of every rank's row shard; CTAs of the
//                    same kernel pull the remote shards over NVLink into local memory and
//                    release them to the MMA pipeline block of rows by block of rows
//   GEMM->reduce-scatter  each output tile is stored straight into the memory of the rank that
//                    owns those rows; when a row block has arrived from every rank its owner adds
//                    the partial tiles up - still inside the same kernel
// Ranks can be real (one process per GPU, peer pointers) or emulated (all ranks in one
// cooperative launch on one GPU, gridDim.y = ranks), exactly like the NVLink collectives.
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "../core/config.h"
#include "../tl/nvlink/nvl_device.cuh"
#include "xccl/xccl.h"

namespace xccl {
namespace tp {

constexpr int kBM = 128, kBN = 256, kBK = 64, kStages = 4;
constexpr int kThreads = 256;           // warp 0: TMA, warp 1: MMA, warps 2-5: epilogue, warps 6-7: copiers (allgather mode)
constexpr int kThreadsFp8 = 384;        // block-scaled fp8: warps 2-9 promote the per-K-block products and run the epilogue, 10-11 copy
constexpr int kMaxTpRanks = 8;

enum Epilogue { EPI_STORE = 0, EPI_SWIGLU = 1 };
enum CommMode { COMM_NONE = 0, COMM_ALLGATHER_A = 1, COMM_REDUCE_SCATTER_C = 2 };

struct GemmParams {
    int M, N, K;          // N counts accumulator columns (gate + up for SwiGLU)
    int epilogue;
    int comm;
    int tp_size;          // ranks taking part (1 without communication)
    int rank_base;        // team rank of blockIdx.y == 0
    int n_gemm_ctas;      // CTAs (per rank) that run MMA tiles; the rest copy (allgather mode, copy_mode 0)
    int copy_mode;        // allgather mode: 0 = whole CTAs set aside for the copy, 1 = two copier warps in every CTA
    int group_rows;       // row blocks of tiles walked together before moving along N (0 = chosen from the shape)
    int group_ramp;       // order of the tile walk while input rows are still arriving from the host.
                          // 1: the groups of the local rows are 1, 1, 2, 4, ... row blocks high, so the first wave of
                          //    tiles needs the first chunk of the copy only;
                          // 2 (allgather mode with copy CTAs): phase c = row block c of EVERY rank's shard (local one
                          //    first) x all column blocks; the copy CTAs pull in the same order, block by block as the
                          //    owners report them landed, so remote tiles start after the first chunks, not after
                          //    the peers' whole shards
    int l2_hint;          // operand loads: 0 no hint, 1 A and B evict_last, 2 A evict_last / B evict_first, 3 the reverse
    int st_stream;        // 1: output stores are marked streaming (evict first)
    // Soft lockstep of the tile walkers: before a tile (and every sync_kblocks K blocks inside it) a walker
    // counts itself into sync_ctr[point] and waits, for at most sync_budget_ns, until all walkers of that
    // point have done so. Walkers that share rows of A or B then ask L2 for the same lines within
    // microseconds of each other; without it they drift apart over many tiles and each fetches from DRAM.
    uint32_t *sync_ctr[kMaxTpRanks];      // per LOCAL rank, zeroed before the launch; null = no lockstep
    int       sync_points;                // counters available
    int       sync_kblocks;               // 0 = only at tile starts
    unsigned  sync_budget_ns;
    uint32_t seq;         // launch sequence number (starts at 1): readiness counters and buffer parity follow it
    uint32_t rs_target;   // reduce-scatter: running total of tiles per (source, row block) for this parity
    int      rs_debug_local;  // diagnostic (wrong results): partial tiles go to local memory and nobody is waited for
    int      rs_fused;    // reduce-scatter: 1 = the tiles of the local rows (walked last) add the other ranks' partial
                          // tiles in their epilogue and write the result; 0 = a reduce phase after the last tile
    unsigned long long budget_ns;
    uint32_t *error;      // device word, 0 = fine
    int ldc;              // leading dimension of the output in elements

    // per LOCAL rank (blockIdx.y)
    __nv_bfloat16 *C[kMaxTpRanks];        // EPI output (COMM_NONE / ALLGATHER) or the reduced shard (REDUCE_SCATTER)
    // allgather mode: xg[r] is rank r's gathered A buffer [M,K] as mapped here; shard s of rank s is valid on entry
    __nv_bfloat16 *xg[kMaxTpRanks];       // indexed by TEAM rank
    uint32_t      *ready[kMaxTpRanks];    // per LOCAL rank: one flag per 128-row block of A, local memory
    // Input rows that are still arriving from the host (optional): the local shard was split into chunks of
    // in_rows_per_flag rows; a stream-ordered 32-bit write sets in_ready[chunk] = in_target after each chunk's
    // host->device copy. Tiles of local rows wait for their chunk; the copy CTAs wait for all chunks before
    // they tell the peers that this rank's shard may be read. Null = the rows are there when the kernel starts.
    const uint32_t *in_ready[kMaxTpRanks];   // per LOCAL rank
    uint32_t        in_target;
    int             in_rows_per_flag;
    // block-scaled fp8 kernels (a_bytes == 1): A is e4m3 with one fp32 scale per row per 128 columns
    int            a_bytes;                // bytes per element of A in xg: 0 or 2 = bf16, 1 = fp8
    float         *sg[kMaxTpRanks];        // TEAM rank: scales of A, [M, K/128]; gathered together with xg in allgather mode
    const float   *sb0[kMaxTpRanks];       // LOCAL rank: scales of B0, [rows/128, K/128]
    const float   *sb1[kMaxTpRanks];       // LOCAL rank: scales of B1 (SwiGLU "up")
    // fp8 SwiGLU: 1 = C is an e4m3 matrix [M, F] (ldc bytes per row) quantised per row and 128 columns in the epilogue,
    // with its scales written to out_scale [M, F / 128]: the activations of the next GEMM, with no pass in between
    int            out_fp8;
    float         *out_scale[kMaxTpRanks]; // LOCAL rank
    // reduce-scatter mode: part[r] = rank r's partial buffer [tp_size][M/tp_size][N] as mapped here
    __nv_bfloat16 *part[kMaxTpRanks];     // indexed by TEAM rank
    uint32_t      *pad[kMaxTpRanks];      // signal pads (TEAM rank) for barriers and arrival counters
};

// Host launcher. tmA / tmB0 / tmB1 are built by make_tensor_map_2d for each local rank.
struct GemmLaunch {
    CUtensorMap tmA[kMaxTpRanks];
    CUtensorMap tmB0[kMaxTpRanks];
    CUtensorMap tmB1[kMaxTpRanks];  // SwiGLU: the "up" weights; otherwise unused
    int         n_local = 1;        // gridDim.y
    int         ctas    = 0;        // gridDim.x; 0 = one per SM (divided among local ranks)
    bool        cooperative = false;
};

// rows x cols bf16 matrix with `ld` elements between rows, tiles of box_rows x 64, 128B swizzle
xccl_status_t make_tensor_map_2d(CUtensorMap *map, const void *base, uint64_t rows, uint64_t cols, uint64_t ld,
                                 uint32_t box_rows);

xccl_status_t launch_gemm(const GemmParams &p, const GemmLaunch &l, cudaStream_t stream);
// The block-scaled fp8 kernel (tp_gemm_fp8.cu): same parameters; tmA / tmB0 / tmB1 are byte maps built by
// make_tensor_map_u8 with boxes of 128 rows (A, plain B) or 64 rows (SwiGLU gate and up halves) x 128 bytes.
xccl_status_t make_tensor_map_u8(CUtensorMap *map, const void *base, uint64_t rows, uint64_t cols, uint32_t box_rows);
xccl_status_t launch_gemm_fp8(const GemmParams &p, const GemmLaunch &l, cudaStream_t stream);

// Tuning options of the fused kernels: the option table "TP_" of the library's configuration system, read once from
// the environment (XCCL_TP_<NAME>) like every other option table and listed by xccl_tp_config_print().
const OptTable &tp_options();

size_t gemm_smem_bytes();
uint32_t *error_word();  // per-device error word shared by the GEMM kernels

}  // namespace tp
}  // namespace xccl

extern "C" {
// Plain C hooks (ctypes). All pointers are device pointers to bf16 row-major matrices.
// C[M,N] = A[M,K] * B[N,K]^T
xccl_status_t xccl_gemm_bf16(const void *A, const void *B, void *C, int M, int N, int K, void *stream);
// H[M,F] = silu(A Wg^T) .* (A Wu^T), Wg and Wu are [F,K]
xccl_status_t xccl_gemm_swiglu_bf16(const void *A, const void *Wg, const void *Wu, void *H, int M, int F, int K,
                                    void *stream);
// Last error word written by a GEMM kernel on the current device (0 = none); clears it.
uint32_t      xccl_gemm_last_error(void);
// Prints the tuning options of the fused kernels (XCCL_TP_*) with their current values and documentation.
void          xccl_tp_config_print(FILE *stream);
}
