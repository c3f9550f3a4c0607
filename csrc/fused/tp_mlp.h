// C interface of the fused tensor-parallel MLP operations (extension; the reference has no GEMM).
//
// A workspace is created collectively by the ranks of a tensor-parallel group (or, with
// oob == NULL, for `emu_ranks` ranks emulated on the current device). Activations are sharded by
// rows: rank r owns rows [r*M/tp, (r+1)*M/tp) and keeps them in its shard slot of the gathered
// buffer (xccl_tp_ws_x_shard). Pointer arrays have one entry per LOCAL rank: one in a real
// group, `emu_ranks` when emulated.
//
//   xccl_tp_ag_gemm_swiglu   H[M, F_local] = silu(X Wg^T) .* (X Wu^T), X = allgather of the shards;
//                            remote shards are fetched over NVLink inside the GEMM kernel
//   xccl_tp_gemm_rs          Y[M/tp, N] = reduce-scatter over ranks of (H[M, F_local] Wd[N, F_local]^T);
//                            partial tiles go straight to the owner's memory from the epilogue
//
// Both kernels bound every wait; xccl_tp_ws_error reads (after a synchronise) the error word,
// 0 when nothing expired. Calls of one workspace must be issued in the same order on every rank
// and on one stream.
#pragma once
#include "xccl/xccl.h"

#ifdef __cplusplus
namespace xccl { namespace tp { struct TpWorkspace; } }
typedef xccl::tp::TpWorkspace *xccl_tp_ws_h;
extern "C" {
#else
typedef struct xccl_tp_workspace *xccl_tp_ws_h;
#endif

xccl_status_t xccl_tp_ws_create(const xccl_oob_collectives_t *oob, int emu_ranks, int M, int K, int N_rs,
                                xccl_tp_ws_h *ws);
void          xccl_tp_ws_destroy(xccl_tp_ws_h ws);
void         *xccl_tp_ws_x_shard(xccl_tp_ws_h ws, int local_rank);  // [M/tp, K] bf16: where this rank's rows live
void         *xccl_tp_ws_x_full(xccl_tp_ws_h ws, int local_rank);   // [M, K] bf16: the gathered buffer
uint32_t      xccl_tp_ws_error(xccl_tp_ws_h ws);
xccl_status_t xccl_tp_ag_gemm_swiglu(xccl_tp_ws_h ws, const void *const *Wg, const void *const *Wu, void *const *Hout,
                                     int F_local, void *stream);
xccl_status_t xccl_tp_gemm_rs(xccl_tp_ws_h ws, const void *const *Hin, const void *const *Wd, void *const *Yout,
                              int F_local, void *stream);

#ifdef __cplusplus
}
#endif
