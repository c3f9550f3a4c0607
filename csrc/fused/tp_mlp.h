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

// Starts the host->device copy of this step's input shards (host_x[i]: pinned [M/tp, K] bf16 of local rank i) on
// `copy_stream`, chunk by chunk, each chunk followed by a stream-ordered flag write. The NEXT xccl_tp_ag_gemm_swiglu
// call (on its own stream, no event between the two) starts at once and consumes the rows as their chunks land, so
// the copy hides behind the first tiles instead of preceding the kernel.
xccl_status_t xccl_tp_h2d_begin(xccl_tp_ws_h ws, const void *const *host_x, void *copy_stream);
/* The same copy in two calls with the launch of xccl_tp_ag_gemm_swiglu between them (expect, launch, issue): the kernel
 * starts at once and the chunks are enqueued while it already runs. Every `expect` must be followed by the launch and
 * the `issue`: the kernel's waits for the rows are bounded. ramp != 0: the local rows are walked in groups of 1, 1, 2,
 * 4, ... row blocks, so that the first tiles need the first chunk only (a step that starts on an idle GPU); ramp == 2:
 * with copy CTAs, every rank reports its rows block by block and the tiles are walked row block by row block over all
 * shards (every rank of the team must ask for the same). */
xccl_status_t xccl_tp_h2d_expect(xccl_tp_ws_h ws, void *copy_stream, int ramp);
xccl_status_t xccl_tp_h2d_issue(xccl_tp_ws_h ws, const void *const *host_x, void *copy_stream);

// ---- block-scaled fp8 variants (e4m3 activations with 1 x 128 scales, e4m3 weights with 128 x 128 scales)
// The fp8 rows and their scales live in the same gathered buffer as the bf16 rows ([M, K] bytes followed by
// [M, K/128] fp32), so a workspace serves either precision, one at a time.
// out8[rows, K] = e4m3(x / s), scales[rows, K/128] = amax over 128 columns / 448; K % 128 == 0
xccl_status_t xccl_tp_quantize_rows(const void *x_bf16, int rows, int K, void *out8, float *scales, void *stream);
void         *xccl_tp_ws_x8_shard(xccl_tp_ws_h ws, int local_rank);   // [M/tp, K] e4m3: this rank's rows
float        *xccl_tp_ws_sx_shard(xccl_tp_ws_h ws, int local_rank);   // [M/tp, K/128] fp32: their scales
// H[M, F_local] (bf16) = silu(X Wg^T) .* (X Wu^T); Wg8 / Wu8: [F_local, K] e4m3, sWg / sWu: [F_local/128, K/128]
xccl_status_t xccl_tp_ag_gemm_swiglu_fp8(xccl_tp_ws_h ws, const void *const *Wg8, const float *const *sWg,
                                         const void *const *Wu8, const float *const *sWu, void *const *Hout, int F_local,
                                         void *stream);
// The same with the output quantised in the epilogue: H8out[M, F_local] e4m3 and sHout[M, F_local/128] fp32 (1 x 128
// blocks), ready to be the activations of xccl_tp_gemm_rs_fp8 without a pass in between.
xccl_status_t xccl_tp_ag_gemm_swiglu_fp8q(xccl_tp_ws_h ws, const void *const *Wg8, const float *const *sWg,
                                          const void *const *Wu8, const float *const *sWu, void *const *H8out,
                                          float *const *sHout, int F_local, void *stream);
// Y[M/tp, N] (bf16) = reduce-scatter of H8 Wd8^T; H8: [M, F_local] e4m3 with sH [M, F_local/128];
// Wd8: [N, F_local] e4m3 with sWd [N/128, F_local/128]
xccl_status_t xccl_tp_gemm_rs_fp8(xccl_tp_ws_h ws, const void *const *H8, const float *const *sH, const void *const *Wd8,
                                  const float *const *sWd, void *const *Yout, int F_local, void *stream);

#ifdef __cplusplus
}
#endif
