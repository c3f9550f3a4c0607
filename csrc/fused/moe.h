// C interface of the fused MoE dispatch / combine kernels (extension).
//
// Experts are sharded E / ranks per rank; expert e lives on rank e / (E / ranks). A workspace is
// created collectively (or, with oob == NULL, for `emu_ranks` ranks emulated on the current
// device). Pointer arrays have one entry per LOCAL rank.
//
//   xccl_moe_dispatch(x[T,H] bf16, ids[T,K] int32)   rows of x land in the owners' RECV buffers,
//        grouped by (local expert, source rank); EXPERT_ROWS says how many rows each local expert
//        received (last entry: total). Ids outside [0, E) are dropped.
//   ... the caller runs its experts over RECV and writes EXPERT_OUT at the same row numbers ...
//   xccl_moe_combine(ids, weights[T,K] fp32, out[T,H] bf16)   out[t] = sum_k w[t,k] * EXPERT_OUT of
//        the row that token t's k-th choice was sent to, pulled from the owner.
// cap_rows <= 0 sizes the buffers for the worst case (every routed row of every rank on one rank).
#pragma once
#include <stdint.h>

#include "xccl/xccl.h"

#ifdef __cplusplus
namespace xccl { namespace moe { struct MoeWorkspace; } }
typedef xccl::moe::MoeWorkspace *xccl_moe_ws_h;
extern "C" {
#else
typedef struct xccl_moe_workspace *xccl_moe_ws_h;
#endif

enum { XCCL_MOE_BUF_RECV = 0, XCCL_MOE_BUF_EXPERT_OUT = 1, XCCL_MOE_BUF_EXPERT_ROWS = 2, XCCL_MOE_BUF_ROW_SOURCE = 3 };

xccl_status_t xccl_moe_ws_create(const xccl_oob_collectives_t *oob, int emu_ranks, int T, int H, int E, int K,
                                 int cap_rows, xccl_moe_ws_h *ws);
void          xccl_moe_ws_destroy(xccl_moe_ws_h ws);
xccl_status_t xccl_moe_dispatch(xccl_moe_ws_h ws, const void *const *x, const int32_t *const *ids, void *stream);
xccl_status_t xccl_moe_combine(xccl_moe_ws_h ws, const int32_t *const *ids, const float *const *weights,
                               void *const *out, void *stream);
// RECV / EXPERT_OUT: [cap_rows, H] bf16; EXPERT_ROWS: [E/ranks + 1] uint32; ROW_SOURCE: [cap_rows] int32
// (source rank * T + token of each received row)
void         *xccl_moe_ws_buffer(xccl_moe_ws_h ws, int local_rank, int which);
int           xccl_moe_ws_cap_rows(xccl_moe_ws_h ws);
uint32_t      xccl_moe_ws_error(xccl_moe_ws_h ws);  // 0 = fine; synchronises

#ifdef __cplusplus
}
#endif
