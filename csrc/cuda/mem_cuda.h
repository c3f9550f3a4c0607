// CUDA side of the memory component.
// Reference: src/utils/cuda/cuda_mem_component.c:28-281 and the three kernels under
// src/utils/cuda/kernels/.
#pragma once
#include <cstddef>

#include "xccl/xccl.h"

namespace xccl {

bool               cuda_available();
xccl_memory_type_t cuda_pointer_type(const void *ptr);  // HOST when the runtime does not know the pointer
xccl_status_t      cuda_alloc(void **ptr, size_t bytes);
xccl_status_t      cuda_free(void *ptr);

// dst = out_cast(scale * (a op v_0 ... op v_{n-1})) on `stream` (a cudaStream_t, may be null = the
// component's own non-blocking stream, in which case the call returns after the kernel finished).
xccl_status_t cuda_reduce_multi(const void *a, const void *vecs, void *dst, size_t n_vectors, size_t count,
                                size_t stride_bytes, xccl_dt_t dt, xccl_op_t op, float scale, xccl_dt_t out_dt,
                                void *stream);
xccl_status_t cuda_reduce_multi_sync(const void *a, const void *vecs, void *dst, size_t n_vectors, size_t count,
                                     size_t stride_bytes, xccl_dt_t dt, xccl_op_t op);

xccl_status_t cuda_copy(void *dst, const void *src, size_t bytes, void *stream_or_null);
// dst block (j, i) = src block (i, j) for rows x cols blocks of block_bytes (out of place)
xccl_status_t cuda_block_transpose(void *dst, const void *src, int rows, int cols, size_t block_bytes, void *stream);
xccl_status_t cuda_stream_sync(void *stream);

// Events: a collective that the host progresses starts only after work already queued on the
// caller's stream has finished.
xccl_status_t cuda_event_record(void *stream, void **event);
xccl_status_t cuda_event_query(void *event);  // XCCL_OK, XCCL_INPROGRESS or an error
xccl_status_t cuda_event_release(void *event);

// Stream hold: makes `stream` wait until hold_release() is called by the host, so that work
// queued after a host-progressed collective runs after it. The holding kernel polls a mapped
// host flag with a budget (XCCL_STREAM_HOLD_TIMEOUT_MS, default 10000): when the budget runs
// out it records a timeout in the slot and returns, it never spins for ever.
struct StreamHold;
xccl_status_t hold_start(void *stream, StreamHold **hold);
xccl_status_t hold_release(StreamHold *hold);       // lets the stream continue
xccl_status_t hold_finish(StreamHold *hold);        // XCCL_OK or XCCL_ERR_TIMED_OUT; frees the slot
void         *cuda_internal_stream();

}  // namespace xccl

extern "C" {
// Test hooks with C linkage (used from Python through ctypes).
xccl_status_t xccl_cuda_reduce_multi(const void *a, const void *vecs, void *dst, size_t n_vectors, size_t count,
                                     size_t stride_bytes, int dt, int op, float scale, int out_dt, void *stream);
// Runs the holding kernel with nobody releasing it and a budget of `budget_ms`; returns the
// status the host reads afterwards (XCCL_ERR_TIMED_OUT expected) and the elapsed milliseconds.
xccl_status_t xccl_cuda_hold_timeout_probe(int budget_ms, float *elapsed_ms);
}
