// Allocation-free entry point of the emulated one-shot allreduce.
//
// This function has no counterpart in the reference (openucx/xccl): it exists for callers that
// are not allowed to allocate device memory when they need a collective - code running inside a
// memory-pool callback, a plugin loaded into a process whose allocator is owned by somebody else,
// or a latency-critical path that must not touch the driver's allocator because cudaMalloc can
// synchronise the whole device. Everything the kernel needs beyond the caller's inputs and
// outputs (the per-rank workspaces and signal pads that xccl_nvlink_emu_create would allocate)
// lives in one static device array that is part of the library image.
#pragma once
#include <stddef.h>

#include "xccl/xccl.h"

#ifdef __cplusplus
extern "C" {
#endif

// Largest problem the static scratch is sized for.
#define XCCL_NOALLOC_MAX_RANKS 8
#define XCCL_NOALLOC_MAX_COUNT 16384   /* fp32 elements per rank (64 KiB) */

// dsts[r][i] = sum over q of srcs[q][i] for the `nranks` emulated ranks, all on the current device.
//
//  - srcs / dsts: host arrays of `nranks` device pointers to `count` floats each. The caller owns
//    them; nothing else is passed in or allocated.
//  - Limits: 1 <= nranks <= XCCL_NOALLOC_MAX_RANKS and count <= XCCL_NOALLOC_MAX_COUNT; anything
//    larger is refused with XCCL_ERR_BUFFER_TOO_SMALL and a message in the log.
//  - The call enqueues a clear of the signal pads, the kernel and a read-back of the kernel's
//    status on `stream`, then waits for the stream: when it returns XCCL_OK the outputs are
//    complete. XCCL_ERR_TIMED_OUT means a bounded device-side wait expired.
//  - No cudaMalloc, cudaFree or other allocating routine is called, here or in what it calls.
//  - The scratch (about 8.2 MiB) is held by every GPU that loads the library until the process
//    exits. It is shared by all calls and keeps the previous call's contents; the parts that
//    must start at zero are cleared by every call. Two calls that overlap on the GPU (different
//    streams or threads) race on it: issue them one at a time.
//  - The first call on each device looks up the device address of the scratch
//    (cudaGetSymbolAddress) with that device current. Make that first call before starting any
//    stream capture.
xccl_status_t xccl_emu_allreduce_f32_sum_noalloc(const float *const *srcs, float *const *dsts, int nranks, size_t count,
                                                 void *stream);

#ifdef __cplusplus
}
#endif
