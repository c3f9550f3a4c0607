// Memory component: what the algorithms need from "the place a buffer lives".
// Host buffers are served here; CUDA buffers are forwarded to csrc/cuda/mem_cuda.cu.
// Reference: src/utils/mem_component.h:28-95, src/utils/mem_component.c:11-257.
#pragma once
#include <cstddef>

#include "xccl/xccl.h"

namespace xccl {

// HOST unless the CUDA runtime says the pointer is device (or managed) memory.
xccl_memory_type_t mem_type_of(const void *ptr);

// Scratch allocation. One buffer of XCCL_MEM_COMPONENT_CACHE_SIZE bytes is kept per memory type
// and handed out when it is free and large enough, so small collectives never allocate.
xccl_status_t mem_alloc(void **ptr, size_t bytes, xccl_memory_type_t mem);
xccl_status_t mem_free(void *ptr, xccl_memory_type_t mem);
void          mem_cache_release();  // drops the cached buffers (library cleanup)

// dst[i] = a[i] op b[i], i < count
xccl_status_t mem_reduce(const void *a, const void *b, void *dst, size_t count, xccl_dt_t dt, xccl_op_t op,
                         xccl_memory_type_t mem);

// dst[i] = a[i] op v_0[i] op v_1[i] ... op v_{n-1}[i], where v_k = (char*)vecs + k * stride_bytes
xccl_status_t mem_reduce_multi(const void *a, const void *vecs, void *dst, size_t n_vectors, size_t count,
                               size_t stride_bytes, xccl_dt_t dt, xccl_op_t op, xccl_memory_type_t mem);

// Host implementations (also the CPU oracle of the GPU kernels).
xccl_status_t host_reduce(const void *a, const void *b, void *dst, size_t count, xccl_dt_t dt, xccl_op_t op);
xccl_status_t host_reduce_multi(const void *a, const void *vecs, void *dst, size_t n_vectors, size_t count,
                                size_t stride_bytes, xccl_dt_t dt, xccl_op_t op);
bool          host_reduce_supported(xccl_dt_t dt, xccl_op_t op);
// dst[i] = out_cast(scale * src[i]); out_dt == XCCL_DT_UNSUPPORTED keeps dt. Same pairs as the GPU epilogue.
xccl_status_t host_scale_cast(const void *src, xccl_dt_t dt, void *dst, xccl_dt_t out_dt, size_t count, float scale);

// Copies between any two memory types. With a stream the device side is asynchronous on it.
xccl_status_t mem_copy(void *dst, const void *src, size_t bytes, xccl_memory_type_t dst_mem, xccl_memory_type_t src_mem,
                       void *cuda_stream_or_null);

}  // namespace xccl

extern "C" {
// C-callable forms used by tests and bindings.
xccl_status_t xccl_mem_reduce(const void *a, const void *b, void *dst, size_t count, xccl_dt_t dt, xccl_op_t op);
xccl_status_t xccl_mem_reduce_multi(const void *a, const void *vecs, void *dst, size_t n_vectors, size_t count,
                                    size_t stride_bytes, xccl_dt_t dt, xccl_op_t op);
int           xccl_mem_type(const void *ptr);
}
