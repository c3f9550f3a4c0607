#include "mem.h"

#include <cstdlib>
#include <cstring>
#include <mutex>

#include "../core/core.h"
#include "../cuda/mem_cuda.h"

namespace xccl {

xccl_memory_type_t mem_type_of(const void *ptr) { return cuda_pointer_type(ptr); }

namespace {
struct Cache {
    void  *ptr   = nullptr;
    size_t bytes = 0;
    bool   busy  = false;
};
std::mutex g_mu;
Cache      g_cache[XCCL_MEMORY_TYPE_LAST];

xccl_status_t raw_alloc(void **p, size_t bytes, xccl_memory_type_t mem)
{
    if (mem == XCCL_MEMORY_TYPE_CUDA) return cuda_alloc(p, bytes);
    *p = std::malloc(bytes);
    return *p != nullptr ? XCCL_OK : XCCL_ERR_NO_MEMORY;
}

void raw_free(void *p, xccl_memory_type_t mem)
{
    if (mem == XCCL_MEMORY_TYPE_CUDA) {
        cuda_free(p);
    } else {
        std::free(p);
    }
}
}  // namespace

xccl_status_t mem_alloc(void **ptr, size_t bytes, xccl_memory_type_t mem)
{
    size_t cache_bytes = (size_t)global_state().opts.num("MEM_COMPONENT_CACHE_SIZE");
    if (bytes == 0) bytes = 1;
    if (bytes <= cache_bytes) {
        std::lock_guard<std::mutex> lock(g_mu);
        Cache                      &c = g_cache[mem];
        if (!c.busy) {
            if (c.ptr == nullptr) {
                xccl_status_t st = raw_alloc(&c.ptr, cache_bytes, mem);
                if (st != XCCL_OK) return st;
                c.bytes = cache_bytes;
            }
            c.busy = true;
            *ptr   = c.ptr;
            return XCCL_OK;
        }
    }
    return raw_alloc(ptr, bytes, mem);
}

xccl_status_t mem_free(void *ptr, xccl_memory_type_t mem)
{
    if (ptr == nullptr) return XCCL_OK;
    {
        std::lock_guard<std::mutex> lock(g_mu);
        Cache                      &c = g_cache[mem];
        if (ptr == c.ptr) {
            c.busy = false;
            return XCCL_OK;
        }
    }
    raw_free(ptr, mem);
    return XCCL_OK;
}

void mem_cache_release()
{
    std::lock_guard<std::mutex> lock(g_mu);
    for (int m = 0; m < XCCL_MEMORY_TYPE_LAST; m++) {
        Cache &c = g_cache[m];
        if (c.ptr != nullptr && !c.busy) {
            raw_free(c.ptr, (xccl_memory_type_t)m);
            c = Cache{};
        }
    }
}

xccl_status_t mem_reduce(const void *a, const void *b, void *dst, size_t count, xccl_dt_t dt, xccl_op_t op,
                         xccl_memory_type_t mem)
{
    return mem_reduce_multi(a, b, dst, 1, count, 0, dt, op, mem);
}

xccl_status_t mem_reduce_multi(const void *a, const void *vecs, void *dst, size_t n_vectors, size_t count,
                               size_t stride_bytes, xccl_dt_t dt, xccl_op_t op, xccl_memory_type_t mem)
{
    if (mem == XCCL_MEMORY_TYPE_CUDA) {
        return cuda_reduce_multi_sync(a, vecs, dst, n_vectors, count, stride_bytes, dt, op);
    }
    return host_reduce_multi(a, vecs, dst, n_vectors, count, stride_bytes, dt, op);
}

xccl_status_t mem_copy(void *dst, const void *src, size_t bytes, xccl_memory_type_t dst_mem, xccl_memory_type_t src_mem,
                       void *stream)
{
    if (bytes == 0 || dst == src) return XCCL_OK;
    if (dst_mem == XCCL_MEMORY_TYPE_HOST && src_mem == XCCL_MEMORY_TYPE_HOST) {
        std::memmove(dst, src, bytes);
        return XCCL_OK;
    }
    return cuda_copy(dst, src, bytes, stream);
}

}  // namespace xccl

extern "C" {

xccl_status_t xccl_mem_reduce(const void *a, const void *b, void *dst, size_t count, xccl_dt_t dt, xccl_op_t op)
{
    return xccl::mem_reduce(a, b, dst, count, dt, op, xccl::mem_type_of(dst));
}

xccl_status_t xccl_mem_reduce_multi(const void *a, const void *vecs, void *dst, size_t n_vectors, size_t count,
                                    size_t stride_bytes, xccl_dt_t dt, xccl_op_t op)
{
    return xccl::mem_reduce_multi(a, vecs, dst, n_vectors, count, stride_bytes, dt, op, xccl::mem_type_of(dst));
}

int xccl_mem_type(const void *ptr) { return (int)xccl::mem_type_of(ptr); }

}  // extern "C"
