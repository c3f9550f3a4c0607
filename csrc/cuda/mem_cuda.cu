#include "mem_cuda.h"

#include <cstdlib>
#include <mutex>

#include "cuda_common.h"

namespace xccl {

bool cuda_available()
{
    static int state = [] {
        int         n = 0;
        cudaError_t e = cudaGetDeviceCount(&n);
        if (e != cudaSuccess) {
            (void)cudaGetLastError();
            return 0;
        }
        return n > 0 ? 1 : 0;
    }();
    return state == 1;
}

void *cuda_driver_fn(const char *name)
{
    if (!cuda_available()) return nullptr;
    void                            *fn = nullptr;
    cudaDriverEntryPointQueryResult  qres;
    if (cudaGetDriverEntryPoint(name, &fn, cudaEnableDefault, &qres) != cudaSuccess || qres != cudaDriverEntryPointSuccess) {
        (void)cudaGetLastError();
        return nullptr;
    }
    return fn;
}

xccl_memory_type_t cuda_pointer_type(const void *ptr)
{
    if (ptr == nullptr || !cuda_available()) return XCCL_MEMORY_TYPE_HOST;
    cudaPointerAttributes attr;
    if (cudaPointerGetAttributes(&attr, ptr) != cudaSuccess) {
        (void)cudaGetLastError();
        return XCCL_MEMORY_TYPE_HOST;
    }
    return (attr.type == cudaMemoryTypeDevice || attr.type == cudaMemoryTypeManaged) ? XCCL_MEMORY_TYPE_CUDA
                                                                                      : XCCL_MEMORY_TYPE_HOST;
}

xccl_status_t cuda_alloc(void **ptr, size_t bytes)
{
    XCCL_CUDA_CHECK(cudaMalloc(ptr, bytes));
    return XCCL_OK;
}

xccl_status_t cuda_free(void *ptr)
{
    XCCL_CUDA_CHECK(cudaFree(ptr));
    return XCCL_OK;
}

void *cuda_internal_stream()
{
    // one non-blocking stream per process and device-in-use at first call
    static cudaStream_t s = [] {
        cudaStream_t st = nullptr;
        if (cudaStreamCreateWithFlags(&st, cudaStreamNonBlocking) != cudaSuccess) {
            (void)cudaGetLastError();
            st = nullptr;
        }
        return st;
    }();
    return (void *)s;
}

xccl_status_t cuda_reduce_multi_sync(const void *a, const void *vecs, void *dst, size_t n_vectors, size_t count,
                                     size_t stride_bytes, xccl_dt_t dt, xccl_op_t op)
{
    cudaStream_t  s  = (cudaStream_t)cuda_internal_stream();
    xccl_status_t st = cuda_reduce_multi(a, vecs, dst, n_vectors, count, stride_bytes, dt, op, 1.0f,
                                         XCCL_DT_UNSUPPORTED, s);
    if (st != XCCL_OK) return st;
    XCCL_CUDA_CHECK(cudaStreamSynchronize(s));
    return XCCL_OK;
}

xccl_status_t cuda_copy(void *dst, const void *src, size_t bytes, void *stream)
{
    if (stream != nullptr) {
        XCCL_CUDA_CHECK(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDefault, (cudaStream_t)stream));
    } else {
        XCCL_CUDA_CHECK(cudaMemcpy(dst, src, bytes, cudaMemcpyDefault));
    }
    return XCCL_OK;
}

xccl_status_t cuda_stream_sync(void *stream)
{
    XCCL_CUDA_CHECK(cudaStreamSynchronize((cudaStream_t)stream));
    return XCCL_OK;
}

xccl_status_t cuda_event_record(void *stream, void **event)
{
    cudaEvent_t ev;
    XCCL_CUDA_CHECK(cudaEventCreateWithFlags(&ev, cudaEventDisableTiming));
    cudaError_t e = cudaEventRecord(ev, (cudaStream_t)stream);
    if (e != cudaSuccess) {
        cudaEventDestroy(ev);
        return cuda_status(e);
    }
    *event = (void *)ev;
    return XCCL_OK;
}

xccl_status_t cuda_event_query(void *event)
{
    cudaError_t e = cudaEventQuery((cudaEvent_t)event);
    if (e == cudaErrorNotReady) return XCCL_INPROGRESS;
    return cuda_status(e);
}

xccl_status_t cuda_event_release(void *event)
{
    XCCL_CUDA_CHECK(cudaEventDestroy((cudaEvent_t)event));
    return XCCL_OK;
}

// ------------------------------------------------------------------ stream hold

struct HoldSlot {
    volatile int release;  // host writes 1
    volatile int status;   // device writes: 1 = released normally, 2 = budget expired
};

struct StreamHold {
    HoldSlot *host = nullptr;
    HoldSlot *dev  = nullptr;
    bool      used = false;
};

namespace {

__global__ void stream_hold_kernel(HoldSlot *slot, unsigned long long budget_ns)
{
    unsigned long long t0, now;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
    int released = 0;
    for (;;) {
        if (slot->release != 0) {
            released = 1;
            break;
        }
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
        if (now - t0 > budget_ns) break;
        __nanosleep(200);
    }
    slot->status = released ? 1 : 2;
    __threadfence_system();
}

constexpr int     kHoldSlots = 4;
std::mutex        g_hold_mu;
StreamHold        g_holds[kHoldSlots];

unsigned long long hold_budget_ns()
{
    const char *e  = std::getenv("XCCL_STREAM_HOLD_TIMEOUT_MS");
    long        ms = (e != nullptr) ? std::atol(e) : 10000;
    if (ms <= 0) ms = 10000;
    return (unsigned long long)ms * 1000000ull;
}

xccl_status_t acquire_slot(StreamHold **out)
{
    std::lock_guard<std::mutex> lock(g_hold_mu);
    for (auto &h : g_holds) {
        if (h.used) continue;
        if (h.host == nullptr) {
            XCCL_CUDA_CHECK(cudaHostAlloc((void **)&h.host, sizeof(HoldSlot), cudaHostAllocMapped));
            XCCL_CUDA_CHECK(cudaHostGetDevicePointer((void **)&h.dev, (void *)h.host, 0));
        }
        h.host->release = 0;
        h.host->status  = 0;
        h.used          = true;
        *out            = &h;
        return XCCL_OK;
    }
    return XCCL_ERR_NO_RESOURCE;
}

}  // namespace

xccl_status_t hold_start(void *stream, StreamHold **hold)
{
    xccl_status_t st = acquire_slot(hold);
    if (st != XCCL_OK) return st;
    stream_hold_kernel<<<1, 1, 0, (cudaStream_t)stream>>>((*hold)->dev, hold_budget_ns());
    XCCL_CUDA_CHECK(cudaGetLastError());
    return XCCL_OK;
}

xccl_status_t hold_release(StreamHold *hold)
{
    hold->host->release = 1;
    return XCCL_OK;
}

xccl_status_t hold_finish(StreamHold *hold)
{
    int                         status = hold->host->status;
    std::lock_guard<std::mutex> lock(g_hold_mu);
    hold->used = false;
    return status == 2 ? XCCL_ERR_TIMED_OUT : XCCL_OK;
}

}  // namespace xccl

using namespace xccl;

extern "C" {

xccl_status_t xccl_cuda_reduce_multi(const void *a, const void *vecs, void *dst, size_t n_vectors, size_t count,
                                     size_t stride_bytes, int dt, int op, float scale, int out_dt, void *stream)
{
    return cuda_reduce_multi(a, vecs, dst, n_vectors, count, stride_bytes, (xccl_dt_t)dt, (xccl_op_t)op, scale,
                             (xccl_dt_t)out_dt, stream);
}

xccl_status_t xccl_cuda_hold_timeout_probe(int budget_ms, float *elapsed_ms)
{
    StreamHold   *h  = nullptr;
    xccl_status_t st = acquire_slot(&h);
    if (st != XCCL_OK) return st;
    cudaEvent_t e0, e1;
    XCCL_CUDA_CHECK(cudaEventCreate(&e0));
    XCCL_CUDA_CHECK(cudaEventCreate(&e1));
    XCCL_CUDA_CHECK(cudaEventRecord(e0, nullptr));
    stream_hold_kernel<<<1, 1>>>(h->dev, (unsigned long long)budget_ms * 1000000ull);
    XCCL_CUDA_CHECK(cudaEventRecord(e1, nullptr));
    XCCL_CUDA_CHECK(cudaEventSynchronize(e1));
    if (elapsed_ms != nullptr) cudaEventElapsedTime(elapsed_ms, e0, e1);
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    return hold_finish(h);
}

}  // extern "C"
