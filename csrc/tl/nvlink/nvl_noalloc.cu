// See nvl_noalloc.h. The scratch that EmuWorld::create obtains with cudaMalloc is replaced by a
// file-scope device array; the kernel is the one-shot allreduce of nvl_kernels.cu, handed
// pointers into that array.
#include <atomic>
#include <cstring>

#include "../../cuda/cuda_common.h"
#include "nvl_kernels.cuh"
#include "nvl_noalloc.h"

namespace {

using namespace xccl::nvl;

constexpr size_t kSlotBytes   = (size_t)XCCL_NOALLOC_MAX_COUNT * sizeof(float);            // one rank's vector
constexpr size_t kWsBytes     = 2 * kSlotBytes * XCCL_NOALLOC_MAX_RANKS;                   // two halves of N slots
constexpr size_t kStatusBytes = 256;                                                       // 4 words per rank, padded
constexpr size_t kPadRegion   = kPadBytes * XCCL_NOALLOC_MAX_RANKS;
constexpr size_t kScratchBytes = kPadRegion + kStatusBytes + kWsBytes * XCCL_NOALLOC_MAX_RANKS;

// Layout: [pads of all ranks][status words][workspace of rank 0][workspace of rank 1]...
// In host code this name is only a handle for cudaGetSymbolAddress, never a device address.
static __device__ __align__(256) unsigned char g_noalloc_scratch[kScratchBytes];

constexpr int kMaxDevices = 64;
std::atomic<void *> g_scratch_ptr[kMaxDevices];

// Device address of the scratch on the current device; looked up once per device. Two threads that make the
// first call on one device at the same time both look it up and store the same address.
xccl_status_t scratch_for_current_device(unsigned char **out)
{
    int dev = 0;
    XCCL_CUDA_CHECK(cudaGetDevice(&dev));
    if (dev < 0 || dev >= kMaxDevices) return XCCL_ERR_INVALID_PARAM;
    void *p = g_scratch_ptr[dev].load(std::memory_order_acquire);
    if (p == nullptr) {
        cudaError_t e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
        if (e != cudaSuccess || p == nullptr) {
            xccl_error("cudaGetSymbolAddress(no-alloc scratch) failed on device %d: %s", dev, cudaGetErrorString(e));
            return xccl::cuda_status(e != cudaSuccess ? e : cudaErrorUnknown);
        }
        g_scratch_ptr[dev].store(p, std::memory_order_release);
    }
    *out = (unsigned char *)p;
    return XCCL_OK;
}

}  // namespace

extern "C" xccl_status_t xccl_emu_allreduce_f32_sum_noalloc(const float *const *srcs, float *const *dsts, int nranks,
                                                            size_t count, void *stream)
{
    if (srcs == nullptr || dsts == nullptr) return XCCL_ERR_INVALID_PARAM;
    if (nranks < 1 || nranks > XCCL_NOALLOC_MAX_RANKS || count > (size_t)XCCL_NOALLOC_MAX_COUNT) {
        xccl_error("xccl_emu_allreduce_f32_sum_noalloc: nranks=%d count=%zu exceeds the static scratch "
                   "(at most %d ranks of %d floats)",
                   nranks, count, XCCL_NOALLOC_MAX_RANKS, XCCL_NOALLOC_MAX_COUNT);
        return XCCL_ERR_BUFFER_TOO_SMALL;
    }
    if (count == 0) return XCCL_OK;
    unsigned char *base = nullptr;
    xccl_status_t  st   = scratch_for_current_device(&base);
    if (st != XCCL_OK) return st;
    cudaStream_t s = (cudaStream_t)stream;

    // pads (flags, epochs, counters) and status words must start at zero; the workspaces are
    // fully overwritten before they are read and need no clearing
    XCCL_CUDA_CHECK(cudaMemsetAsync(base, 0, kPadRegion + kStatusBytes, s));

    World w{};
    w.size           = nranks;
    w.rank_base      = 0;
    w.n_local        = nranks;
    w.mc_ws          = nullptr;
    w.ws_bytes       = kWsBytes;
    w.wait_budget_ns = 2000000000ull;
    Call c{};
    for (int r = 0; r < nranks; r++) {
        w.pad[r]    = (uint32_t *)(base + (size_t)r * kPadBytes);
        w.status[r] = (uint32_t *)(base + kPadRegion) + 4 * r;
        w.ws[r]     = (char *)(base + kPadRegion + kStatusBytes + (size_t)r * kWsBytes);
        c.src[r]    = srcs[r];
        c.dst[r]    = dsts[r];
    }
    c.count    = count;
    c.len      = count * sizeof(float);
    c.op       = XCCL_OP_SUM;
    c.scale    = 1.0f;
    c.do_scale = 0;
    c.parity   = 0;
    LaunchCfg cfg;
    cfg.cooperative = true;  // the emulated ranks wait for one another inside one launch
    st = launch_allreduce(w, c, XCCL_DT_FLOAT32, XCCL_DT_UNSUPPORTED, ALG_ONE_SHOT, cfg, s);
    if (st != XCCL_OK) return st;

    uint32_t status[4 * XCCL_NOALLOC_MAX_RANKS];
    std::memset(status, 0, sizeof(status));
    XCCL_CUDA_CHECK(cudaMemcpyAsync(status, base + kPadRegion, sizeof(uint32_t) * 4 * (size_t)nranks,
                                    cudaMemcpyDeviceToHost, s));
    XCCL_CUDA_CHECK(cudaStreamSynchronize(s));
    for (int r = 0; r < nranks; r++) {
        if (status[4 * r] == NVL_TIMEOUT) return XCCL_ERR_TIMED_OUT;
        if (status[4 * r] != NVL_OK) return XCCL_ERR_NO_MESSAGE;
    }
    return XCCL_OK;
}
