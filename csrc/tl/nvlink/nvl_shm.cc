#include "nvl_shm.h"

#include <atomic>
#include <cerrno>
#include <chrono>
#include <cstdio>
#include <cstring>
#include <sys/socket.h>
#include <sys/un.h>
#include <unistd.h>

#include "../../core/core.h"
#include "../../cuda/cuda_common.h"

namespace xccl {
namespace nvl {

namespace {

struct PeerCard {  // exchanged out of band before any descriptor moves
    char     sock[64];
    uint64_t host_hash;
    int32_t  device;
    int32_t  pid;
    int32_t  mc_capable;
    int32_t  fd_capable;
    char     bus_id[32];
};

struct FdMsg {
    int32_t src_rank;
    int32_t kind;  // 0 = memory handle, 1 = multicast handle, 2 = "no multicast object"
};

std::atomic<int> g_sock_counter{0};

int make_socket(char (&name)[64])
{
    int fd = socket(AF_UNIX, SOCK_DGRAM | SOCK_CLOEXEC | SOCK_NONBLOCK, 0);
    if (fd < 0) return -1;
    std::snprintf(name, sizeof(name), "xccl-nvl-%d-%d-%llx", (int)getpid(), g_sock_counter.fetch_add(1),
                  (unsigned long long)std::chrono::steady_clock::now().time_since_epoch().count());
    sockaddr_un addr{};
    addr.sun_family = AF_UNIX;
    size_t n        = std::strlen(name);
    std::memcpy(addr.sun_path + 1, name, n);  // abstract namespace: leading NUL, no file to clean up
    if (bind(fd, (sockaddr *)&addr, (socklen_t)(offsetof(sockaddr_un, sun_path) + 1 + n)) != 0) {
        close(fd);
        return -1;
    }
    return fd;
}

// 0 = sent, 1 = try again later, -1 = error
int send_fd(int sock, const char *dest, int fd, const FdMsg &msg)
{
    sockaddr_un addr{};
    addr.sun_family = AF_UNIX;
    size_t n        = std::strlen(dest);
    std::memcpy(addr.sun_path + 1, dest, n);
    iovec iov{(void *)&msg, sizeof(msg)};
    char  ctrl[CMSG_SPACE(sizeof(int))] = {0};
    msghdr m{};
    m.msg_name       = &addr;
    m.msg_namelen    = (socklen_t)(offsetof(sockaddr_un, sun_path) + 1 + n);
    m.msg_iov        = &iov;
    m.msg_iovlen     = 1;
    m.msg_control    = ctrl;
    m.msg_controllen = sizeof(ctrl);
    cmsghdr *c       = CMSG_FIRSTHDR(&m);
    c->cmsg_level    = SOL_SOCKET;
    c->cmsg_type     = SCM_RIGHTS;
    c->cmsg_len      = CMSG_LEN(sizeof(int));
    std::memcpy(CMSG_DATA(c), &fd, sizeof(int));
    if (sendmsg(sock, &m, MSG_DONTWAIT) >= 0) return 0;
    if (errno == EAGAIN || errno == EWOULDBLOCK || errno == ENOBUFS || errno == ECONNREFUSED || errno == ENOENT) return 1;
    return -1;
}

// 0 = received, 1 = nothing yet, -1 = error
int recv_fd(int sock, int *fd, FdMsg *msg)
{
    iovec iov{msg, sizeof(*msg)};
    char  ctrl[CMSG_SPACE(sizeof(int))] = {0};
    msghdr m{};
    m.msg_iov        = &iov;
    m.msg_iovlen     = 1;
    m.msg_control    = ctrl;
    m.msg_controllen = sizeof(ctrl);
    ssize_t r        = recvmsg(sock, &m, MSG_DONTWAIT | MSG_CMSG_CLOEXEC);
    if (r < 0) return (errno == EAGAIN || errno == EWOULDBLOCK) ? 1 : -1;
    cmsghdr *c = CMSG_FIRSTHDR(&m);
    if (r != (ssize_t)sizeof(*msg) || c == nullptr || c->cmsg_type != SCM_RIGHTS) return -1;
    std::memcpy(fd, CMSG_DATA(c), sizeof(int));
    return 0;
}

size_t round_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

}  // namespace

SymmetricRegion::~SymmetricRegion()
{
    auto cuMemUnmap_       = reinterpret_cast<decltype(&::cuMemUnmap)>(cuda_driver_fn("cuMemUnmap"));
    auto cuMemAddressFree_ = reinterpret_cast<decltype(&::cuMemAddressFree)>(cuda_driver_fn("cuMemAddressFree"));
    auto cuMemRelease_     = reinterpret_cast<decltype(&::cuMemRelease)>(cuda_driver_fn("cuMemRelease"));
    auto cuMulticastUnbind_ = reinterpret_cast<decltype(&::cuMulticastUnbind)>(cuda_driver_fn("cuMulticastUnbind"));
    if (cuMemUnmap_ == nullptr || cuMemAddressFree_ == nullptr || cuMemRelease_ == nullptr) return;
    cudaDeviceSynchronize();
    if (mc_mapped_) {
        cuMemUnmap_((CUdeviceptr)mc_va_, mc_bytes_);
        cuMemAddressFree_((CUdeviceptr)mc_va_, mc_bytes_);
    }
    if (mc_bound_ && cuMulticastUnbind_ != nullptr) cuMulticastUnbind_(mc_handle_, (CUdevice)device, 0, mc_bytes_);
    if (mc_have_) cuMemRelease_(mc_handle_);
    for (int r = 0; r < size; r++) {
        if ((size_t)r < mapped_.size() && mapped_[(size_t)r]) {
            cuMemUnmap_((CUdeviceptr)base[(size_t)r], bytes);
            cuMemAddressFree_((CUdeviceptr)base[(size_t)r], bytes);
            cuMemRelease_(handles_[(size_t)r]);
        }
    }
}

xccl_status_t SymmetricRegion::create(const OobGroup &g, size_t bytes, bool want_multicast, SymmetricRegion **out)
{
    auto         *r  = new SymmetricRegion;
    xccl_status_t st = r->setup(g, bytes, want_multicast);
    if (st != XCCL_OK) {
        delete r;
        return st;
    }
    *out = r;
    return XCCL_OK;
}

xccl_status_t SymmetricRegion::setup(const OobGroup &g, size_t want_bytes, bool want_multicast)
{
    if (!cuda_available()) return XCCL_ERR_NO_RESOURCE;
    XCCL_DRIVER_FN(cuMemCreate);
    XCCL_DRIVER_FN(cuMemGetAllocationGranularity);
    XCCL_DRIVER_FN(cuMemAddressReserve);
    XCCL_DRIVER_FN(cuMemMap);
    XCCL_DRIVER_FN(cuMemSetAccess);
    XCCL_DRIVER_FN(cuMemExportToShareableHandle);
    XCCL_DRIVER_FN(cuMemImportFromShareableHandle);
    XCCL_DRIVER_FN(cuDeviceGetAttribute);
    auto cuMulticastCreate_ = reinterpret_cast<decltype(&::cuMulticastCreate)>(cuda_driver_fn("cuMulticastCreate"));
    auto cuMulticastAddDevice_ = reinterpret_cast<decltype(&::cuMulticastAddDevice)>(cuda_driver_fn("cuMulticastAddDevice"));
    auto cuMulticastBindMem_ = reinterpret_cast<decltype(&::cuMulticastBindMem)>(cuda_driver_fn("cuMulticastBindMem"));
    auto cuMulticastGetGranularity_ =
        reinterpret_cast<decltype(&::cuMulticastGetGranularity)>(cuda_driver_fn("cuMulticastGetGranularity"));

    rank = g.rank;
    size = g.size;
    XCCL_CUDA_CHECK(cudaFree(nullptr));  // makes the primary context current
    XCCL_CUDA_CHECK(cudaGetDevice(&device));
    base.assign((size_t)size, nullptr);
    handles_.assign((size_t)size, 0);
    mapped_.assign((size_t)size, false);

    // ---- 1. who is where
    PeerCard mine{};
    int      sock = make_socket(mine.sock);
    if (sock < 0) return XCCL_ERR_NO_RESOURCE;
    struct SockGuard {
        int fd;
        ~SockGuard() { close(fd); }
    } sock_guard{sock};
    int fd_ok = 0, mc_ok = 0;
    cuDeviceGetAttribute(&fd_ok, CU_DEVICE_ATTRIBUTE_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR_SUPPORTED, (CUdevice)device);
    cuDeviceGetAttribute(&mc_ok, CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED, (CUdevice)device);
    bool have_mc_api = cuMulticastCreate_ != nullptr && cuMulticastAddDevice_ != nullptr &&
                       cuMulticastBindMem_ != nullptr && cuMulticastGetGranularity_ != nullptr;
    mine.host_hash  = global_state().host_hash;
    mine.device     = device;
    mine.pid        = (int32_t)getpid();
    mine.fd_capable = fd_ok;
    mine.mc_capable = (want_multicast && mc_ok && have_mc_api && size > 1) ? 1 : 0;
    cudaDeviceGetPCIBusId(mine.bus_id, (int)sizeof(mine.bus_id), device);
    std::vector<PeerCard> cards((size_t)size);
    xccl_status_t         st = g.allgather_blocking(&mine, cards.data(), sizeof(PeerCard));
    if (st != XCCL_OK) return st;
    bool use_mc = true;
    for (int p = 0; p < size; p++) {
        const PeerCard &c = cards[(size_t)p];
        if (c.host_hash != mine.host_hash || !c.fd_capable) return XCCL_ERR_UNREACHABLE;
        use_mc = use_mc && c.mc_capable;
        for (int q = 0; q < p; q++) {
            if (std::strncmp(cards[(size_t)q].bus_id, c.bus_id, sizeof(c.bus_id)) == 0) {
                xccl_debug("nvlink: ranks %d and %d share GPU %s; one process per GPU is required", q, p, c.bus_id);
                return XCCL_ERR_UNSUPPORTED;
            }
        }
    }

    // ---- 2. my allocation
    CUmemAllocationProp prop{};
    prop.type                 = CU_MEM_ALLOCATION_TYPE_PINNED;
    prop.location.type        = CU_MEM_LOCATION_TYPE_DEVICE;
    prop.location.id          = device;
    prop.requestedHandleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
    size_t gran = 0;
    XCCL_CU_CHECK(cuMemGetAllocationGranularity(&gran, &prop, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED));
    CUmulticastObjectProp mcp{};
    if (use_mc) {
        mcp.numDevices  = (unsigned)size;
        mcp.size        = round_up(want_bytes, gran);
        mcp.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
        size_t mgran    = 0;
        if (cuMulticastGetGranularity_(&mgran, &mcp, CU_MULTICAST_GRANULARITY_RECOMMENDED) == CUDA_SUCCESS && mgran > 0) {
            gran = std::max(gran, mgran);
        } else {
            use_mc = false;  // same answer on every rank: same devices, same size
        }
    }
    bytes     = round_up(want_bytes, gran);
    mcp.size  = bytes;
    mc_bytes_ = bytes;
    CUmemAccessDesc acc_desc{};
    acc_desc.location = prop.location;
    acc_desc.flags    = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
    XCCL_CU_CHECK(cuMemCreate(&handles_[(size_t)rank], bytes, &prop, 0));
    CUdeviceptr va = 0;
    XCCL_CU_CHECK(cuMemAddressReserve(&va, bytes, gran, 0, 0));
    XCCL_CU_CHECK(cuMemMap(va, bytes, 0, handles_[(size_t)rank], 0));
    XCCL_CU_CHECK(cuMemSetAccess(va, bytes, &acc_desc, 1));
    base[(size_t)rank]    = (char *)va;
    mapped_[(size_t)rank] = true;
    XCCL_CUDA_CHECK(cudaMemset((void *)va, 0, bytes));
    XCCL_CUDA_CHECK(cudaDeviceSynchronize());
    int my_fd = -1;
    XCCL_CU_CHECK(cuMemExportToShareableHandle(&my_fd, handles_[(size_t)rank], CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0));

    // ---- 3. rank 0 creates the multicast object
    int mc_fd = -1, mc_kind = 2;
    if (use_mc && rank == 0) {
        if (cuMulticastCreate_(&mc_handle_, &mcp) == CUDA_SUCCESS) {
            mc_have_ = true;
            if (cuMemExportToShareableHandle(&mc_fd, mc_handle_, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0) == CUDA_SUCCESS) {
                mc_kind = 1;
            }
        }
        if (mc_kind != 1) xccl_info("nvlink: multicast object could not be created; NVLS disabled");
    }

    // ---- 4. descriptors travel over the unix sockets
    struct Out {
        int   dest, fd;
        FdMsg msg;
    };
    std::vector<Out> outbox;
    for (int p = 0; p < size; p++) {
        if (p == rank) continue;
        outbox.push_back(Out{p, my_fd, FdMsg{rank, 0}});
        if (use_mc && rank == 0) outbox.push_back(Out{p, mc_kind == 1 ? mc_fd : my_fd, FdMsg{rank, mc_kind}});
    }
    std::vector<int> peer_fd((size_t)size, -1);
    int              got_mc_fd = -1, got_mc_kind = (use_mc && rank != 0) ? -1 : mc_kind;
    int              expect = (size - 1) + ((use_mc && rank != 0) ? 1 : 0), received = 0;
    size_t           sent  = 0;
    double           limit = global_state().opts.real("OOB_TIMEOUT");
    auto             t0    = std::chrono::steady_clock::now();
    bool             io_error = false;
    while ((sent < outbox.size() || received < expect) && !io_error) {
        if (sent < outbox.size()) {
            int rc = send_fd(sock, cards[(size_t)outbox[sent].dest].sock, outbox[sent].fd, outbox[sent].msg);
            if (rc == 0) sent++;
            if (rc < 0) io_error = true;
        }
        int   fd = -1;
        FdMsg msg{};
        int   rc = recv_fd(sock, &fd, &msg);
        if (rc == 0) {
            received++;
            if (msg.kind == 0 && msg.src_rank >= 0 && msg.src_rank < size) {
                peer_fd[(size_t)msg.src_rank] = fd;
            } else {
                got_mc_kind = msg.kind;
                if (msg.kind == 1) {
                    got_mc_fd = fd;
                } else {
                    close(fd);
                }
            }
        } else if (rc < 0) {
            io_error = true;
        }
        double dt = std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
        if (limit > 0 && dt > limit) io_error = true;
    }
    close(my_fd);
    if (mc_fd >= 0) close(mc_fd);

    // ---- 5. map the peers
    int ok = io_error ? 0 : 1;
    for (int p = 0; p < size && ok; p++) {
        if (p == rank) continue;
        if (peer_fd[(size_t)p] < 0) {
            ok = 0;
            break;
        }
        CUmemGenericAllocationHandle h = 0;
        if (cuMemImportFromShareableHandle(&h, (void *)(uintptr_t)peer_fd[(size_t)p],
                                           CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR) != CUDA_SUCCESS) {
            ok = 0;
            break;
        }
        CUdeviceptr pva = 0;
        if (cuMemAddressReserve(&pva, bytes, gran, 0, 0) != CUDA_SUCCESS || cuMemMap(pva, bytes, 0, h, 0) != CUDA_SUCCESS ||
            cuMemSetAccess(pva, bytes, &acc_desc, 1) != CUDA_SUCCESS) {
            xccl_debug("nvlink: cannot map the memory of rank %d (no peer access?)", p);
            ok = 0;
            break;
        }
        handles_[(size_t)p] = h;
        base[(size_t)p]     = (char *)pva;
        mapped_[(size_t)p]  = true;
    }
    for (int p = 0; p < size; p++) {
        if (peer_fd[(size_t)p] >= 0) close(peer_fd[(size_t)p]);
    }
    int mc_stage = 0;
    if (ok && use_mc && got_mc_kind == 1) {
        if (rank != 0) {
            if (cuMemImportFromShareableHandle(&mc_handle_, (void *)(uintptr_t)got_mc_fd,
                                               CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR) == CUDA_SUCCESS) {
                mc_have_ = true;
            }
        }
        if (mc_have_ && cuMulticastAddDevice_(mc_handle_, (CUdevice)device) == CUDA_SUCCESS) mc_stage = 1;
    }
    if (got_mc_fd >= 0) close(got_mc_fd);

    // ---- 6. agree on the outcome; every device must be added before anyone binds memory
    int              flags[2] = {ok, mc_stage};
    std::vector<int> all((size_t)size * 2);
    st = g.allgather_blocking(flags, all.data(), sizeof(flags));
    if (st != XCCL_OK) return st;
    bool all_ok = true, all_mc = true;
    for (int p = 0; p < size; p++) {
        all_ok = all_ok && all[(size_t)p * 2] != 0;
        all_mc = all_mc && all[(size_t)p * 2 + 1] != 0;
    }
    if (!all_ok) return XCCL_ERR_UNREACHABLE;
    int bound = 0;
    if (all_mc) {
        if (cuMulticastBindMem_(mc_handle_, 0, handles_[(size_t)rank], 0, bytes, 0) == CUDA_SUCCESS) {
            mc_bound_        = true;
            CUdeviceptr mcva = 0;
            if (cuMemAddressReserve(&mcva, bytes, gran, 0, 0) == CUDA_SUCCESS) {
                if (cuMemMap(mcva, bytes, 0, mc_handle_, 0) == CUDA_SUCCESS &&
                    cuMemSetAccess(mcva, bytes, &acc_desc, 1) == CUDA_SUCCESS) {
                    mc_base    = (char *)mcva;
                    mc_va_     = (char *)mcva;
                    mc_mapped_ = true;
                    bound      = 1;
                }
            }
        }
    }
    std::vector<int> all_bound((size_t)size);
    st = g.allgather_blocking(&bound, all_bound.data(), sizeof(int));
    if (st != XCCL_OK) return st;
    for (int p = 0; p < size; p++) {
        if (!all_bound[(size_t)p]) {
            mc_base = nullptr;  // the mapping (if any) is released by the destructor
        }
    }
    xccl_debug("nvlink: symmetric region of %zu bytes on %d ranks, multicast %s", bytes, size,
               mc_base != nullptr ? "on" : "off");
    return XCCL_OK;
}

}  // namespace nvl
}  // namespace xccl
