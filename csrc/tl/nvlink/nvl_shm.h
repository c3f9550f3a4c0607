// Symmetric device memory shared between the processes of one node.
//
// A SymmetricRegion is one CUDA VMM allocation per rank, exported as a POSIX file descriptor,
// passed to every peer over a unix datagram socket (SCM_RIGHTS), imported and mapped there.
// After creation base[r] is rank r's region as mapped in this process (base[rank] is my own).
// When every device supports multicast, the regions are also bound to one NVSwitch multicast
// object and mc_base is its mapping: multimem instructions on mc_base + off act on offset `off`
// of every rank's region at once.
//
// Creation is collective over an OobGroup and uses blocking out-of-band exchanges with the
// XCCL_OOB_TIMEOUT deadline. Peers must be distinct GPUs of one host with peer access.
#pragma once
#include <cuda.h>

#include <string>
#include <vector>

#include "../../core/tl.h"

namespace xccl {
namespace nvl {

class SymmetricRegion {
public:
    ~SymmetricRegion();
    // bytes is rounded up to the allocation (and multicast) granularity
    static xccl_status_t create(const OobGroup &g, size_t bytes, bool want_multicast, SymmetricRegion **out);

    int                 rank = 0, size = 1, device = 0;
    size_t              bytes = 0;
    std::vector<char *> base;        // [size]
    char               *mc_base = nullptr;

private:
    xccl_status_t                             setup(const OobGroup &g, size_t bytes, bool want_multicast);
    std::vector<CUmemGenericAllocationHandle> handles_;  // [size], mine at [rank]
    std::vector<bool>                         mapped_;
    CUmemGenericAllocationHandle              mc_handle_ = 0;
    bool                                      mc_bound_ = false, mc_mapped_ = false, mc_have_ = false;
    size_t                                    mc_bytes_ = 0;
    char                                     *mc_va_    = nullptr;
};

}  // namespace nvl
}  // namespace xccl
