// NCCL team library: public bits. The p2p functions are an extension of the API: the Teams API
// of the reference has no user-visible send/recv (its README lists it as a goal only); pipeline
// parallel stages use these, carried by NCCL's own p2p.
#pragma once
#include "xccl/xccl.h"

namespace xccl {
namespace nccltl {
bool nccl_available();
}
}  // namespace xccl

extern "C" {
int           xccl_nccl_version(void);  // NCCL_VERSION_CODE of the library found at run time, 0 if none
// A point-to-point communicator over the ranks of `oob` (collective call).
xccl_status_t xccl_p2p_comm_create(const xccl_oob_collectives_t *oob, void **comm);
void          xccl_p2p_comm_destroy(void *comm);
// Stream-ordered send / receive of raw bytes; pair them inside group_start / group_end when one
// rank both sends and receives, as with any NCCL p2p.
xccl_status_t xccl_p2p_send(void *comm, const void *buf, size_t bytes, int peer, void *stream);
xccl_status_t xccl_p2p_recv(void *comm, void *buf, size_t bytes, int peer, void *stream);
xccl_status_t xccl_p2p_group_start(void);
xccl_status_t xccl_p2p_group_end(void);
}
