/*
 * xccl-b200: identifiers of team libraries (TLs).
 *
 * Bit positions 0..7 are those of openucx/xccl (src/api/xccl_tls.h:12-24) so that a
 * TLS bitmask built by an existing caller selects the corresponding team here:
 *   ucx    -> the host point-to-point team (shared-memory transport, all collectives)
 *   nccl   -> NCCL library calls (the comparison baseline, pipeline send/recv)
 *   hier   -> hierarchy / schedule layer
 *   mpod   -> pod-split layer, mrail -> multirail replication
 *   sharp  -> in-fabric reduction: served by NVSwitch multimem (NVLS) kernels
 *   hmc    -> hardware multicast broadcast: served by NVSwitch multimem stores
 *   shmseg -> shared-segment team with FANOUT_GET and global memory map
 * Bit 8 (nvlink) is new: hand-written sm_100a kernels over peer memory.
 */
#ifndef XCCL_B200_TLS_H_
#define XCCL_B200_TLS_H_

#include <string.h>
#include <stdint.h>
#include "xccl_def.h"

typedef enum xccl_tl_id {
    XCCL_TL_NULL   = 0,
    XCCL_TL_UCX    = XCCL_BIT(0),
    XCCL_TL_HIER   = XCCL_BIT(1),
    XCCL_TL_SHARP  = XCCL_BIT(2),
    XCCL_TL_HMC    = XCCL_BIT(3),
    XCCL_TL_SHMSEG = XCCL_BIT(4),
    XCCL_TL_MRAIL  = XCCL_BIT(5),
    XCCL_TL_NCCL   = XCCL_BIT(6),
    XCCL_TL_MPOD   = XCCL_BIT(7),
    XCCL_TL_NVLINK = XCCL_BIT(8),
    XCCL_TL_LAST,
    XCCL_TL_ALL    = (XCCL_TL_LAST << 1) - 3
} xccl_tl_id_t;

#define XCCL_TL_COUNT 9

static inline const char *xccl_tl_str(xccl_tl_id_t id)
{
    static const char *const names[XCCL_TL_COUNT] = {
        "ucx", "hier", "sharp", "hmc", "shmseg", "mrail", "nccl", "mpod", "nvlink"
    };
    int i;
    for (i = 0; i < XCCL_TL_COUNT; i++) {
        if ((uint64_t)id == XCCL_BIT(i)) {
            return names[i];
        }
    }
    return NULL;
}

/* "ucx,nccl" -> bitmask. A name matches when it occurs anywhere in the string,
 * which is the reference behaviour (src/api/xccl_tls.h:53-69). */
static inline xccl_tl_id_t xccl_tls_str_to_bitmap(const char *s)
{
    uint64_t bits = 0;
    int      i;
    if (s == NULL) {
        return XCCL_TL_NULL;
    }
    for (i = 0; i < XCCL_TL_COUNT; i++) {
        if (strstr(s, xccl_tl_str((xccl_tl_id_t)XCCL_BIT(i))) != NULL) {
            bits |= XCCL_BIT(i);
        }
    }
    return (xccl_tl_id_t)bits;
}

#endif
