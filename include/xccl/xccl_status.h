/*
 * xccl-b200: status codes returned by every entry point of the library.
 *
 * The numeric values follow the Teams API of openucx/xccl (src/api/xccl_status.h:10-30)
 * so that programs written against it keep their error handling unchanged.
 * XCCL_ERR_TIMED_OUT is an addition: it is what a bounded device-side or host-side
 * wait reports when a peer never arrived.
 */
#ifndef XCCL_B200_STATUS_H_
#define XCCL_B200_STATUS_H_

typedef enum xccl_status {
    XCCL_OK                    = 0,   /* finished */
    XCCL_INPROGRESS            = 1,   /* posted, not finished yet: call test/progress again */

    XCCL_ERR_NO_MESSAGE        = -1,
    XCCL_ERR_NO_RESOURCE       = -2,
    XCCL_ERR_NO_MEMORY         = -4,
    XCCL_ERR_INVALID_PARAM     = -5,
    XCCL_ERR_UNREACHABLE       = -6,
    XCCL_ERR_NOT_IMPLEMENTED   = -8,
    XCCL_ERR_MESSAGE_TRUNCATED = -9,
    XCCL_ERR_NO_PROGRESS       = -10,
    XCCL_ERR_BUFFER_TOO_SMALL  = -11,
    XCCL_ERR_NO_ELEM           = -12,
    XCCL_ERR_UNSUPPORTED       = -22,
    XCCL_ERR_TIMED_OUT         = -30, /* extension: a bounded wait expired */
    XCCL_ERR_LAST              = -100
} xccl_status_t;

#ifdef __cplusplus
extern "C" {
#endif
/* Human-readable name of a status code; never returns NULL. */
const char *xccl_status_str(xccl_status_t st);
#ifdef __cplusplus
}
#endif

#endif
