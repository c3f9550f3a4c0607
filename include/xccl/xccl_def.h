/*
 * xccl-b200: opaque handle types of the public API.
 * Same handle names as openucx/xccl (src/api/xccl_def.h:13-56).
 */
#ifndef XCCL_B200_DEF_H_
#define XCCL_B200_DEF_H_

#include <stddef.h>
#include <stdint.h>

#define XCCL_BIT(i)  (1ull << (i))
#define XCCL_MASK(i) (XCCL_BIT(i) - 1)

/* library instance: the set of team libraries usable by contexts made from it */
typedef struct xccl_lib         *xccl_lib_h;
/* communication context: per-process resources of every selected team library */
typedef struct xccl_context     *xccl_context_h;
/* team: an ordered group of context endpoints that run collectives together */
typedef struct xccl_team        *xccl_team_h;
/* persistent collective request: init once, post any number of times */
typedef struct xccl_coll_req    *xccl_coll_req_h;
/* team-wide memory registration */
typedef struct xccl_mem_handle  *xccl_mem_h;

typedef struct xccl_lib_config     xccl_lib_config_t;
typedef struct xccl_context_config xccl_context_config_t;

/* where a buffer lives; detected per collective from the source pointer */
typedef enum xccl_memory_type {
    XCCL_MEMORY_TYPE_HOST = 0,
    XCCL_MEMORY_TYPE_CUDA = 1,
    XCCL_MEMORY_TYPE_LAST
} xccl_memory_type_t;

#endif
