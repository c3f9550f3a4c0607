/*
 * xccl-b200 public C API.
 *
 * A collective communication library for one NVLink 5 / NVSwitch box of B200 GPUs with the
 * Teams API of openucx/xccl: lib -> context -> team -> persistent collective request.
 * Every name and numeric value that exists in openucx/xccl (src/api/xccl.h:31-530) keeps
 * its meaning; additions are marked "extension".
 *
 * Conventions that callers rely on (all taken from the reference's behaviour):
 *  - buffer_info.len is the total byte count for allreduce / reduce / bcast, the byte count
 *    PER PEER for alltoall, and the byte count of the WHOLE gathered result for allgather.
 *  - alltoallv counts and displacements are element counts of src_datatype / dst_datatype.
 *  - src_buffer == XCCL_IN_PLACE means "operate on dst_buffer".
 *  - stream.stream points AT a cudaStream_t; it is not the stream value itself.
 *  - Ranks of a team must call collective_init / post in the same order.
 */
#ifndef XCCL_B200_H_
#define XCCL_B200_H_

#include <stdio.h>
#include <stddef.h>
#include <stdint.h>

#include "xccl_def.h"
#include "xccl_status.h"
#include "xccl_tls.h"
#include "xccl_version.h"

#ifdef __cplusplus
extern "C" {
#endif

/* ------------------------------------------------------------------ library ---------- */

enum xccl_lib_params_field {
    XCCL_LIB_PARAM_FIELD_REPRODUCIBLE = XCCL_BIT(0),
    XCCL_LIB_PARAM_FIELD_THREAD_MODE  = XCCL_BIT(1),
    XCCL_LIB_PARAM_FIELD_TEAM_USAGE   = XCCL_BIT(2),
    XCCL_LIB_PARAM_FIELD_COLL_TYPES   = XCCL_BIT(4)
};

enum xccl_reproducibility_mode {
    XCCL_REPRODUCIBILITY_MODE_REPRODUCIBLE     = XCCL_BIT(0),
    XCCL_REPRODUCIBILITY_MODE_NON_REPRODUCIBLE = XCCL_BIT(1)
};

enum xccl_thread_mode {
    XCCL_THREAD_MODE_MULTIPLE = XCCL_BIT(0),
    XCCL_THREAD_MODE_SINGLE   = XCCL_BIT(1)
};

enum xccl_lib_params_team_usage_field {
    XCCL_LIB_PARAMS_TEAM_USAGE_HW_COLLECTIVES = XCCL_BIT(0),
    XCCL_LIB_PARAMS_TEAM_USAGE_SW_COLLECTIVES = XCCL_BIT(1)
};

typedef enum {
    XCCL_BARRIER = 0,
    XCCL_BCAST,
    XCCL_ALLREDUCE,
    XCCL_REDUCE,
    XCCL_ALLTOALL,
    XCCL_ALLTOALLV,
    XCCL_ALLGATHER,
    XCCL_FANIN,
    XCCL_FANOUT,
    XCCL_FANOUT_GET,
    XCCL_REDUCE_SCATTER,   /* extension: block r of the reduced vector lands on rank r */
    XCCL_COLL_LAST
} xccl_collective_type_t;

typedef enum {
    XCCL_COLL_CAP_BARRIER        = XCCL_BIT(XCCL_BARRIER),
    XCCL_COLL_CAP_BCAST          = XCCL_BIT(XCCL_BCAST),
    XCCL_COLL_CAP_ALLREDUCE      = XCCL_BIT(XCCL_ALLREDUCE),
    XCCL_COLL_CAP_REDUCE         = XCCL_BIT(XCCL_REDUCE),
    XCCL_COLL_CAP_ALLTOALL       = XCCL_BIT(XCCL_ALLTOALL),
    XCCL_COLL_CAP_ALLTOALLV      = XCCL_BIT(XCCL_ALLTOALLV),
    XCCL_COLL_CAP_ALLGATHER      = XCCL_BIT(XCCL_ALLGATHER),
    XCCL_COLL_CAP_FANIN          = XCCL_BIT(XCCL_FANIN),
    XCCL_COLL_CAP_FANOUT         = XCCL_BIT(XCCL_FANOUT),
    XCCL_COLL_CAP_FANOUT_GET     = XCCL_BIT(XCCL_FANOUT_GET),
    XCCL_COLL_CAP_REDUCE_SCATTER = XCCL_BIT(XCCL_REDUCE_SCATTER),
    XCCL_COLL_CAP_ALL            = XCCL_MASK(XCCL_COLL_LAST)
} xccl_collective_cap_t;

/* Filters the team libraries a lib instance exposes: a TL is kept when its capabilities
 * intersect every field selected by field_mask. */
typedef struct xccl_lib_params {
    uint64_t field_mask;
    unsigned reproducible;
    unsigned thread_mode;
    uint64_t team_usage;
    uint64_t coll_types;
} xccl_lib_params_t;

typedef unsigned xccl_config_print_flags_t;
#define XCCL_CONFIG_PRINT_CONFIG XCCL_BIT(0)
#define XCCL_CONFIG_PRINT_HEADER XCCL_BIT(1)
#define XCCL_CONFIG_PRINT_DOC    XCCL_BIT(2)

/* Reads the global options from the environment. With a prefix P the variables looked up
 * are P_XCCL_*, with the plain XCCL_* names as fallback. `filename` may name a file of
 * NAME=VALUE lines; a missing file is not an error. */
xccl_status_t xccl_lib_config_read(const char *env_prefix, const char *filename,
                                   xccl_lib_config_t **config_p);
void          xccl_lib_config_release(xccl_lib_config_t *config);
void          xccl_lib_config_print(const xccl_lib_config_t *config, FILE *stream,
                                    const char *title, xccl_config_print_flags_t flags);

xccl_status_t xccl_lib_init(const xccl_lib_params_t *params, const xccl_lib_config_t *config,
                            xccl_lib_h *lib_p);
void          xccl_lib_cleanup(xccl_lib_h lib);

/* ------------------------------------------------------------------ queries ---------- */

xccl_status_t xccl_get_tl_list(xccl_lib_h lib, xccl_tl_id_t **tls, unsigned *tl_count);
void          xccl_free_tl_list(xccl_tl_id_t *tls);

enum xccl_tl_attr_field {
    XCCL_TL_ATTR_FIELD_CONTEXT_CREATE_MODE = XCCL_BIT(0),
    XCCL_TL_ATTR_FIELD_DEVICES_COUNT       = XCCL_BIT(1),
    XCCL_TL_ATTR_FILED_DEVICES             = XCCL_BIT(2), /* spelling kept for source compatibility */
    XCCL_TL_ATTR_FIELD_DEVICES             = XCCL_BIT(2)
};

typedef enum {
    XCCL_TEAM_LIB_CONTEXT_CREATE_MODE_LOCAL  = 0,
    XCCL_TEAM_LIB_CONTEXT_CREATE_MODE_GLOBAL = 1
} xccl_context_create_mode_t;

typedef struct xccl_tl_attr {
    uint64_t                   field_mask;
    xccl_context_create_mode_t context_create_mode;
    int                        devices_count;
    char                     (*devices)[16];
} xccl_tl_attr_t;

xccl_status_t xccl_tl_query(xccl_lib_h lib, xccl_tl_id_t *tl, xccl_tl_attr_t *attr);
void          xccl_free_tl_attr(xccl_tl_attr_t *attr);

enum xccl_ctx_attr_field {
    XCCL_CTX_ATTR_FIELD_SUPPORTED_COLLS = XCCL_BIT(0)
};

typedef struct xccl_ctx_attr {
    uint64_t field_mask;
    uint64_t supported_colls;
} xccl_ctx_attr_t;

xccl_status_t xccl_ctx_query(xccl_context_h ctx, xccl_ctx_attr_t *attr);
void          xccl_free_ctx_attr(xccl_ctx_attr_t *attr);

/* ------------------------------------------------------------------ endpoint ranges -- */

typedef enum {
    XCCL_EP_RANGE_UNDEFINED = 0, /* the library decides; identity in practice */
    XCCL_EP_RANGE_FULL      = 1, /* team rank i is context rank i */
    XCCL_EP_RANGE_STRIDED   = 2, /* start + i * stride */
    XCCL_EP_RANGE_MAP       = 3, /* map[i] */
    XCCL_EP_RANGE_CB        = 4  /* cb(i, cb_ctx) */
} xccl_ep_range_type_t;

struct xccl_ep_range_strided { int start; int stride; };
struct xccl_ep_range_map     { int *map; };
struct xccl_ep_range_cb      { int (*cb)(int rank, void *cb_ctx); void *cb_ctx; };

typedef struct xccl_ep_range_t {
    xccl_ep_range_type_t type;
    int                  ep_num;
    union {
        struct xccl_ep_range_strided strided;
        struct xccl_ep_range_map     map;
        struct xccl_ep_range_cb      cb;
    };
} xccl_ep_range_t;

/* team rank -> context rank; -1 for an undefined range */
static inline int xccl_range_to_rank(xccl_ep_range_t range, int rank)
{
    if (range.type == XCCL_EP_RANGE_FULL)    return rank;
    if (range.type == XCCL_EP_RANGE_STRIDED) return range.strided.start + rank * range.strided.stride;
    if (range.type == XCCL_EP_RANGE_MAP)     return range.map.map[rank];
    if (range.type == XCCL_EP_RANGE_CB)      return range.cb.cb(rank, range.cb.cb_ctx);
    return -1;
}

/* ------------------------------------------------------------------ out-of-band ------ */

/* The one bootstrap primitive the library needs from its caller: a non-blocking allgather.
 * allgather() starts gathering `size` bytes from each member and may finish at once;
 * req_test() says XCCL_OK or XCCL_INPROGRESS; req_free() releases the request.
 * With range.type == XCCL_EP_RANGE_UNDEFINED the group is all of coll_context; otherwise the
 * group has range.ep_num members, my_rank is the caller's index in it and member i is
 * context rank xccl_range_to_rank(range, i). One OOB allgather per context is in flight at
 * a time. See xccl_oob.h for ready-made providers. */
typedef struct xccl_oob_collectives {
    int           (*allgather)(void *src_buf, void *recv_buf, size_t size, int my_rank,
                               xccl_ep_range_t range, void *coll_context, void **request);
    xccl_status_t (*req_test)(void *request);
    xccl_status_t (*req_free)(void *request);
    void          *coll_context;
    int            rank;
    int            size;
} xccl_oob_collectives_t;

/* ------------------------------------------------------------------ context ---------- */

enum xccl_context_params_field {
    XCCL_CONTEXT_PARAM_FIELD_THREAD_MODE          = XCCL_BIT(0),
    XCCL_CONTEXT_PARAM_FIELD_TEAM_COMPLETION_TYPE = XCCL_BIT(1),
    XCCL_CONTEXT_PARAM_FIELD_OOB                  = XCCL_BIT(2),
    XCCL_CONTEXT_PARAM_FIELD_TLS                  = XCCL_BIT(3)
};

typedef enum xccl_team_completion_type {
    XCCL_TEAM_COMPLETION_TYPE_BLOCKING    = 0,
    XCCL_TEAM_COMPLETION_TYPE_NONBLOCKING = 1,
    XCCL_TEAM_COMPLETION_TYPE_SPLIT_PHASE = 2
} xccl_team_completion_type_t;

typedef struct xccl_context_params {
    uint64_t                    field_mask;
    unsigned                    thread_mode;
    xccl_team_completion_type_t completion_type;
    xccl_oob_collectives_t      oob;
    uint64_t                    tls;    /* bitmask of xccl_tl_id_t; all TLs when the field is unset */
} xccl_context_params_t;

/* Per-TL context options come from XCCL_TEAM_<TL>_<NAME>; with env_prefix P the lookup is
 * P_XCCL_TEAM_<TL>_<NAME> first. config_modify overrides one option of one TL by name. */
xccl_status_t xccl_context_config_read(xccl_lib_h lib, const char *env_prefix, const char *filename,
                                       xccl_context_config_t **config);
xccl_status_t xccl_context_config_modify(xccl_tl_id_t *tl_id, xccl_context_config_t *config,
                                         const char *name, const char *value);
void          xccl_context_config_release(xccl_context_config_t *config);

xccl_status_t xccl_context_create(xccl_lib_h lib, const xccl_context_params_t *params,
                                  const xccl_context_config_t *config, xccl_context_h *context);
/* Drives every host-progressed team library and the context's task queue once. */
xccl_status_t xccl_context_progress(xccl_context_h context);
xccl_status_t xccl_context_destroy(xccl_context_h context);

/* ------------------------------------------------------------------ team ------------- */

enum xccl_team_params_field {
    XCCL_TEAM_PARAM_FIELD_EP_RANGE = XCCL_BIT(0),
    XCCL_TEAM_PARAM_FIELD_OOB      = XCCL_BIT(1)
};

typedef struct xccl_team_params {
    uint64_t               field_mask;
    xccl_ep_range_t        range;
    xccl_oob_collectives_t oob;
} xccl_team_params_t;

/* Non-blocking: post, then call test until it stops returning XCCL_INPROGRESS. */
xccl_status_t xccl_team_create_post(xccl_context_h context, xccl_team_params_t *params,
                                    xccl_team_h *team);
xccl_status_t xccl_team_create_test(xccl_team_h team);
void          xccl_team_destroy(xccl_team_h team);

/* ------------------------------------------------------------------ collectives ------ */

typedef enum {
    XCCL_OP_MAX,
    XCCL_OP_MIN,
    XCCL_OP_SUM,
    XCCL_OP_PROD,
    XCCL_OP_AND,
    XCCL_OP_OR,
    XCCL_OP_XOR,
    XCCL_OP_LAND,
    XCCL_OP_LOR,
    XCCL_OP_LXOR,
    XCCL_OP_BAND,
    XCCL_OP_BOR,
    XCCL_OP_BXOR,
    XCCL_OP_MAXLOC,
    XCCL_OP_MINLOC,
    XCCL_OP_LAST_PREDEFINED,
    XCCL_OP_UNSUPPORTED
} xccl_op_t;

typedef enum {
    XCCL_DT_INT8,
    XCCL_DT_INT16,
    XCCL_DT_INT32,
    XCCL_DT_INT64,
    XCCL_DT_INT128,
    XCCL_DT_UINT8,
    XCCL_DT_UINT16,
    XCCL_DT_UINT32,
    XCCL_DT_UINT64,
    XCCL_DT_UINT128,
    XCCL_DT_FLOAT16,
    XCCL_DT_FLOAT32,
    XCCL_DT_FLOAT64,
    XCCL_DT_BFLOAT16,       /* extension */
    XCCL_DT_LAST_PREDEFINED,
    XCCL_DT_UNSUPPORTED
} xccl_dt_t;

static inline size_t xccl_dt_size(xccl_dt_t dt)
{
    static const unsigned char bytes[XCCL_DT_LAST_PREDEFINED] = {
        1, 2, 4, 8, 16,   /* int8 .. int128   */
        1, 2, 4, 8, 16,   /* uint8 .. uint128 */
        2, 4, 8,          /* fp16, fp32, fp64 */
        2                 /* bf16             */
    };
    return ((unsigned)dt < (unsigned)XCCL_DT_LAST_PREDEFINED) ? bytes[dt] : 0;
}

#define XCCL_IN_PLACE ((void *)0x1)

typedef struct xccl_reduce_info {
    xccl_dt_t dt;
    xccl_op_t op;
    size_t    count;
} xccl_reduce_info_t;

typedef struct xccl_coll_buffer_info {
    void      *src_buffer;
    uint32_t  *src_counts;
    uint32_t  *src_displacements;
    xccl_dt_t  src_datatype;
    void      *dst_buffer;
    uint32_t  *dst_counts;
    uint32_t  *dst_displacements;
    xccl_dt_t  dst_datatype;
    size_t     len;
} xccl_coll_buffer_info_t;

/* XCCL_FANOUT_GET: every rank copies `len` bytes at `offset` of the root's mapped region */
typedef struct xccl_coll_get_info {
    xccl_mem_h memh;
    ptrdiff_t  offset;
    void      *local_buffer;
    size_t     len;
} xccl_coll_get_info_t;

typedef struct xccl_coll_algorithm {
    uint8_t set_by_user : 1;
    uint8_t id          : 7;
} xccl_coll_algorithm_t;

typedef enum {
    XCCL_STREAM_TYPE_CUDA
} xccl_stream_type_t;

typedef struct xccl_stream {
    xccl_stream_type_t type;
    void              *stream;  /* address of a cudaStream_t */
} xccl_stream_t;

enum xccl_coll_op_args_field {
    XCCL_COLL_OP_ARGS_FIELD_STREAM   = XCCL_BIT(0),
    XCCL_COLL_OP_ARGS_FIELD_EPILOGUE = XCCL_BIT(1)  /* extension: `epilogue` below is valid */
};

/* extension: work fused into the last pass of a reduction. The reduced value is multiplied
 * by `scale` (skipped when exactly 1) and stored as `out_dt`; XCCL_DT_UNSUPPORTED keeps the
 * reduction datatype. Accumulation of fp16/bf16 is always in fp32. Typical use: gradient
 * averaging (scale = 1/world) with an fp32 -> bf16 cast in the same kernel. */
typedef struct xccl_coll_epilogue {
    float     scale;
    xccl_dt_t out_dt;
} xccl_coll_epilogue_t;

typedef struct xccl_coll_op_args {
    uint64_t               field_mask;
    xccl_collective_type_t coll_type;
    union {
        xccl_coll_buffer_info_t buffer_info;
        xccl_coll_get_info_t    get_info;
    };
    xccl_reduce_info_t     reduce_info;
    int                    root;
    xccl_coll_algorithm_t  alg;
    uint16_t               tag;
    xccl_stream_t          stream;
    xccl_coll_epilogue_t   epilogue;   /* extension, read only with ..._FIELD_EPILOGUE */
} xccl_coll_op_args_t;

/* Algorithm ids accepted in alg.id when alg.set_by_user is 1. */
enum xccl_host_alg_id {                 /* host ("ucx") team */
    XCCL_HOST_ALG_LINEAR = 0,           /* reduce, bcast: linear; alltoall: pairwise */
    XCCL_HOST_ALG_KNOMIAL = 1,          /* allreduce: recursive k-nomial; bcast/reduce: k-nomial tree;
                                           alltoall: in-place linear shift */
    XCCL_HOST_ALG_SRA = 2               /* allreduce: scatter-reduce + allgather */
};
enum xccl_nvlink_alg_id {               /* nvlink team allreduce */
    XCCL_NVLINK_ALG_AUTO = 0,
    XCCL_NVLINK_ALG_ONE_SHOT = 1,
    XCCL_NVLINK_ALG_TWO_SHOT = 2,
    XCCL_NVLINK_ALG_NVLS = 3,
    XCCL_NVLINK_ALG_DIRECT = 4,  /* zero-copy kernels on buffers registered with the peers at init */
    XCCL_NVLINK_ALG_SYMMETRIC = 5 /* in-switch reduction and multicast directly on buffers from xccl_team_mem_alloc */
};

/* Persistent request life cycle. init captures the arguments; post starts one execution and
 * may be repeated after the previous execution has completed; test/wait observe completion;
 * finalize releases a request that is not in flight. */
xccl_status_t xccl_collective_init(xccl_coll_op_args_t *coll_args, xccl_coll_req_h *request,
                                   xccl_team_h team);
xccl_status_t xccl_collective_post(xccl_coll_req_h request);
xccl_status_t xccl_collective_wait(xccl_coll_req_h request);
xccl_status_t xccl_collective_test(xccl_coll_req_h request);
xccl_status_t xccl_collective_finalize(xccl_coll_req_h request);

/* ------------------------------------------------------------------ global memory ---- */

typedef enum xccl_mem_map_params_field_mask {
    XCCL_MEM_MAP_PARAM_FIELD_ADDRESS = XCCL_BIT(0),
    XCCL_MEM_MAP_PARAM_FIELD_LENGTH  = XCCL_BIT(1),
    XCCL_MEM_MAP_PARAM_FIELD_ROOT    = XCCL_BIT(2)
} xccl_mem_map_params_field_mask_t;

/* A region owned by team rank `root` that every member can read afterwards. */
typedef struct xccl_mem_map_params {
    uint64_t field_mask;
    void    *address;
    size_t   length;
    int      root;
} xccl_mem_map_params_t;

xccl_status_t xccl_global_mem_map_start(xccl_team_h team, xccl_mem_map_params_t params,
                                        xccl_mem_h *memh_p);
xccl_status_t xccl_global_mem_map_test(xccl_mem_h memh);
xccl_status_t xccl_global_mem_unmap(xccl_mem_h memh);

/* ------------------------------------------------------------------ extensions ------- */

/* Size and rank of a created team. */
xccl_status_t xccl_team_query(xccl_team_h team, int *rank, int *size);
/* Which TL serves (coll, memory type) on this team; XCCL_TL_NULL when none does. */
xccl_tl_id_t  xccl_team_coll_tl(xccl_team_h team, xccl_collective_type_t coll, xccl_memory_type_t mem);
/* Symmetric device memory (extension; collective over the team: every member calls it with the same
 * size, in the same order relative to its other collective calls on the team). Each member gets `bytes`
 * of device memory on its own GPU that every other member has mapped and that is bound to the NVSwitch
 * multicast object when the fabric offers one. Collectives whose buffers lie in such memory, at the SAME
 * OFFSET of the allocation on every member, run zero-copy: the in-switch reduction (multimem.ld_reduce)
 * reads the source buffers in place and the multicast store writes the destinations in place, nothing is
 * staged through the team's workspace. This is the NVSwitch counterpart of registering user buffers with
 * the SHARP library. XCCL_ERR_NOT_IMPLEMENTED when no team library of the team offers it. Memory is
 * returned with xccl_team_mem_free (collective too) or when the team is destroyed. */
xccl_status_t xccl_team_mem_alloc(xccl_team_h team, size_t bytes, void **ptr);
xccl_status_t xccl_team_mem_free(xccl_team_h team, void *ptr);
/* Device time of the last completed execution of a CUDA request in microseconds, or a
 * negative value when the request keeps no timing (host requests, timing disabled). */
double        xccl_collective_elapsed_us(xccl_coll_req_h request);

#ifdef __cplusplus
}
#endif

#endif
