/*
 * Minimal C user of the public API: N processes (forked here) form a team over the shared-memory
 * out-of-band provider and run a persistent allreduce, a broadcast and a barrier on host buffers.
 * The call sequence is the one of the reference's own test driver (test/test_mpi.c:99-197,
 * test/test_mpi_allreduce.c): lib -> context -> team -> collective init/post/test/finalize.
 *
 *   cc -std=c11 -I include examples/allreduce_host.c -L xccl_b200/lib -lxccl -Wl,-rpath,$PWD/xccl_b200/lib -o allreduce_host
 *   ./allreduce_host 4
 */
#define _GNU_SOURCE
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <sys/wait.h>
#include <unistd.h>

#include <xccl/xccl.h>
#include <xccl/xccl_oob.h>

#define CHECK(expr)                                                                          \
    do {                                                                                     \
        xccl_status_t st_ = (expr);                                                          \
        if (st_ != XCCL_OK) {                                                                \
            fprintf(stderr, "rank %d: %s -> %s\n", rank, #expr, xccl_status_str(st_));       \
            return 1;                                                                        \
        }                                                                                    \
    } while (0)

static int run_rank(const char *job, int rank, int size)
{
    xccl_oob_collectives_t oob;
    CHECK(xccl_oob_shm_create(job, rank, size, &oob));

    xccl_lib_params_t lib_params = {.field_mask = XCCL_LIB_PARAM_FIELD_TEAM_USAGE,
                                    .team_usage = XCCL_LIB_PARAMS_TEAM_USAGE_SW_COLLECTIVES |
                                                  XCCL_LIB_PARAMS_TEAM_USAGE_HW_COLLECTIVES};
    xccl_lib_h lib;
    CHECK(xccl_lib_init(&lib_params, NULL, &lib));

    xccl_context_params_t ctx_params = {.field_mask = XCCL_CONTEXT_PARAM_FIELD_OOB | XCCL_CONTEXT_PARAM_FIELD_TLS |
                                                      XCCL_CONTEXT_PARAM_FIELD_THREAD_MODE,
                                        .thread_mode = XCCL_THREAD_MODE_SINGLE,
                                        .oob         = oob,
                                        .tls         = XCCL_TL_UCX};
    xccl_context_config_t *cfg;
    xccl_context_h         ctx;
    CHECK(xccl_context_config_read(lib, NULL, NULL, &cfg));
    CHECK(xccl_context_create(lib, &ctx_params, cfg, &ctx));
    xccl_context_config_release(cfg);

    xccl_team_params_t team_params = {.field_mask = XCCL_TEAM_PARAM_FIELD_EP_RANGE,
                                      .range      = {.type = XCCL_EP_RANGE_FULL, .ep_num = size}};
    xccl_team_h        team;
    CHECK(xccl_team_create_post(ctx, &team_params, &team));
    xccl_status_t st;
    while ((st = xccl_team_create_test(team)) == XCCL_INPROGRESS) xccl_context_progress(ctx);
    CHECK(st);

    enum { COUNT = 4096 };
    static int src[COUNT], dst[COUNT];
    for (int i = 0; i < COUNT; i++) src[i] = i % 13 + rank;

    xccl_coll_op_args_t ar;
    memset(&ar, 0, sizeof(ar));
    ar.coll_type              = XCCL_ALLREDUCE;
    ar.buffer_info.src_buffer = src;
    ar.buffer_info.dst_buffer = dst;
    ar.buffer_info.len        = sizeof(src);
    ar.reduce_info.dt         = XCCL_DT_INT32;
    ar.reduce_info.op         = XCCL_OP_SUM;
    ar.reduce_info.count      = COUNT;
    xccl_coll_req_h req;
    CHECK(xccl_collective_init(&ar, &req, team));
    for (int iter = 0; iter < 3; iter++) {          /* persistent: post the same request again */
        memset(dst, 0, sizeof(dst));
        CHECK(xccl_collective_post(req));
        while ((st = xccl_collective_test(req)) == XCCL_INPROGRESS) xccl_context_progress(ctx);
        CHECK(st);
        for (int i = 0; i < COUNT; i++) {
            int want = size * (i % 13) + size * (size - 1) / 2;
            if (dst[i] != want) {
                fprintf(stderr, "rank %d: allreduce[%d] = %d, expected %d\n", rank, i, dst[i], want);
                return 1;
            }
        }
    }
    CHECK(xccl_collective_finalize(req));

    double msg[8];
    for (int i = 0; i < 8; i++) msg[i] = rank == 1 % size ? 2.5 * i : -1.0;
    xccl_coll_op_args_t bc;
    memset(&bc, 0, sizeof(bc));
    bc.coll_type              = XCCL_BCAST;
    bc.buffer_info.src_buffer = msg;
    bc.buffer_info.dst_buffer = msg;
    bc.buffer_info.len        = sizeof(msg);
    bc.root                   = 1 % size;
    CHECK(xccl_collective_init(&bc, &req, team));
    CHECK(xccl_collective_post(req));
    CHECK(xccl_collective_wait(req));
    CHECK(xccl_collective_finalize(req));
    for (int i = 0; i < 8; i++) {
        if (msg[i] != 2.5 * i) {
            fprintf(stderr, "rank %d: bcast[%d] = %f\n", rank, i, msg[i]);
            return 1;
        }
    }

    xccl_coll_op_args_t bar;
    memset(&bar, 0, sizeof(bar));
    bar.coll_type = XCCL_BARRIER;
    CHECK(xccl_collective_init(&bar, &req, team));
    CHECK(xccl_collective_post(req));
    CHECK(xccl_collective_wait(req));
    CHECK(xccl_collective_finalize(req));

    xccl_team_destroy(team);
    CHECK(xccl_context_destroy(ctx));
    xccl_lib_cleanup(lib);
    xccl_oob_shm_destroy(&oob);
    if (rank == 0) printf("allreduce, bcast and barrier correct on %d ranks\n", size);
    return 0;
}

int main(int argc, char **argv)
{
    int  size = argc > 1 ? atoi(argv[1]) : 4;
    char job[64];
    snprintf(job, sizeof(job), "example-%d", (int)getpid());
    if (size < 1 || size > 64) return 2;
    for (int r = 1; r < size; r++) {
        pid_t pid = fork();
        if (pid == 0) _exit(run_rank(job, r, size));
        if (pid < 0) return 2;
    }
    int rc = run_rank(job, 0, size), status = 0;
    while (wait(&status) > 0) {
        if (!WIFEXITED(status) || WEXITSTATUS(status) != 0) rc = 1;
    }
    return rc;
}
