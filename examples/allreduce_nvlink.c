/*
 * C user of the public API on GPUs: N processes (forked here), one GPU each, form a team served by the NVLink team
 * library and run, in stream order, a persistent gradient-style allreduce (fp32 sum, scaled by 1/N and stored as fp32)
 * and an allgather on device buffers. Bootstrap is the shared-memory out-of-band provider, as in allreduce_host.c.
 * The counterpart in the reference is its CUDA test (test/test_mpi_cuda_allreduce.c:10-93), which drives its UCX team
 * on device memory.
 *
 *   cc -std=c11 -I include -I /usr/local/cuda/include examples/allreduce_nvlink.c -L xccl_b200/lib -lxccl \
 *      -L /usr/local/cuda/lib64 -lcudart -Wl,-rpath,$PWD/xccl_b200/lib -o allreduce_nvlink
 *   ./allreduce_nvlink 2        # needs as many GPUs with peer access as ranks
 */
#define _GNU_SOURCE
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <sys/wait.h>
#include <unistd.h>

#include <cuda_runtime_api.h>

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
#define CUDA(expr)                                                                           \
    do {                                                                                     \
        cudaError_t e_ = (expr);                                                             \
        if (e_ != cudaSuccess) {                                                             \
            fprintf(stderr, "rank %d: %s -> %s\n", rank, #expr, cudaGetErrorString(e_));     \
            return 1;                                                                        \
        }                                                                                    \
    } while (0)

enum { COUNT = 1 << 20, PER = 4096 };

static int run_rank(const char *job, int rank, int size)
{
    /* nothing has touched CUDA before the fork: every process creates its own context here */
    CUDA(cudaSetDevice(rank));
    cudaStream_t stream;
    CUDA(cudaStreamCreateWithFlags(&stream, cudaStreamNonBlocking));

    xccl_oob_collectives_t oob;
    CHECK(xccl_oob_shm_create(job, rank, size, &oob));
    xccl_lib_params_t lib_params = {.field_mask = XCCL_LIB_PARAM_FIELD_TEAM_USAGE,
                                    .team_usage = XCCL_LIB_PARAMS_TEAM_USAGE_SW_COLLECTIVES |
                                                  XCCL_LIB_PARAMS_TEAM_USAGE_HW_COLLECTIVES};
    xccl_lib_h lib;
    CHECK(xccl_lib_init(&lib_params, NULL, &lib));
    xccl_context_params_t ctx_params = {.field_mask = XCCL_CONTEXT_PARAM_FIELD_OOB | XCCL_CONTEXT_PARAM_FIELD_TLS,
                                        .oob        = oob,
                                        .tls        = XCCL_TL_NVLINK | XCCL_TL_UCX};
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
    if (xccl_team_coll_tl(team, XCCL_ALLREDUCE, XCCL_MEMORY_TYPE_CUDA) != XCCL_TL_NVLINK) {
        fprintf(stderr, "rank %d: the NVLink team does not serve this team (no peer access?)\n", rank);
        return 1;
    }

    float *host = (float *)malloc(sizeof(float) * COUNT);
    float *grad, *avg;
    CUDA(cudaMalloc((void **)&grad, sizeof(float) * COUNT));
    CUDA(cudaMalloc((void **)&avg, sizeof(float) * COUNT));

    /* persistent allreduce with the scale fused into its last pass: avg = sum(grad) / size */
    xccl_coll_op_args_t ar;
    memset(&ar, 0, sizeof(ar));
    ar.field_mask             = XCCL_COLL_OP_ARGS_FIELD_STREAM | XCCL_COLL_OP_ARGS_FIELD_EPILOGUE;
    ar.coll_type              = XCCL_ALLREDUCE;
    ar.buffer_info.src_buffer = grad;
    ar.buffer_info.dst_buffer = avg;
    ar.buffer_info.len        = sizeof(float) * COUNT;
    ar.reduce_info.dt         = XCCL_DT_FLOAT32;
    ar.reduce_info.op         = XCCL_OP_SUM;
    ar.reduce_info.count      = COUNT;
    ar.stream.type            = XCCL_STREAM_TYPE_CUDA;
    ar.stream.stream          = &stream;
    ar.epilogue.scale         = 1.0f / (float)size;
    ar.epilogue.out_dt        = XCCL_DT_FLOAT32;
    xccl_coll_req_h req;
    CHECK(xccl_collective_init(&ar, &req, team));
    for (int iter = 0; iter < 3; iter++) {
        for (int i = 0; i < COUNT; i++) host[i] = (float)((i + iter) % 17 + rank);   /* small integers: exact sums */
        CUDA(cudaMemcpyAsync(grad, host, sizeof(float) * COUNT, cudaMemcpyHostToDevice, stream));
        CHECK(xccl_collective_post(req));                /* ordered after the copy: same stream */
        CUDA(cudaMemcpyAsync(host, avg, sizeof(float) * COUNT, cudaMemcpyDeviceToHost, stream));   /* and before this one */
        CUDA(cudaStreamSynchronize(stream));
        CHECK(xccl_collective_test(req));                /* the stream has drained: the request is complete */
        for (int i = 0; i < COUNT; i++) {
            float want = ((float)(size * ((i + iter) % 17)) + (float)(size * (size - 1) / 2)) / (float)size;
            float diff = host[i] - want;
            if (diff > 1e-5f * want + 1e-6f || -diff > 1e-5f * want + 1e-6f) {   /* the kernel multiplies by 1/size */
                fprintf(stderr, "rank %d: allreduce[%d] = %f, expected %f\n", rank, i, host[i], want);
                return 1;
            }
        }
    }
    CHECK(xccl_collective_finalize(req));

    /* allgather of PER ints per rank */
    int *piece, *all, *all_host = (int *)malloc(sizeof(int) * PER * (size_t)size);
    CUDA(cudaMalloc((void **)&piece, sizeof(int) * PER));
    CUDA(cudaMalloc((void **)&all, sizeof(int) * PER * (size_t)size));
    for (int i = 0; i < PER; i++) all_host[i] = rank * 100000 + i;
    CUDA(cudaMemcpyAsync(piece, all_host, sizeof(int) * PER, cudaMemcpyHostToDevice, stream));
    xccl_coll_op_args_t ag;
    memset(&ag, 0, sizeof(ag));
    ag.field_mask             = XCCL_COLL_OP_ARGS_FIELD_STREAM;
    ag.coll_type              = XCCL_ALLGATHER;
    ag.buffer_info.src_buffer = piece;
    ag.buffer_info.dst_buffer = all;
    ag.buffer_info.len        = sizeof(int) * PER * (size_t)size;   /* bytes of the gathered buffer */
    ag.stream.type            = XCCL_STREAM_TYPE_CUDA;
    ag.stream.stream          = &stream;
    CHECK(xccl_collective_init(&ag, &req, team));
    CHECK(xccl_collective_post(req));
    CHECK(xccl_collective_wait(req));
    CHECK(xccl_collective_finalize(req));
    CUDA(cudaMemcpy(all_host, all, sizeof(int) * PER * (size_t)size, cudaMemcpyDeviceToHost));
    for (int r = 0; r < size; r++) {
        for (int i = 0; i < PER; i++) {
            if (all_host[r * PER + i] != r * 100000 + i) {
                fprintf(stderr, "rank %d: allgather[%d][%d] = %d\n", rank, r, i, all_host[r * PER + i]);
                return 1;
            }
        }
    }

    xccl_team_destroy(team);
    CHECK(xccl_context_destroy(ctx));
    xccl_lib_cleanup(lib);
    xccl_oob_shm_destroy(&oob);
    CUDA(cudaFree(grad));
    CUDA(cudaFree(avg));
    CUDA(cudaFree(piece));
    CUDA(cudaFree(all));
    CUDA(cudaStreamDestroy(stream));
    free(host);
    free(all_host);
    if (rank == 0) printf("allreduce and allgather on device buffers correct on %d GPUs\n", size);
    return 0;
}

int main(int argc, char **argv)
{
    int  size = argc > 1 ? atoi(argv[1]) : 2;
    char job[64];
    snprintf(job, sizeof(job), "example-gpu-%d", (int)getpid());
    if (size < 1 || size > 16) return 2;
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
