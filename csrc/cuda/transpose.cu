// Block transpose used by the pod-split alltoall: an array of rows x cols blocks of
// `block_bytes` becomes cols x rows blocks. The reference does this in place by following
// permutation cycles with cudaMemcpyAsync (src/team_lib/mpod/xccl_mpod_alltoall.c:9-96); here it is
// one out-of-place kernel launch.
#include <algorithm>

#include "cuda_common.h"
#include "mem_cuda.h"

namespace xccl {

namespace {
__global__ void block_transpose_kernel(unsigned char *dst, const unsigned char *src, int rows, int cols, size_t block_bytes,
                                       int vec)
{
    const int i = blockIdx.y / cols, j = blockIdx.y % cols;  // source block (i, j)
    const unsigned char *s = src + ((size_t)i * cols + j) * block_bytes;
    unsigned char       *d = dst + ((size_t)j * rows + i) * block_bytes;
    const size_t tid = (size_t)blockIdx.x * blockDim.x + threadIdx.x, nthr = (size_t)gridDim.x * blockDim.x;
    if (vec) {
        const size_t n = block_bytes / 16;
        for (size_t k = tid; k < n; k += nthr) reinterpret_cast<uint4 *>(d)[k] = reinterpret_cast<const uint4 *>(s)[k];
    } else {
        for (size_t k = tid; k < block_bytes; k += nthr) d[k] = s[k];
    }
}
}  // namespace

xccl_status_t cuda_block_transpose(void *dst, const void *src, int rows, int cols, size_t block_bytes, void *stream)
{
    if (rows <= 0 || cols <= 0 || block_bytes == 0) return XCCL_OK;
    int    vec  = ((uintptr_t)dst % 16 == 0) && ((uintptr_t)src % 16 == 0) && (block_bytes % 16 == 0);
    size_t work = vec ? block_bytes / 16 : block_bytes;
    int    gx   = (int)std::min<size_t>((work + 255) / 256, 64);
    dim3   grid((unsigned)std::max(gx, 1), (unsigned)(rows * cols));
    block_transpose_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>((unsigned char *)dst, (const unsigned char *)src, rows,
                                                                 cols, block_bytes, vec);
    XCCL_CUDA_CHECK(cudaGetLastError());
    return XCCL_OK;
}

}  // namespace xccl
