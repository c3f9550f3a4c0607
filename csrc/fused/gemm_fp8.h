// Block-scaled fp8 GEMM entry point (extension). A8: [M,K] e4m3, sa: [M, K/128] fp32 (one scale
// per row per 128 columns); B8: [N,K] e4m3, sb: [N/128, K/128] fp32 (one scale per 128 x 128 block);
// C: [M,N] bf16. K and N must be multiples of 128. Errors of bounded waits are reported through
// xccl_gemm_last_error().
#pragma once
#include "xccl/xccl.h"

#ifdef __cplusplus
extern "C" {
#endif
xccl_status_t xccl_gemm_fp8_blockscaled(const void *A8, const float *sa, const void *B8, const float *sb, void *C, int M,
                                        int N, int K, void *stream);
#ifdef __cplusplus
}
#endif
