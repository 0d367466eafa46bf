/*
 * aclnnGroupedMatmulSwigluQuant: grouped int8 GEMM fused with dequantisation, SwiGLU and dynamic per-token int8
 * requantisation, on NVIDIA B200.
 *
 * Drop-in for the reference's entry points declared at
 *   gmm/grouped_matmul_swiglu_quant/op_host/op_api/aclnn_grouped_matmul_swiglu_quant.h:37-52.
 *
 *   x int8 [M, K];  weight int8 [E, K, N] (format ND or FRACTAL_NZ);  weightScale [E, N] fp32 / fp16 / bf16;  xScale fp32 [M];
 *   groupList int64 [<=E], running totals;  output int8 [M, N/2];  outputScale fp32 [M].
 *   C = ((x @ weight[e]) * xScale[m]) * weightScale[e, n];  S = Swish(C[:, :N/2]) * C[:, N/2:];
 *   outputScale = max|S| / 127;  output = int8(rint(half(S * (1 / outputScale)))).
 *   bias, offset and outputOffset are accepted and ignored, as in the reference
 *   (aclnn_grouped_matmul_swiglu_quant.cpp:86-104).  N even, N <= 10240, K < 65536.
 * Rows at and beyond groupList[-1] are left untouched.
 * Layout note: the reference's A8W8 path insists on the FRACTAL_NZ weight storage format
 * (aclnn_grouped_matmul_swiglu_quant.cpp:326-336).  This build takes both: format ACL_FORMAT_FRACTAL_NZ with storage
 * [E, N/32, K/16, 16, 32] (view of 3 or 5 dimensions; K % 16 == 0, N % 32 == 0), read by the tensor cores as it lies,
 * and the plain ND [E, K, N] tensor.
 */
#ifndef B200_ACLNN_GROUPED_MATMUL_SWIGLU_QUANT_H
#define B200_ACLNN_GROUPED_MATMUL_SWIGLU_QUANT_H
#include "aclnn/aclnn_base.h"

#ifdef __cplusplus
extern "C" {
#endif

/* Replaces gmm/grouped_matmul_swiglu_quant/op_host/op_api/aclnn_grouped_matmul_swiglu_quant.h:37-40
 * (aclnn_grouped_matmul_swiglu_quant.cpp:467-481).  Host only; never reads groupList. */
ACL_FUNC_VISIBILITY aclnnStatus aclnnGroupedMatmulSwigluQuantGetWorkspaceSize(
    const aclTensor *x, const aclTensor *weight, const aclTensor *bias, const aclTensor *offset,
    const aclTensor *weightScale, const aclTensor *xScale, const aclTensor *groupList, aclTensor *output,
    aclTensor *outputScale, aclTensor *outputOffset, uint64_t *workspaceSize, aclOpExecutor **executor);

/* Replaces gmm/grouped_matmul_swiglu_quant/op_host/op_api/aclnn_grouped_matmul_swiglu_quant.h:51-52
 * (aclnn_grouped_matmul_swiglu_quant.cpp:518-525).  Enqueues on `stream` and returns; consumes the executor. */
ACL_FUNC_VISIBILITY aclnnStatus aclnnGroupedMatmulSwigluQuant(void *workspace, uint64_t workspaceSize,
                                                              aclOpExecutor *executor, aclrtStream stream);

#ifdef __cplusplus
}
#endif
#endif /* B200_ACLNN_GROUPED_MATMUL_SWIGLU_QUANT_H */
