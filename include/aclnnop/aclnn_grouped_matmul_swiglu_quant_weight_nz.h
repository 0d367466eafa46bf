/*
 * aclnnGroupedMatmulSwigluQuantWeightNZ: aclnnGroupedMatmulSwigluQuant for a weight stored in FRACTAL_NZ, on NVIDIA B200.
 *
 * Drop-in for the reference's entry points declared at
 *   gmm/grouped_matmul_swiglu_quant/op_host/op_api/aclnn_grouped_matmul_swiglu_quant_weight_nz.h:37-54
 * (aclnn_grouped_matmul_swiglu_quant.cpp:483-516).  The weight's storage shape must have 5 dimensions
 * ([E, N/32, K/16, 16, 32], int8) and is treated as FRACTAL_NZ unconditionally; the view may have 3 or 5 dimensions.
 * K % 16 == 0 and N % 32 == 0.  Arithmetic and outputs are those of aclnn_grouped_matmul_swiglu_quant.h.
 */
#ifndef B200_ACLNN_GROUPED_MATMUL_SWIGLU_QUANT_WEIGHT_NZ_H
#define B200_ACLNN_GROUPED_MATMUL_SWIGLU_QUANT_WEIGHT_NZ_H
#include "aclnn/aclnn_base.h"

#ifdef __cplusplus
extern "C" {
#endif

/* Replaces gmm/grouped_matmul_swiglu_quant/op_host/op_api/aclnn_grouped_matmul_swiglu_quant_weight_nz.h:37-40. */
ACL_FUNC_VISIBILITY aclnnStatus aclnnGroupedMatmulSwigluQuantWeightNZGetWorkspaceSize(
    const aclTensor *x, const aclTensor *weight, const aclTensor *bias, const aclTensor *offset,
    const aclTensor *weightScale, const aclTensor *xScale, const aclTensor *groupList, aclTensor *output,
    aclTensor *outputScale, aclTensor *outputOffset, uint64_t *workspaceSize, aclOpExecutor **executor);

/* Replaces gmm/grouped_matmul_swiglu_quant/op_host/op_api/aclnn_grouped_matmul_swiglu_quant_weight_nz.h:51-54. */
ACL_FUNC_VISIBILITY aclnnStatus aclnnGroupedMatmulSwigluQuantWeightNZ(void *workspace, uint64_t workspaceSize,
                                                                      aclOpExecutor *executor, aclrtStream stream);

#ifdef __cplusplus
}
#endif
#endif /* B200_ACLNN_GROUPED_MATMUL_SWIGLU_QUANT_WEIGHT_NZ_H */
