/*
 * aclnnGroupedMatmulWeightNz: aclnnGroupedMatmulV5 for a weight stored in FRACTAL_NZ, on NVIDIA B200.
 *
 * Drop-in for the reference's entry points declared at
 *   gmm/grouped_matmul/op_host/op_api/aclnn_grouped_matmul_weight_nz.h:50-70.
 * The weight's storage is taken to be FRACTAL_NZ whatever its format field says: int8 [E, N/32, K/16, 16, 32], element
 * (k, n) of expert e at ((n/32 * K/16 + k/16) * 16 + k%16) * 32 + n%32.  The view may have 3 ([E, K, N]) or 5 dimensions.
 * K % 16 == 0 and N % 32 == 0.  The tensor cores read that storage directly (a 5-dimensional TMA map with 32-byte
 * swizzle); there is no conversion pass.  quantGroupSize belongs to the reference's per-group-quantised modes and must be
 * non-negative; it has no effect on the per-token int8 mode built here.
 */
#ifndef B200_ACLNN_GROUPED_MATMUL_WEIGHT_NZ_H
#define B200_ACLNN_GROUPED_MATMUL_WEIGHT_NZ_H
#include "aclnn/aclnn_base.h"
#include "aclnnop/aclnn_grouped_matmul_v4.h"

#ifdef __cplusplus
extern "C" {
#endif

/* Replaces gmm/grouped_matmul/op_host/op_api/aclnn_grouped_matmul_weight_nz.h:50-59. */
ACL_FUNC_VISIBILITY aclnnStatus aclnnGroupedMatmulWeightNzGetWorkspaceSize(
    const aclTensorList *x, const aclTensorList *weight, const aclTensorList *biasOptional,
    const aclTensorList *scaleOptional, const aclTensorList *offsetOptional,
    const aclTensorList *antiquantScaleOptional, const aclTensorList *antiquantOffsetOptional,
    const aclTensorList *perTokenScaleOptional, const aclTensor *groupListOptional,
    const aclTensorList *activationInputOptional, const aclTensorList *activationQuantScaleOptional,
    const aclTensorList *activationQuantOffsetOptional, int64_t splitItem, int64_t groupType, int64_t groupListType,
    int64_t actType, aclIntArray *tuningConfigOptional, int64_t quantGroupSize, aclTensorList *out,
    aclTensorList *activationFeatureOutOptional, aclTensorList *dynQuantScaleOutOptional, uint64_t *workspaceSize,
    aclOpExecutor **executor);

/* Replaces gmm/grouped_matmul/op_host/op_api/aclnn_grouped_matmul_weight_nz.h:69-70. */
ACL_FUNC_VISIBILITY aclnnStatus aclnnGroupedMatmulWeightNz(void *workspace, uint64_t workspaceSize,
                                                           aclOpExecutor *executor, aclrtStream stream);

#ifdef __cplusplus
}
#endif
#endif /* B200_ACLNN_GROUPED_MATMUL_WEIGHT_NZ_H */
