/*
 * aclnnGroupedMatmulV5: aclnnGroupedMatmulV4 plus tuningConfigOptional, on NVIDIA B200.
 *
 * Drop-in for the reference's entry points declared at
 *   gmm/grouped_matmul/op_host/op_api/aclnn_grouped_matmul_v5.h:49-69.
 * tuningConfigOptional[0] is the number of rows the caller expects per group; the reference feeds it to its host tiling
 * (aclnn_grouped_matmul.cpp:1336-1360).  Here the tile schedule is built on the device from group_list itself; the value
 * is validated (no negative entries) and, when positive, replaces M / len(group_list) in the choice between 128-row tiles
 * and 256-row CTA-pair tiles (pairs from 384 rows per group), which helps when many groups are empty.  Everything else is
 * as in aclnn_grouped_matmul_v4.h.
 */
#ifndef B200_ACLNN_GROUPED_MATMUL_V5_H
#define B200_ACLNN_GROUPED_MATMUL_V5_H
#include "aclnn/aclnn_base.h"
#include "aclnnop/aclnn_grouped_matmul_v4.h"

#ifdef __cplusplus
extern "C" {
#endif

/* Replaces gmm/grouped_matmul/op_host/op_api/aclnn_grouped_matmul_v5.h:49-58. */
ACL_FUNC_VISIBILITY aclnnStatus aclnnGroupedMatmulV5GetWorkspaceSize(
    const aclTensorList *x, const aclTensorList *weight, const aclTensorList *biasOptional,
    const aclTensorList *scaleOptional, const aclTensorList *offsetOptional,
    const aclTensorList *antiquantScaleOptional, const aclTensorList *antiquantOffsetOptional,
    const aclTensorList *perTokenScaleOptional, const aclTensor *groupListOptional,
    const aclTensorList *activationInputOptional, const aclTensorList *activationQuantScaleOptional,
    const aclTensorList *activationQuantOffsetOptional, int64_t splitItem, int64_t groupType, int64_t groupListType,
    int64_t actType, aclIntArray *tuningConfigOptional, aclTensorList *out, aclTensorList *activationFeatureOutOptional,
    aclTensorList *dynQuantScaleOutOptional, uint64_t *workspaceSize, aclOpExecutor **executor);

/* Replaces gmm/grouped_matmul/op_host/op_api/aclnn_grouped_matmul_v5.h:68-69. */
ACL_FUNC_VISIBILITY aclnnStatus aclnnGroupedMatmulV5(void *workspace, uint64_t workspaceSize, aclOpExecutor *executor,
                                                     aclrtStream stream);

#ifdef __cplusplus
}
#endif
#endif /* B200_ACLNN_GROUPED_MATMUL_V5_H */
