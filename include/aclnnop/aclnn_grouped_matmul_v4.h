/*
 * aclnnGroupedMatmulV4: grouped GEMM over experts, here in its W8A8 per-token-quantised mode on NVIDIA B200.
 *
 * Drop-in for the reference's entry points declared at
 *   gmm/grouped_matmul/op_host/op_api/aclnn_grouped_matmul_v4.h:66-86
 * (two-phase call: GetWorkspaceSize builds an executor on the host, the second call enqueues the work on a stream).
 *
 * Supported on this path (anything else returns ACLNN_ERR_PARAM_INVALID with a message):
 *   x               list of 1 tensor, int8 [M, K]
 *   weight          list of 1 tensor, int8 [E, K, N]; a transposed view (strides (N*K, 1, K)) is accepted; with format
 *                   ACL_FORMAT_FRACTAL_NZ the storage is [E, N/32, K/16, 16, 32] (view of 3 or 5 dimensions, K % 16 == 0,
 *                   N % 32 == 0) and is read by the tensor cores as it lies
 *   biasOptional    null, or list of 1 tensor int32 [E, N] (added to the accumulator) or bf16 [E, N] (added in fp32)
 *   scaleOptional   list of 1 tensor [E, N], bf16 or fp32 (per-channel weight scale); null only for an int32 result
 *   perTokenScaleOptional  list of 1 tensor fp32 [M]
 *   groupListOptional      int64 [<=E] device tensor; groupListType 0 = running total, 1 = per-group count
 *   splitItem 2 or 3, groupType 0, actType NONE / RELU / GELU_TANH / FAST_GELU / SILU (GELU_ERR_FUNC is rejected, as in
 *                   the reference); an int32 result ignores the activation
 *   out             list of 1 tensor, bf16 [M, N] (y = bf16(act((acc * scale[n]) * perTokenScale[m] [+ bias]))),
 *                   float16 [M, N] (same arithmetic; scale must then be fp32) or int32 [M, N] (raw accumulators, no scales)
 *   offset / antiquant* / activation* / dynQuant*  must be null.
 * Rows of `out` not covered by group_list are left untouched.
 */
#ifndef B200_ACLNN_GROUPED_MATMUL_V4_H
#define B200_ACLNN_GROUPED_MATMUL_V4_H
#include "aclnn/aclnn_base.h"

#ifdef __cplusplus
extern "C" {
#endif

typedef enum {
    GMM_ACT_TYPE_NONE = 0L,
    GMM_ACT_TYPE_RELU = 1L,
    GMM_ACT_TYPE_GELU_TANH = 2L,
    GMM_ACT_TYPE_GELU_ERR_FUNC = 3L,
    GMM_ACT_TYPE_FAST_GELU = 4L,
    GMM_ACT_TYPE_SILU = 5L,
} GMMActType;

/* Replaces gmm/grouped_matmul/op_host/op_api/aclnn_grouped_matmul_v4.h:66-80
 * (implementation in the reference: aclnn_grouped_matmul.cpp:1994-2029).  Host only; never reads group_list. */
ACL_FUNC_VISIBILITY aclnnStatus aclnnGroupedMatmulV4GetWorkspaceSize(
    const aclTensorList *x, const aclTensorList *weight, const aclTensorList *biasOptional,
    const aclTensorList *scaleOptional, const aclTensorList *offsetOptional,
    const aclTensorList *antiquantScaleOptional, const aclTensorList *antiquantOffsetOptional,
    const aclTensorList *perTokenScaleOptional, const aclTensor *groupListOptional,
    const aclTensorList *activationInputOptional, const aclTensorList *activationQuantScaleOptional,
    const aclTensorList *activationQuantOffsetOptional, int64_t splitItem, int64_t groupType, int64_t groupListType,
    int64_t actType, aclTensorList *out, aclTensorList *activationFeatureOutOptional,
    aclTensorList *dynQuantScaleOutOptional, uint64_t *workspaceSize, aclOpExecutor **executor);

/* Replaces gmm/grouped_matmul/op_host/op_api/aclnn_grouped_matmul_v4.h:82-83 (aclnn_grouped_matmul.cpp:2149-2155).
 * Enqueues on `stream` (a cudaStream_t) and returns; consumes the executor. */
ACL_FUNC_VISIBILITY aclnnStatus aclnnGroupedMatmulV4(void *workspace, uint64_t workspaceSize, aclOpExecutor *executor,
                                                     aclrtStream stream);

#ifdef __cplusplus
}
#endif
#endif /* B200_ACLNN_GROUPED_MATMUL_V4_H */
