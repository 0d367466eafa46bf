/*
 * aclnnGroupedMatmulFinalizeRoutingWeightNz (and V2): the down-projection grouped GEMM of an MoE layer fused with the
 * combine that follows it (MoeFinalizeRouting), W8A8, on NVIDIA B200.
 *
 * Drop-in for the reference's entry points declared at
 *   gmm/grouped_matmul_finalize_routing/op_host/op_api/aclnn_grouped_matmul_finalize_routing_weight_nz.h:48-64
 *   gmm/grouped_matmul_finalize_routing/op_host/op_api/aclnn_grouped_matmul_finalize_routing_weight_nz_v2.h:55-71
 * (implementation: aclnn_grouped_matmul_finalize_routing.cpp:949-1083; kernel: op_kernel/grouped_matmul_finalize_routing.h).
 *
 *   x1 int8 [m, k];  x2 int8, format ACL_FORMAT_FRACTAL_NZ, view [e, k, n] over storage [e, n/32, k/16, 16, 32] (or viewed
 *   with those 5 dimensions);  scale [e, n] fp32 or bf16;  bias null or bf16 [e, n];  pertokenScaleOptional null or fp32 [m];
 *   groupList int64 [e], per-group counts (groupListType must be 1);  rowIndex int64 or int32 [m];
 *   out fp32 [batch, n], batch <= m.   k % 16 == 0, n % 32 == 0, n >= 256; dtype 0; no transposes.
 * Scene 1 - sharedInput bf16 [sharedRows, n] and logit fp32 [m] both given:
 *   out[r, :]  = float(sharedInput[r - sharedInputOffset, :]) * sharedInputWeight   for r in [sharedInputOffset, +sharedRows), else 0
 *   out[rowIndex[i], :] += ((acc[i, :] * scale[g, :]) * (pertokenScale[i] * logit[i])) + logit[i] * float(bias[g, :])
 *   for every row i covered by groupList; the additions are fp32 atomics, so their order (and the last bits) vary
 *   from run to run, as in the reference (SetAtomicAdd, grouped_matmul_finalize_routing.h:343-366).
 * Scene 2 - sharedInput and logit both null: out[rowIndex[i], :] = (acc * scale) * pertokenScale [+ bias], plain stores,
 *   rows not named by rowIndex keep their contents.
 * Any other combination of null arguments returns ACLNN_ERR_PARAM_NULLPTR.  rowIndex values outside [0, batch) are
 * skipped (the reference does not check them).  The int4-weight (W4A8) family of this operator - the plain
 * aclnnGroupedMatmulFinalizeRouting / V2 / V3 entry points, int64 packed scales, offset - is not part of this build.
 * V2 adds offsetOptional (must be null here), two unused antiquant arguments and tuningConfigOptional (validated:
 * 0 <= value <= m; unused, the tile schedule is built on the device).
 */
#ifndef B200_ACLNN_GROUPED_MATMUL_FINALIZE_ROUTING_WEIGHT_NZ_H
#define B200_ACLNN_GROUPED_MATMUL_FINALIZE_ROUTING_WEIGHT_NZ_H
#include <stdbool.h>

#include "aclnn/aclnn_base.h"

#ifdef __cplusplus
extern "C" {
#endif

/* Replaces .../aclnn_grouped_matmul_finalize_routing_weight_nz.h:48-53. */
ACL_FUNC_VISIBILITY aclnnStatus aclnnGroupedMatmulFinalizeRoutingWeightNzGetWorkspaceSize(
    const aclTensor *x1, const aclTensor *x2, const aclTensor *scale, const aclTensor *bias,
    const aclTensor *pertokenScaleOptional, const aclTensor *groupList, const aclTensor *sharedInput, const aclTensor *logit,
    const aclTensor *rowIndex, int64_t dtype, float sharedInputWeight, int64_t sharedInputOffset, bool transposeX1,
    bool transposeX2, int64_t groupListType, aclTensor *out, uint64_t *workspaceSize, aclOpExecutor **executor);

/* Replaces .../aclnn_grouped_matmul_finalize_routing_weight_nz.h:63-64. */
ACL_FUNC_VISIBILITY aclnnStatus aclnnGroupedMatmulFinalizeRoutingWeightNz(void *workspace, uint64_t workspaceSize,
                                                                          aclOpExecutor *executor, aclrtStream stream);

/* Replaces .../aclnn_grouped_matmul_finalize_routing_weight_nz_v2.h:55-61. */
ACL_FUNC_VISIBILITY aclnnStatus aclnnGroupedMatmulFinalizeRoutingWeightNzV2GetWorkspaceSize(
    const aclTensor *x1, aclTensor *x2, const aclTensor *scale, const aclTensor *bias, const aclTensor *offsetOptional,
    const aclTensor *antiquantScaleOptional, const aclTensor *antiquantOffsetOptional, const aclTensor *pertokenScaleOptional,
    const aclTensor *groupList, const aclTensor *sharedInput, const aclTensor *logit, const aclTensor *rowIndex, int64_t dtype,
    float sharedInputWeight, int64_t sharedInputOffset, bool transposeX1, bool transposeX2, int64_t groupListType,
    const aclIntArray *tuningConfigOptional, aclTensor *out, uint64_t *workspaceSize, aclOpExecutor **executor);

/* Replaces .../aclnn_grouped_matmul_finalize_routing_weight_nz_v2.h:70-71. */
ACL_FUNC_VISIBILITY aclnnStatus aclnnGroupedMatmulFinalizeRoutingWeightNzV2(void *workspace, uint64_t workspaceSize,
                                                                            aclOpExecutor *executor, aclrtStream stream);

#ifdef __cplusplus
}
#endif
#endif /* B200_ACLNN_GROUPED_MATMUL_FINALIZE_ROUTING_WEIGHT_NZ_H */
