/*
 * aclnnMoeInitRoutingV3: MoE routing - the token rows grouped by expert, optionally quantised per row to int8, the row map
 * and the per-expert counts - on NVIDIA B200.  It produces what the grouped GEMM operators of this library consume:
 * expandedXOut (int8) -> x, expandedScaleOut -> per-token scale, expertTokensCountOrCumsumOut -> group list (count form).
 *
 * Drop-in for the reference's entry points declared at
 *   moe/moe_init_routing_v3/op_host/op_api/aclnn_moe_init_routing_v3.h:24-47
 * (checks: aclnn_moe_init_routing_v3.cpp:52-207; kernels: moe/moe_init_routing_v3/op_kernel/).
 *
 *   x [n, h] float32 / float16 / bfloat16 (int8 only with quantMode -1);  expertIdx int32 [n, k];
 *   pair j = token * k + slot.  The pairs whose expert lies in activeExpertRange = [start, end) are ordered by expert id,
 *   pairs of one expert in ascending j (a stable sort); availableIdxNum of them exist.  For output row i < availableIdxNum:
 *     quantMode -1: expandedXOut[i, :] = x[j / k, :];  expandedScaleOut[i] = scaleOptional[j / k] if scaleOptional ([n]) is given
 *     quantMode  1: v = float(x[j / k, :]) (* scaleOptional[expert - start, :] if given, [end - start, h]);
 *                   expandedScaleOut[i] = max|v| / 127;  expandedXOut[i, :] = int8(round_half_away(half_towards_zero(v / scale)))
 *                   (an all-zero row gives scale 0 and zeros)
 *   rowIdxType 1: expandedRowIdxOut[i] = j (rows beyond availableIdxNum are not written);
 *   rowIdxType 0: expandedRowIdxOut[j] = i, -1 for pairs outside the active range.
 *   expertTokensNumType 1: expertTokensCountOrCumsumOut [end - start] = rows per active expert;
 *   expertTokensNumType 2: [expertNum, 2] = (expert id, rows) of the non-empty active experts, packed, then zero entries up
 *                          to min(end - start + 1, expertNum) entries; later entries are not written.
 * Rows of expandedXOut / expandedScaleOut beyond availableIdxNum are not written.
 * Accepted attribute values, as in the reference: dropPadMode 0, expertTokensNumFlag true, quantMode 1 or -1,
 * activeNum = n * k (or 0), expertCapacity >= 0 (unused), expertNum <= 10240 (5120 for key-value counts),
 * offsetOptional unused.  A violation returns ACLNN_ERR_PARAM_INVALID from the first phase (the reference reports
 * some of them from its tiling step).  Without quantisation expandedXOut must have x's dtype: the example in the
 * reference's documentation (docs/aclnnMoeInitRoutingV3.md:521-586) declares an int8 expandedXOut of 24 bytes for float32
 * rows with quantMode -1, which cannot hold them; that combination is refused here instead of writing past the buffer.
 */
#ifndef B200_ACLNN_MOE_INIT_ROUTING_V3_H
#define B200_ACLNN_MOE_INIT_ROUTING_V3_H
#include <stdbool.h>

#include "aclnn/aclnn_base.h"

#ifdef __cplusplus
extern "C" {
#endif

/* Replaces moe/moe_init_routing_v3/op_host/op_api/aclnn_moe_init_routing_v3.h:24-42. */
ACL_FUNC_VISIBILITY aclnnStatus aclnnMoeInitRoutingV3GetWorkspaceSize(
    const aclTensor *x, const aclTensor *expertIdx, const aclTensor *scaleOptional, const aclTensor *offsetOptional,
    int64_t activeNum, int64_t expertCapacity, int64_t expertNum, int64_t dropPadMode, int64_t expertTokensNumType,
    bool expertTokensNumFlag, int64_t quantMode, const aclIntArray *activeExpertRangeOptional, int64_t rowIdxType,
    const aclTensor *expandedXOut, const aclTensor *expandedRowIdxOut, const aclTensor *expertTokensCountOrCumsumOut,
    const aclTensor *expandedScaleOut, uint64_t *workspaceSize, aclOpExecutor **executor);

/* Replaces moe/moe_init_routing_v3/op_host/op_api/aclnn_moe_init_routing_v3.h:45-46. */
ACL_FUNC_VISIBILITY aclnnStatus aclnnMoeInitRoutingV3(void *workspace, uint64_t workspaceSize, aclOpExecutor *executor,
                                                      aclrtStream stream);

#ifdef __cplusplus
}
#endif
#endif /* B200_ACLNN_MOE_INIT_ROUTING_V3_H */
