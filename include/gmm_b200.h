/*
 * Entry points of libgmm_b200.so that have no counterpart in the reference's headers: a status read-back for the
 * asynchronous second-phase calls, and flat (handle-free) launchers for bindings that do not want to build
 * aclTensor objects.  Plain C ABI: pointers, sizes and a CUDA stream passed as void*.
 */
#ifndef B200_GMM_B200_H
#define B200_GMM_B200_H
#include "aclnn/aclnn_base.h"

#ifdef __cplusplus
extern "C" {
#endif

/* Library version, major*10000 + minor*100 + patch. */
ACL_FUNC_VISIBILITY int32_t gmmB200Version(void);

/* The second-phase calls only enqueue work, so a device-side problem (a bounded wait that ran out) cannot be
 * returned by them.  This call waits for `stream`, copies the 4-word status record that the kernels keep at the
 * start of `workspace` and returns ACLNN_SUCCESS when it is clean, ACLNN_ERR_RUNTIME_ERROR otherwise.
 * record[0] = code (0 clean, 1 wait timed out, 2 bad scatter index), record[1] = CTA, record[2] = waiting role, record[3] = detail.
 * `record` may be null.  Plays the role of the reference's aclrtSynchronizeStream + error query after
 * aclnnGroupedMatmulV4 (gmm/grouped_matmul/examples/test_aclnn_grouped_matmul.cpp:180-196). */
ACL_FUNC_VISIBILITY aclnnStatus gmmB200CheckStatus(const void *workspace, uint64_t workspaceSize, aclrtStream stream,
                                                  int32_t record[4]);

/* Per-call launch options.  They belong to one executor (gmmB200SetExecutorOptions, between the two phases of an aclnn
 * call) or to one flat call (the trailing `options` argument, may be null), never to the process, so threads that launch on
 * different streams do not see each other's settings.  No counterpart in the reference, where the AI-core count comes from
 * the platform (gmm/grouped_matmul/op_host/op_tiling/grouped_matmul_tiling.cpp:908-918) and phases are traced with
 * L2_DFX_PHASE_1/2 (gmm/grouped_matmul/op_host/op_api/aclnn_grouped_matmul.cpp:2005, 2151).
 *   structSize       sizeof(gmmB200LaunchOptions) as the caller compiled it (fields beyond it read as 0).
 *   maxCtas          the GEMM kernels are persistent and normally launch one CTA per SM; a caller that overlaps them with
 *                    other work on the same GPU (the exchange kernels of an expert-parallel layer) can cap the CTAs. 0 = no cap.
 *   startEvent /     cudaEvent_t handles created by the caller: recorded right before and right after the tensor-core GEMM
 *   stopEvent        kernel(s) of the call on the launch stream, so a benchmark can time them alone inside a multi-kernel
 *                    operator.  Null = off.
 *   waitLimitCycles  bound of every device-side wait (SM clock cycles) before a CTA gives up, records a status and returns;
 *                    0 = the default of 2^31 cycles (about a second).
 *   testSkipKBlocks  test only: the copy-issuing warp leaves this many K blocks out of its last tile, so that the bounded wait
 *                    of the warp that consumes them runs out and the abort path (status record, clean exit) can be exercised
 *                    without touching memory the call does not own.  Results are then undefined.  0 = off. */
typedef struct gmmB200LaunchOptions {
    uint32_t structSize;
    int32_t maxCtas;
    void *startEvent;
    void *stopEvent;
    int64_t waitLimitCycles;
    int32_t testSkipKBlocks;
    int32_t reserved;
} gmmB200LaunchOptions;
ACL_FUNC_VISIBILITY aclnnStatus gmmB200SetExecutorOptions(aclOpExecutor *executor, const gmmB200LaunchOptions *options);

/* Flat form of aclnnGroupedMatmulV4 for the W8A8 path (same arithmetic, same validation of sizes).
 * scaleDtype / biasDtype / yDtype use aclDataType codes; bias may be null (biasDtype ignored);
 * weightTransposed is the weight's layout: 0 = [E, K, N], 1 = [E, N, K], 2 = FRACTAL_NZ [E, N/32, K/16, 16, 32]
 * (K % 16 == 0, N % 32 == 0).  actType is a GMMActType; yDtype bf16, float16 (scale then fp32) or int32.
 * outRowIndex (optional, int64 [m] on the device, may be null): result row r is written to row outRowIndex[r] of y
 * instead of row r, which lets a caller fold the un-permute that follows the down projection of an MoE layer into the
 * GEMM (the row scatter of the reference's GroupedMatmulFinalizeRouting, gmm/grouped_matmul_finalize_routing/README.md:11-14,
 * without its weighting).  The indices must be a permutation onto rows of y.  outRows = the rows of y (and of every
 * peer buffer): a row whose index is negative, at or beyond outRows, or names a GPU that is no peer is not stored; the
 * first such row is reported by gmmB200CheckStatus (code 2, record[3] = the source row).  outRows 0 = no upper bound.
 * outPeers / numPeers (optional, bf16 result only): with numPeers in [1, 8], outRowIndex[r] = (gpu << 40) | row and the
 * row is stored into outPeers[gpu] (a [rows, n] bf16 buffer that may live on another GPU of the node, see
 * gmmB200PeerImport) instead of y: the return all-to-all of an expert-parallel layer folded into the GEMM epilogue,
 * the role of the reference's GroupedMatMulAlltoAllv (mc2/grouped_mat_mul_allto_allv/README.md:12-24).  The caller
 * orders the GPUs (a barrier after the kernels) before anyone reads those buffers. */
ACL_FUNC_VISIBILITY aclnnStatus gmmB200GroupedMatmulW8A8WorkspaceSize(int64_t m, int64_t k, int64_t n, int64_t e,
                                                                     int32_t yDtype, uint64_t *workspaceSize);
ACL_FUNC_VISIBILITY aclnnStatus gmmB200GroupedMatmulW8A8(const void *x, const void *weight, const void *scale,
                                                        int32_t scaleDtype, const void *perTokenScale, const void *bias,
                                                        int32_t biasDtype, const void *groupList, int64_t groupListLen,
                                                        int32_t groupListType, int64_t m, int64_t k, int64_t n, int64_t e,
                                                        int32_t weightTransposed, int32_t actType, const void *outRowIndex,
                                                        void *const *outPeers, int32_t numPeers, int64_t outRows, void *y, int32_t yDtype,
                                                        void *workspace, uint64_t workspaceSize, aclrtStream stream,
                                                        const gmmB200LaunchOptions *options);

/* Buffers that other GPUs of the node can write into (CUDA IPC).  PeerAlloc/PeerFree own device memory of the calling
 * process; PeerExport fills a 64-byte handle that another process passes to PeerImport to obtain a device pointer to the
 * same memory (peer access is enabled on first use); PeerRelease drops an imported mapping.  Set-up calls, not for the
 * hot path.  They stand in for the HCCL window memory the reference's mc2 operators obtain from
 * AscendC::GetHcclContext (mc2/moe_distribute_dispatch_v2/op_kernel/moe_distribute_dispatch_v2.h:317-319). */
ACL_FUNC_VISIBILITY aclnnStatus gmmB200PeerAlloc(uint64_t bytes, void **devPtr);
ACL_FUNC_VISIBILITY aclnnStatus gmmB200PeerFree(void *devPtr);
ACL_FUNC_VISIBILITY aclnnStatus gmmB200PeerExport(const void *devPtr, void *handle64);
ACL_FUNC_VISIBILITY aclnnStatus gmmB200PeerImport(const void *handle64, void **devPtr);
ACL_FUNC_VISIBILITY aclnnStatus gmmB200PeerRelease(void *devPtr);

/* Expert-parallel dispatch of already quantised token rows: send row i is token srcToken[i] of x (int8 [tokens, hidden],
 * scale xScale[tokens]) and is stored as row (dest[i] & (2^40-1)) of GPU (dest[i] >> 40)'s activation buffer peerX[gpu]
 * (int8 [capacity, hidden]) with its scale in peerScale[gpu]; dest[i] < 0 skips the row.  One pass of stores over NVLink
 * replaces gather + all-to-all + re-ordering (reference: MoeDistributeDispatchV2 with quantMode 2 followed by
 * MoeReRouting, mc2/moe_distribute_dispatch_v2/README.md:167-186, moe/moe_re_routing/README.md:12-26).  Rows whose
 * destination is beyond `capacity` are dropped and counted in *overflowCounter (int32 on the device, cleared by the
 * caller).  firstRow (optional, int64 on the device): the send row the kernel starts with, wrapping around; giving every
 * rank the first row of a different destination keeps the ranks from all storing into one GPU at a time.
 * maxBlocks (0 = no cap): most blocks of 256 threads the kernel launches; 8 fit an SM, so 8 * s keeps it on about s SMs
 * when it runs beside a GEMM whose CTAs were capped accordingly (gmmB200LaunchOptions.maxCtas).
 * The caller orders the GPUs (a barrier) before the receivers read. */
ACL_FUNC_VISIBILITY aclnnStatus gmmB200EpDispatch(const void *x, const void *xScale, const void *srcToken, const void *dest,
                                                 int64_t rows, int64_t hidden, int64_t capacity, void *const *peerX,
                                                 void *const *peerScale, int32_t numPeers, void *overflowCounter,
                                                 const void *firstRow, int32_t maxBlocks, aclrtStream stream);

/* Routing for the expert-parallel dispatch, in two launches around the all-gather of the per-expert counts, without any
 * read on the host.  topk: int64 [nPairs] global expert of every (token, slot) pair (pair i belongs to token i / topK).
 *   gmmB200EpCount: totals[nExperts] (int64) = pairs per global expert, blockHist [ceil(nPairs/1024)][nExperts] (int32)
 *                   = the same per block of 1024 pairs.
 *   gmmB200EpRoute: allCounts int64 [world][world][expertsPerRank] = every rank's totals (all-gathered).  Writes the send
 *                   order grouped by global expert: srcToken[pos] (= tokenBase + pair / topK), order[pos] (= pair),
 *                   sendDest[pos] = (gpu << 40) | row in that GPU's expert-major activation buffer; retDest[capacity]:
 *                   for every activation row of this rank (gpu << 40) | (resultBase + position in that GPU's send order),
 *                   -1 beyond the rows received; groupList[expertsPerRank] running totals of this rank's experts;
 *                   firstRow[1] for gmmB200EpDispatch.
 * They play the part of the index outputs of the reference's MoeInitRouting / MoeDistributeDispatch
 * (moe/moe_init_routing_v3/README.md:21-62, mc2/moe_distribute_dispatch_v2/README.md:216-250) and of MoeReRouting's
 * offsets (moe/moe_re_routing/README.md:12-26). */
ACL_FUNC_VISIBILITY aclnnStatus gmmB200EpCount(const void *topk, int64_t nPairs, int32_t nExperts, void *blockHist, void *totals,
                                              aclrtStream stream);
ACL_FUNC_VISIBILITY aclnnStatus gmmB200EpRoute(const void *topk, const void *blockHist, const void *allCounts, int64_t nPairs,
                                              int32_t topK, int32_t world, int32_t expertsPerRank, int32_t rank, int64_t capacity,
                                              int64_t tokenBase, int64_t resultBase, void *srcToken, void *order, void *sendDest,
                                              void *retDest, void *groupList, void *firstRow, aclrtStream stream);

/* The consumer of the expert-parallel path: every token's result rows, which the down GEMM's epilogue stored into this
 * GPU's result buffer in send order, weighted and summed into one row per token - the last step of the reference's
 * MoeDistributeCombineV2, xOut = Sum(expertScales * ataOut) (mc2/moe_distribute_combine_v2/README.md:12-17; fp32 Muls and
 * Add per slot in slot order, CAST_RINT to bf16 at the end: op_kernel/moe_distribute_combine_v2.h:1130-1134, 1195-1258).
 *   gmmB200EpInverseMap: pairRow[order[i]] = resultBase + i for i < min(*rowsInUse, maxRows).  order (int64, from
 *                   gmmB200EpRoute) and rowsInUse (int64[1]) are on the device; pairRow is int32 [nPairs], which the caller
 *                   has filled with -1 (pairs without a row - dropped or outside this piece - stay -1); entries of order
 *                   outside [0, nPairs) are skipped and counted in *badCounter (int32 on the device).
 *   gmmB200EpCombine: out[t] = bf16(sum over s < topK with pairRow[t*topK+s] >= 0 of float(y[pairRow[t*topK+s]]) * weights[t*topK+s]).
 *                   y bf16 [yRows, hidden], weights fp32 [tokens, topK], out bf16 [tokens, hidden]; hidden a multiple of 8.
 * The caller orders the GPUs (a barrier) between the down GEMM and the combine. */
ACL_FUNC_VISIBILITY aclnnStatus gmmB200EpInverseMap(const void *order, const void *rowsInUse, int64_t maxRows, int64_t resultBase,
                                                   int64_t nPairs, void *pairRow, void *badCounter, aclrtStream stream);
ACL_FUNC_VISIBILITY aclnnStatus gmmB200EpCombine(const void *y, const void *pairRow, const void *weights, void *out, int64_t tokens,
                                                int32_t topK, int64_t hidden, int64_t yRows, aclrtStream stream);

/* Flat form of aclnnGroupedMatmulFinalizeRoutingWeightNz (include/aclnnop/aclnn_grouped_matmul_finalize_routing_weight_nz.h),
 * with two freedoms the aclnn form lacks: weightLayout 0 ([e, k, n], the faster layout on B200) besides 2 (FRACTAL_NZ), and
 * groupListType 0 (running totals) besides 1.  sharedInput and logit are given together (rows are added to y, which the
 * call first fills with the weighted shared rows and zeros) or both null (rows are stored, y is not initialised).
 * y is fp32 [yRows, n]; rowIndexDtype is ACL_INT64 or ACL_INT32; the workspace needs 256 bytes. */
ACL_FUNC_VISIBILITY aclnnStatus gmmB200GroupedMatmulFinalizeRouting(
    const void *x, const void *weight, int32_t weightLayout, const void *scale, int32_t scaleDtype, const void *bias,
    const void *perTokenScale, const void *groupList, int64_t groupListLen, int32_t groupListType, const void *sharedInput,
    int64_t sharedRows, int64_t sharedOffset, float sharedWeight, const void *logit, const void *rowIndex, int32_t rowIndexDtype,
    int64_t m, int64_t k, int64_t n, int64_t e, void *y, int64_t yRows, void *workspace, uint64_t workspaceSize,
    aclrtStream stream, const gmmB200LaunchOptions *options);

/* Flat form of aclnnGroupedMatmulSwigluQuant.  weightLayout: 0 = [e, k, n], 2 = FRACTAL_NZ [e, n/32, k/16, 16, 32]. */
ACL_FUNC_VISIBILITY aclnnStatus gmmB200GroupedMatmulSwigluQuantWorkspaceSize(int64_t m, int64_t k, int64_t n, int64_t e,
                                                                            uint64_t *workspaceSize);
ACL_FUNC_VISIBILITY aclnnStatus gmmB200GroupedMatmulSwigluQuant(const void *x, const void *weight, const void *weightScale,
                                                               int32_t weightScaleDtype, const void *xScale,
                                                               const void *groupList, int64_t groupListLen, int64_t m,
                                                               int64_t k, int64_t n, int64_t e, int32_t weightLayout,
                                                               void *output, void *outputScale, void *workspace,
                                                               uint64_t workspaceSize, aclrtStream stream,
                                                               const gmmB200LaunchOptions *options);

/* grouped_matmul_swiglu_quant without any device allocation.  This entry point has no counterpart in the reference.
 *
 * For callers that cannot allocate at the point of the call - a server whose memory pool is frozen after warm-up,
 * a plugin living inside another runtime's arena, a loop that cannot afford the device-wide synchronisation that
 * cudaMalloc / cudaFree imply.  The operator's scratch memory is a fixed array of
 * GMM_B200_NO_ALLOC_SCRATCH_BYTES inside the library image, which every GPU that loads the library keeps until the
 * process ends.  Same arguments and results as gmmB200GroupedMatmulSwigluQuant minus the workspace.
 *   - Limit: the scratch needed is 256 + 4*m + 8*(m/128 + 2*groupListLen + 2) + 4*m*(n/2) bytes, each part rounded up to 256; a larger problem is rejected
 *     with ACLNN_ERR_PARAM_INVALID and a message (e.g. at n = 4096, m = 4096 rows fit and m = 8192 do not).
 *   - The first call on each device looks up the array's device address (once, with that device current); make that
 *     first call before any stream capture begins.
 *   - All calls share the one array and it keeps the previous call's contents; the part that must start at zero is
 *     cleared on `stream` by every call.  Two calls that can overlap on the GPU (different streams, no ordering
 *     between them) race on it: order them, or use the workspace variant for one of them.
 * The first call on a device is a warm-up: loading the library's code and the array onto that device, and the first launch
 * of each kernel variant, may allocate inside the CUDA runtime.  After that neither this call nor anything it calls
 * allocates or frees device memory.
 * gmmB200NoAllocCheckStatus: the kernels' status record sits at the start of the built-in array, out of the caller's reach;
 * this call waits for `stream` and reports it exactly as gmmB200CheckStatus does for a caller-provided workspace (a bounded
 * device-side wait that ran out gives ACLNN_ERR_RUNTIME_ERROR and fills `record`, which may be null). */
#define GMM_B200_NO_ALLOC_SCRATCH_BYTES (32u * 1024u * 1024u + 64u * 1024u)
ACL_FUNC_VISIBILITY uint64_t gmmB200NoAllocScratchBytes(void);
ACL_FUNC_VISIBILITY aclnnStatus gmmB200GroupedMatmulSwigluQuantNoAlloc(const void *x, const void *weight, const void *weightScale,
                                                                      int32_t weightScaleDtype, const void *xScale,
                                                                      const void *groupList, int64_t groupListLen, int64_t m,
                                                                      int64_t k, int64_t n, int64_t e, void *output,
                                                                      void *outputScale, aclrtStream stream);
ACL_FUNC_VISIBILITY aclnnStatus gmmB200NoAllocCheckStatus(aclrtStream stream, int32_t record[4]);

#ifdef __cplusplus
}
#endif
#endif /* B200_GMM_B200_H */
