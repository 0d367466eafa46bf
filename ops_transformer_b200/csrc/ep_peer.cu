// Peer-memory plumbing for the expert-parallel path: buffers that the other GPUs of the node can write into
// (CUDA IPC), and the dispatch kernel that gathers a rank's token rows and stores each one straight into the row
// of the owning GPU's expert-major activation buffer - gather, all-to-all and re-ordering in one pass of stores over
// NVLink.  It takes the place of the reference's MoeDistributeDispatch window writes
// (mc2/moe_distribute_dispatch_v2/docs/MoeDistributeDispatch-Combine算子设计介绍.md:40-66) followed by MoeReRouting
// (moe/moe_re_routing/README.md:12-26) for rows that are already quantised.
// Only plain stores to peer memory are used; no bulk-tensor copies touch another GPU's memory.
#include <cuda_bf16.h>

#include <algorithm>
#include <cstring>

#include "acl_shim.h"
#include "gmm_b200.h"

namespace {

struct PeerPtrs {
    int8_t *x[8];
    float *s[8];
};

constexpr long long kRowMask = (1ll << 40) - 1;

// One warp per row.  dest[i] = (gpu << 40) | row, or negative to skip the row.  A destination row at or beyond
// `capacity`, or a gpu field that names no peer, is not written; the kernel counts such rows in *overflow instead.
__global__ void __launch_bounds__(256) ep_dispatch_kernel(const int8_t *__restrict__ x, const float *__restrict__ xs,
                                                           const long long *__restrict__ src_token,
                                                           const long long *__restrict__ dest, long long rows, int hidden,
                                                           long long capacity, PeerPtrs pp, int num_peers, int *overflow,
                                                           const long long *__restrict__ first_row)
{
    const int lane = threadIdx.x & 31;
    const long long warps = (long long)gridDim.x * (blockDim.x >> 5);
    const int vecs = hidden >> 4;
    // Rows are walked starting at *first_row (wrapping around): when every rank starts with a different destination GPU,
    // the ranks do not all store into the same GPU at the same time.
    long long rot = first_row ? *first_row : 0;
    rot = rot > 0 && rot < rows ? rot : 0;
    for (long long it = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); it < rows; it += warps) {
        const long long row = it + rot < rows ? it + rot : it + rot - rows;
        const long long d = dest[row];
        if (d < 0) continue;
        const long long gpu_field = d >> 40;
        const int gpu = (int)gpu_field;
        const long long drow = d & kRowMask;
        if (gpu_field >= num_peers || drow >= capacity) {
            if (lane == 0) atomicAdd(overflow, 1);
            continue;
        }
        const long long tok = src_token[row];
        const uint4 *src = reinterpret_cast<const uint4 *>(x + tok * hidden);
        uint4 *dst = reinterpret_cast<uint4 *>(pp.x[gpu] + drow * hidden);
        int i = lane;
        for (; i + 96 < vecs; i += 128) {  // four 16-byte pieces per lane in flight
            const uint4 a = src[i], b = src[i + 32], c = src[i + 64], e = src[i + 96];
            dst[i] = a; dst[i + 32] = b; dst[i + 64] = c; dst[i + 96] = e;
        }
        for (; i < vecs; i += 32) dst[i] = src[i];
        if (lane == 0) pp.s[gpu][drow] = xs[tok];
    }
    __threadfence_system();
}


// ---------------------------------------------------------------------------------------------------------
// Routing: the send order of a rank's (token, slot) pairs and the row maps of the peer-memory pipeline, in two
// launches with the count all-gather between them (the host never reads a value).
//   ep_count_kernel : per-block histograms of the destination experts (blocks of kRouteBlock pairs) and the totals
//   ep_route_kernel : from the all-gathered totals all_counts[src][dst][e]:
//       send order  - pairs grouped by global expert (dst-major); inside an expert by block, inside a block in arrival
//                     order of a shared-memory counter (any order inside an expert is valid: rows are independent);
//       src_token[pos], order[pos], send_dest[pos] = (dst << 40) | row in dst's expert-major buffer (MoeReRouting's
//                     DstOffset, moe/moe_re_routing/README.md:12-26);
//       ret_dest[p]   = (src << 40) | position of activation row p in src's send order (where its result goes back);
//       group_list[e] = running totals of this rank's local experts; first_row = first send row for rank+1.
// ---------------------------------------------------------------------------------------------------------

constexpr int kRouteBlock = 1024;   // pairs per block
constexpr int kMaxSegments = 1024;  // world * experts_per_rank, also the most groups a GEMM call accepts

__global__ void __launch_bounds__(256) ep_count_kernel(const long long *__restrict__ topk, int n_pairs, int n_experts,
                                                        int *__restrict__ block_hist, long long *__restrict__ totals)
{
    __shared__ int h[kMaxSegments];
    for (int i = threadIdx.x; i < n_experts; i += blockDim.x) h[i] = 0;
    __syncthreads();
    const int base = blockIdx.x * kRouteBlock;
    for (int i = threadIdx.x; i < kRouteBlock && base + i < n_pairs; i += blockDim.x) {
        const long long e = topk[base + i];
        if (e >= 0 && e < n_experts) atomicAdd(&h[(int)e], 1);
    }
    __syncthreads();
    for (int i = threadIdx.x; i < n_experts; i += blockDim.x) {
        block_hist[(size_t)blockIdx.x * n_experts + i] = h[i];
        if (h[i]) atomicAdd(reinterpret_cast<unsigned long long *>(totals + i), (unsigned long long)h[i]);
    }
}

struct RouteParams {
    const long long *topk;        // [n_pairs] global expert of every (token, slot) pair
    const int *block_hist;        // [n_blocks][world*E]
    const long long *all_counts;  // [world(src)][world(dst)][E]
    int n_pairs, top_k, world, experts, rank, n_blocks, capacity, token_base;
    long long result_base;        // first row of this chunk in the result buffers
    long long *src_token, *order, *send_dest;  // [n_pairs]
    long long *ret_dest;          // [capacity]
    long long *group_list;        // [E]
    long long *first_row;         // [1]
};

// grid = n_blocks (send side) + ceil(capacity / kRouteBlock) (return side)
__global__ void __launch_bounds__(256) ep_route_kernel(const RouteParams p)
{
    __shared__ long long s_a[kMaxSegments];   // send side: first send position of this block's pairs per expert
    __shared__ long long s_b[kMaxSegments];   // send side: destination row of the segment's first pair / return side: ends
    __shared__ long long s_c[kMaxSegments];   // return side: position in the source's send order of the segment's first row
    __shared__ int s_cursor[kMaxSegments];
    const int G = p.world, E = p.experts, S = G * E, tid = threadIdx.x;
    const long long *C = p.all_counts;
    if ((int)blockIdx.x < p.n_blocks) {
        // ---- send side ----
        for (int seg = tid; seg < S; seg += blockDim.x) {
            const int dst = seg / E, e = seg % E;
            long long seg_start = 0;                         // pairs of this rank for segments before (dst, e)
            for (int s2 = 0; s2 < seg; ++s2) seg_start += C[(size_t)p.rank * S + s2];
            long long before_blocks = 0;                     // same segment, earlier blocks
            for (int b = 0; b < (int)blockIdx.x; ++b) before_blocks += p.block_hist[(size_t)b * S + seg];
            long long expert_off = 0;                        // rows of dst's experts before e
            for (int e2 = 0; e2 < e; ++e2)
                for (int s3 = 0; s3 < G; ++s3) expert_off += C[((size_t)s3 * G + dst) * E + e2];
            long long src_off = 0;                           // rows of lower ranks inside the expert
            for (int s3 = 0; s3 < p.rank; ++s3) src_off += C[((size_t)s3 * G + dst) * E + e];
            s_a[seg] = seg_start + before_blocks;
            s_b[seg] = expert_off + src_off + before_blocks;
            s_cursor[seg] = 0;
        }
        __syncthreads();
        const int base = blockIdx.x * kRouteBlock;
        for (int i = tid; i < kRouteBlock && base + i < p.n_pairs; i += blockDim.x) {
            const long long ge = p.topk[base + i];
            if (ge < 0 || ge >= S) continue;
            const int w = atomicAdd(&s_cursor[(int)ge], 1);
            const long long pos = s_a[(int)ge] + w;
            p.src_token[pos] = (long long)p.token_base + (base + i) / p.top_k;
            p.order[pos] = base + i;
            p.send_dest[pos] = ((long long)(ge / E) << 40) | (s_b[(int)ge] + w);
        }
        if (blockIdx.x == 0) {
            if (tid == 0) {
                const int nxt = (p.rank + 1) % G;
                long long fr = 0;
                for (int s2 = 0; s2 < nxt * E; ++s2) fr += C[(size_t)p.rank * S + s2];
                *p.first_row = fr;
            }
            for (int e = tid; e < E; e += blockDim.x) {
                long long run = 0;
                for (int e2 = 0; e2 <= e; ++e2)
                    for (int s3 = 0; s3 < G; ++s3) run += C[((size_t)s3 * G + p.rank) * E + e2];
                p.group_list[e] = run;
            }
        }
    } else {
        // ---- return side: this rank's activation buffer is ordered (e, src) ----
        for (int seg = tid; seg < S; seg += blockDim.x) {
            const int e = seg / G, src = seg % G;
            long long back = 0;                              // start of segment (rank, e) in src's send order
            for (int s2 = 0; s2 < p.rank * E + e; ++s2) back += C[(size_t)src * S + s2];
            s_c[seg] = back;
            s_b[seg] = C[((size_t)src * G + p.rank) * E + e];  // segment length, turned into running ends below
        }
        __syncthreads();
        if (tid == 0) {
            long long run = 0;
            for (int seg = 0; seg < S; ++seg) { run += s_b[seg]; s_b[seg] = run; }
        }
        __syncthreads();
        const long long total = s_b[S - 1];
        const long long pbase = (long long)((int)blockIdx.x - p.n_blocks) * kRouteBlock;
        for (int i = tid; i < kRouteBlock; i += blockDim.x) {
            const long long q = pbase + i;
            if (q >= p.capacity) break;
            long long out = -1;
            if (q < total) {
                int lo = 0, hi = S - 1;                      // first segment whose end is beyond q
                while (lo < hi) {
                    const int mid = (lo + hi) >> 1;
                    if (s_b[mid] > q) hi = mid; else lo = mid + 1;
                }
                const long long seg_begin = lo ? s_b[lo - 1] : 0;
                out = ((long long)(lo % G) << 40) | (p.result_base + s_c[lo] + (q - seg_begin));
            }
            p.ret_dest[q] = out;
        }
    }
}

}  // namespace

// Inverse of the send order: pair_row[order[i]] = result_base + i for the rows in use.
__global__ void __launch_bounds__(256) ep_inverse_map_kernel(const long long *order, const long long *rows_in_use, long long max_rows,
                                                             long long result_base, int n_pairs, int *pair_row, int *bad)
{
    const long long n = min(*rows_in_use, max_rows);
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        const long long pair = order[i];
        if (pair >= 0 && pair < n_pairs) pair_row[pair] = (int)(result_base + i);
        else atomicAdd(bad, 1);   // a send position that names no pair: skipped and counted
    }
}

// One CTA per token: out[token] = bf16( sum over the token's slots, in slot order, of float(y[row]) * weight ), every product
// and every sum rounded on its own (Muls then Add on fp32, CAST_RINT at the end:
// mc2/moe_distribute_combine_v2/op_kernel/moe_distribute_combine_v2.h:1130-1134, 1195, 1258).  Slots without a row are left out.
__global__ void __launch_bounds__(256) ep_combine_kernel(const uint4 *y, const int *pair_row, const float *weights, uint4 *out,
                                                         int top_k, int h8, long long y_rows)
{
    const long long token = blockIdx.x;
    for (int c = threadIdx.x; c < h8; c += blockDim.x) {
        float acc[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] = 0.0f;
        for (int s = 0; s < top_k; ++s) {
            const int row = pair_row[token * top_k + s];
            if (row < 0 || row >= y_rows) continue;
            const float w = weights[token * top_k + s];
            const uint4 v = y[(size_t)row * h8 + c];   // written by other GPUs before the barrier: a plain (coherent) load
            const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                acc[2 * j] = __fadd_rn(acc[2 * j], __fmul_rn(__uint_as_float(u[j] << 16), w));
                acc[2 * j + 1] = __fadd_rn(acc[2 * j + 1], __fmul_rn(__uint_as_float(u[j] & 0xffff0000u), w));
            }
        }
        uint32_t o[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const __nv_bfloat162 b = __floats2bfloat162_rn(acc[2 * j], acc[2 * j + 1]);
            o[j] = *reinterpret_cast<const uint32_t *>(&b);
        }
        out[(size_t)token * h8 + c] = make_uint4(o[0], o[1], o[2], o[3]);
    }
}

extern "C" {

aclnnStatus gmmB200PeerAlloc(uint64_t bytes, void **devPtr)
{
    gmm::clear_error();
    if (!devPtr) return gmm::fail(ACLNN_ERR_PARAM_NULLPTR, "devPtr must not be nullptr.");
    cudaError_t e = cudaMalloc(devPtr, bytes);
    if (e != cudaSuccess) return gmm::fail(ACLNN_ERR_RUNTIME_ERROR, "cudaMalloc of %llu bytes failed: %s", (unsigned long long)bytes, cudaGetErrorString(e));
    return ACLNN_SUCCESS;
}

aclnnStatus gmmB200PeerFree(void *devPtr)
{
    gmm::clear_error();
    cudaError_t e = cudaFree(devPtr);
    if (e != cudaSuccess) return gmm::fail(ACLNN_ERR_RUNTIME_ERROR, "cudaFree failed: %s", cudaGetErrorString(e));
    return ACLNN_SUCCESS;
}

aclnnStatus gmmB200PeerExport(const void *devPtr, void *handle64)
{
    gmm::clear_error();
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "handle size");
    if (!devPtr || !handle64) return gmm::fail(ACLNN_ERR_PARAM_NULLPTR, "devPtr and handle64 must not be nullptr.");
    cudaIpcMemHandle_t h;
    cudaError_t e = cudaIpcGetMemHandle(&h, const_cast<void *>(devPtr));
    if (e != cudaSuccess) return gmm::fail(ACLNN_ERR_RUNTIME_ERROR, "cudaIpcGetMemHandle failed: %s", cudaGetErrorString(e));
    memcpy(handle64, &h, sizeof(h));
    return ACLNN_SUCCESS;
}

aclnnStatus gmmB200PeerImport(const void *handle64, void **devPtr)
{
    gmm::clear_error();
    if (!devPtr || !handle64) return gmm::fail(ACLNN_ERR_PARAM_NULLPTR, "devPtr and handle64 must not be nullptr.");
    cudaIpcMemHandle_t h;
    memcpy(&h, handle64, sizeof(h));
    cudaError_t e = cudaIpcOpenMemHandle(devPtr, h, cudaIpcMemLazyEnablePeerAccess);
    if (e != cudaSuccess) return gmm::fail(ACLNN_ERR_RUNTIME_ERROR, "cudaIpcOpenMemHandle failed: %s", cudaGetErrorString(e));
    return ACLNN_SUCCESS;
}

aclnnStatus gmmB200PeerRelease(void *devPtr)
{
    gmm::clear_error();
    cudaError_t e = cudaIpcCloseMemHandle(devPtr);
    if (e != cudaSuccess) return gmm::fail(ACLNN_ERR_RUNTIME_ERROR, "cudaIpcCloseMemHandle failed: %s", cudaGetErrorString(e));
    return ACLNN_SUCCESS;
}

aclnnStatus gmmB200EpDispatch(const void *x, const void *xScale, const void *srcToken, const void *dest, int64_t rows,
                              int64_t hidden, int64_t capacity, void *const *peerX, void *const *peerScale, int32_t numPeers,
                              void *overflowCounter, const void *firstRow, int32_t maxBlocks, aclrtStream stream)
{
    gmm::clear_error();
    if (!x || !xScale || !srcToken || !dest || !peerX || !peerScale || !overflowCounter)
        return gmm::fail(ACLNN_ERR_PARAM_NULLPTR, "x, xScale, srcToken, dest, peerX, peerScale and overflowCounter must not be nullptr.");
    if (numPeers < 1 || numPeers > 8) return gmm::fail(ACLNN_ERR_PARAM_INVALID, "numPeers must be in [1, 8].");
    if (hidden <= 0 || hidden % 16 != 0 || (reinterpret_cast<uintptr_t>(x) & 15))
        return gmm::fail(ACLNN_ERR_PARAM_INVALID, "hidden must be a positive multiple of 16 and x 16-byte aligned.");
    if (rows <= 0) return ACLNN_SUCCESS;
    PeerPtrs pp = {};
    for (int i = 0; i < numPeers; ++i) {
        if (!peerX[i] || !peerScale[i] || (reinterpret_cast<uintptr_t>(peerX[i]) & 15))
            return gmm::fail(ACLNN_ERR_PARAM_INVALID, "peer buffer %d is null or not 16-byte aligned.", i);
        pp.x[i] = static_cast<int8_t *>(peerX[i]);
        pp.s[i] = static_cast<float *>(peerScale[i]);
    }
    int sms = gmm::device_sm_count();
    if (sms <= 0) sms = 148;
    int grid = (int)std::min<int64_t>((rows + 7) / 8, (int64_t)sms * 8);
    if (maxBlocks > 0 && grid > maxBlocks) grid = maxBlocks;   // leave the other SMs to a GEMM running beside the dispatch
    ep_dispatch_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const int8_t *>(x), static_cast<const float *>(xScale), static_cast<const long long *>(srcToken),
        static_cast<const long long *>(dest), rows, (int)hidden, capacity, pp, numPeers, static_cast<int *>(overflowCounter),
        static_cast<const long long *>(firstRow));
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return gmm::fail(ACLNN_ERR_INNER, "dispatch kernel launch failed: %s", cudaGetErrorString(e));
    return ACLNN_SUCCESS;
}

aclnnStatus gmmB200EpCount(const void *topk, int64_t nPairs, int32_t nExperts, void *blockHist, void *totals, aclrtStream stream)
{
    gmm::clear_error();
    if (!topk || !blockHist || !totals) return gmm::fail(ACLNN_ERR_PARAM_NULLPTR, "topk, blockHist and totals must not be nullptr.");
    if (nPairs <= 0 || nPairs > 0x7fffffff || nExperts <= 0 || nExperts > kMaxSegments)
        return gmm::fail(ACLNN_ERR_PARAM_INVALID, "need 0 < nPairs < 2^31 and 0 < nExperts <= %d.", kMaxSegments);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    cudaError_t e = cudaMemsetAsync(totals, 0, sizeof(long long) * (size_t)nExperts, st);
    if (e != cudaSuccess) return gmm::fail(ACLNN_ERR_INNER, "memset failed: %s", cudaGetErrorString(e));
    const int blocks = (int)((nPairs + kRouteBlock - 1) / kRouteBlock);
    ep_count_kernel<<<blocks, 256, 0, st>>>(static_cast<const long long *>(topk), (int)nPairs, nExperts, static_cast<int *>(blockHist),
                                            static_cast<long long *>(totals));
    e = cudaGetLastError();
    if (e != cudaSuccess) return gmm::fail(ACLNN_ERR_INNER, "count kernel launch failed: %s", cudaGetErrorString(e));
    return ACLNN_SUCCESS;
}

aclnnStatus gmmB200EpRoute(const void *topk, const void *blockHist, const void *allCounts, int64_t nPairs, int32_t topK, int32_t world,
                           int32_t expertsPerRank, int32_t rank, int64_t capacity, int64_t tokenBase, int64_t resultBase, void *srcToken,
                           void *order, void *sendDest, void *retDest, void *groupList, void *firstRow, aclrtStream stream)
{
    gmm::clear_error();
    if (!topk || !blockHist || !allCounts || !srcToken || !order || !sendDest || !retDest || !groupList || !firstRow)
        return gmm::fail(ACLNN_ERR_PARAM_NULLPTR, "all buffers must not be nullptr.");
    if (nPairs <= 0 || nPairs > 0x7fffffff || topK <= 0 || world < 1 || world > 8 || expertsPerRank < 1 ||
        world * expertsPerRank > kMaxSegments || rank < 0 || rank >= world || capacity <= 0 || capacity > 0x7fffffff)
        return gmm::fail(ACLNN_ERR_PARAM_INVALID, "bad sizes (world <= 8, world*expertsPerRank <= %d, sizes below 2^31).", kMaxSegments);
    RouteParams p;
    p.topk = static_cast<const long long *>(topk);
    p.block_hist = static_cast<const int *>(blockHist);
    p.all_counts = static_cast<const long long *>(allCounts);
    p.n_pairs = (int)nPairs; p.top_k = topK; p.world = world; p.experts = expertsPerRank; p.rank = rank;
    p.n_blocks = (int)((nPairs + kRouteBlock - 1) / kRouteBlock);
    p.capacity = (int)capacity; p.token_base = (int)tokenBase; p.result_base = resultBase;
    p.src_token = static_cast<long long *>(srcToken); p.order = static_cast<long long *>(order);
    p.send_dest = static_cast<long long *>(sendDest); p.ret_dest = static_cast<long long *>(retDest);
    p.group_list = static_cast<long long *>(groupList); p.first_row = static_cast<long long *>(firstRow);
    const int grid = p.n_blocks + (int)((capacity + kRouteBlock - 1) / kRouteBlock);
    ep_route_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(p);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return gmm::fail(ACLNN_ERR_INNER, "route kernel launch failed: %s", cudaGetErrorString(e));
    return ACLNN_SUCCESS;
}

aclnnStatus gmmB200EpInverseMap(const void *order, const void *rowsInUse, int64_t maxRows, int64_t resultBase, int64_t nPairs,
                                void *pairRow, void *badCounter, aclrtStream stream)
{
    gmm::clear_error();
    if (!order || !rowsInUse || !pairRow || !badCounter)
        return gmm::fail(ACLNN_ERR_PARAM_NULLPTR, "order, rowsInUse, pairRow and badCounter must not be nullptr.");
    if (maxRows < 0 || nPairs <= 0 || nPairs > 0x7fffffff || resultBase < 0 || resultBase + maxRows > 0x7fffffff)
        return gmm::fail(ACLNN_ERR_PARAM_INVALID, "need 0 < nPairs < 2^31, maxRows >= 0 and resultBase + maxRows < 2^31.");
    if (maxRows == 0) return ACLNN_SUCCESS;
    int sms = gmm::device_sm_count();
    if (sms <= 0) sms = 148;
    const int grid = (int)std::min<int64_t>((maxRows + 255) / 256, (int64_t)sms * 8);
    ep_inverse_map_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const long long *>(order), static_cast<const long long *>(rowsInUse), maxRows, resultBase, (int)nPairs,
        static_cast<int *>(pairRow), static_cast<int *>(badCounter));
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return gmm::fail(ACLNN_ERR_INNER, "inverse map kernel launch failed: %s", cudaGetErrorString(e));
    return ACLNN_SUCCESS;
}

aclnnStatus gmmB200EpCombine(const void *y, const void *pairRow, const void *weights, void *out, int64_t tokens, int32_t topK,
                             int64_t hidden, int64_t yRows, aclrtStream stream)
{
    gmm::clear_error();
    if (!y || !pairRow || !weights || !out) return gmm::fail(ACLNN_ERR_PARAM_NULLPTR, "y, pairRow, weights and out must not be nullptr.");
    if (tokens < 0 || tokens > 0x7fffffff || topK <= 0 || hidden <= 0 || hidden % 8 != 0 || yRows < 0 ||
        ((reinterpret_cast<uintptr_t>(y) | reinterpret_cast<uintptr_t>(out)) & 15))
        return gmm::fail(ACLNN_ERR_PARAM_INVALID, "hidden must be a positive multiple of 8, y and out 16-byte aligned, tokens < 2^31.");
    if (tokens == 0) return ACLNN_SUCCESS;
    ep_combine_kernel<<<(unsigned)tokens, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint4 *>(y), static_cast<const int *>(pairRow), static_cast<const float *>(weights), static_cast<uint4 *>(out),
        topK, (int)(hidden / 8), yRows);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return gmm::fail(ACLNN_ERR_INNER, "combine kernel launch failed: %s", cudaGetErrorString(e));
    return ACLNN_SUCCESS;
}

}  // extern "C"
