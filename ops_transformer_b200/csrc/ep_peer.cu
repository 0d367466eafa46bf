// Peer-memory plumbing for the expert-parallel path: buffers that the other GPUs of the node can write into
// (CUDA IPC), and the dispatch kernel that gathers a rank's token rows and stores each one straight into the row
// of the owning GPU's expert-major activation buffer - gather, all-to-all and re-ordering in one pass of stores over
// NVLink.  It takes the place of the reference's MoeDistributeDispatch window writes
// (mc2/moe_distribute_dispatch_v2/docs/MoeDistributeDispatch-Combine算子设计介绍.md:40-66) followed by MoeReRouting
// (moe/moe_re_routing/README.md:12-26) for rows that are already quantised.
// Only plain stores to peer memory are used; no bulk-tensor copies touch another GPU's memory.
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
// `capacity` is not written; the kernel counts such rows in *overflow instead.
__global__ void __launch_bounds__(256) ep_dispatch_kernel(const int8_t *__restrict__ x, const float *__restrict__ xs,
                                                           const long long *__restrict__ src_token,
                                                           const long long *__restrict__ dest, long long rows, int hidden,
                                                           long long capacity, PeerPtrs pp, int *overflow,
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
        const int gpu = (int)(d >> 40) & 7;
        const long long drow = d & kRowMask;
        if (drow >= capacity) {
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

}  // namespace

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
                              void *overflowCounter, const void *firstRow, aclrtStream stream)
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
    const int grid = (int)std::min<int64_t>((rows + 7) / 8, (int64_t)sms * 8);
    ep_dispatch_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const int8_t *>(x), static_cast<const float *>(xScale), static_cast<const long long *>(srcToken),
        static_cast<const long long *>(dest), rows, (int)hidden, capacity, pp, static_cast<int *>(overflowCounter),
        static_cast<const long long *>(firstRow));
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return gmm::fail(ACLNN_ERR_INNER, "dispatch kernel launch failed: %s", cudaGetErrorString(e));
    return ACLNN_SUCCESS;
}

}  // extern "C"
