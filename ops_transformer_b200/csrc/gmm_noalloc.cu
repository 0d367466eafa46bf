// grouped_matmul_swiglu_quant for callers that must not allocate device memory.
//
// Some hosts of this library cannot call cudaMalloc at the point where they run the operator: an inference
// server that freezes its memory pool after warm-up, a plugin that runs inside someone else's allocator
// arena, a latency-critical loop where the implicit device synchronisation of cudaMalloc / cudaFree is not
// acceptable.  For them the scratch memory that the operator needs (the status word, the per-row maxima and the
// fp32 SwiGLU staging) lives in a fixed array inside the library image instead of a caller-provided workspace.
// The price: every GPU that loads the library holds kNoAllocScratchBytes of device memory until the process
// exits, and problems whose scratch does not fit are rejected.
#include <mutex>

#include "acl_shim.h"
#include "gmm_b200.h"

namespace {

constexpr size_t kNoAllocScratchBytes = GMM_B200_NO_ALLOC_SCRATCH_BYTES;
constexpr int kMaxDevices = 64;

// The scratch itself.  In host code this name is only a handle for cudaGetSymbolAddress, never an address.
static __device__ __align__(256) unsigned char g_noalloc_scratch[kNoAllocScratchBytes];

std::mutex g_mu;
void *g_scratch_addr[kMaxDevices] = {nullptr};

// Device address of the array on the current device; resolved once per device, with that device current.
cudaError_t scratch_address(void **out)
{
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 0 || dev >= kMaxDevices) return cudaErrorInvalidDevice;
    std::lock_guard<std::mutex> lk(g_mu);
    if (!g_scratch_addr[dev]) {
        void *ptr = nullptr;
        e = cudaGetSymbolAddress(&ptr, g_noalloc_scratch);
        if (e != cudaSuccess) return e;
        if (!ptr) return cudaErrorInvalidSymbol;
        g_scratch_addr[dev] = ptr;
    }
    *out = g_scratch_addr[dev];
    return cudaSuccess;
}

}  // namespace

extern "C" {

uint64_t gmmB200NoAllocScratchBytes(void) { return kNoAllocScratchBytes; }

aclnnStatus gmmB200GroupedMatmulSwigluQuantNoAlloc(const void *x, const void *weight, const void *weightScale,
                                                   int32_t weightScaleDtype, const void *xScale, const void *groupList,
                                                   int64_t groupListLen, int64_t m, int64_t k, int64_t n, int64_t e,
                                                   void *output, void *outputScale, aclrtStream stream)
{
    using namespace gmm;
    clear_error();
    if (!(x && weight && weightScale && xScale && groupList && output && outputScale))
        return fail(ACLNN_ERR_PARAM_NULLPTR, "x, weight, weightScale, xScale, groupList, output and outputScale must not be nullptr.");
    if (!(m >= 0 && m <= 0x7fffffffll / 2 && k > 0 && n > 0 && e > 0 && k < 65536 && n <= 10240 && n % 2 == 0))
        return fail(ACLNN_ERR_PARAM_INVALID, "need 0 <= m < 2^30, 0 < k < 65536, 0 < n <= 10240 and even, e > 0.");
    if (!(weightScaleDtype == ACL_FLOAT || weightScaleDtype == ACL_FLOAT16 || weightScaleDtype == ACL_BF16))
        return fail(ACLNN_ERR_PARAM_INVALID, "weightScaleDtype must be float32, float16 or bfloat16.");
    if (!(groupListLen >= 0 && groupListLen <= e && groupListLen <= 1024))
        return fail(ACLNN_ERR_PARAM_INVALID, "groupListLen %lld out of range [0, min(e, 1024)].", (long long)groupListLen);
    if (m == 0 || groupListLen == 0) return ACLNN_SUCCESS;

    Problem p;
    p.x = static_cast<const int8_t *>(x);
    p.w = static_cast<const int8_t *>(weight);
    p.w_scale = weightScale;
    p.w_scale_dtype = weightScaleDtype;
    p.x_scale = static_cast<const float *>(xScale);
    p.group_list = static_cast<const int64_t *>(groupList);
    p.gl_len = (int)groupListLen;
    p.gl_type = 0;
    p.M = m; p.K = k; p.N = n; p.E = e;
    p.mode = kModeSwigluQuant;
    p.out0 = output;
    p.out1 = outputScale;
    Plan plan;
    make_plan(p, &plan);
    if (plan.ws_bytes > kNoAllocScratchBytes)
        return fail(ACLNN_ERR_PARAM_INVALID,
                    "problem needs %llu bytes of scratch (about 4*m*n/2), more than the %llu bytes built into the library; "
                    "use aclnnGroupedMatmulSwigluQuant with a caller-provided workspace for this size.",
                    (unsigned long long)plan.ws_bytes, (unsigned long long)kNoAllocScratchBytes);
    void *scratch = nullptr;
    cudaError_t ce = scratch_address(&scratch);
    if (ce != cudaSuccess) return fail(ACLNN_ERR_RUNTIME_ERROR, "cannot resolve the built-in scratch array: %s", cudaGetErrorString(ce));
    // launch() clears the status word and the row maxima (the part that must start at zero) on `stream`.
    ce = launch(p, plan, scratch, kNoAllocScratchBytes, static_cast<cudaStream_t>(stream));
    if (ce != cudaSuccess) return fail(ACLNN_ERR_INNER, "kernel launch failed: %s", cudaGetErrorString(ce));
    return ACLNN_SUCCESS;
}

// The kernels keep their 4-word status record at the start of the scratch array, which a caller of the entry point above
// cannot address.  This call waits for `stream`, copies the record out (into pageable host memory: no allocation) and
// reports it like gmmB200CheckStatus does for a caller-provided workspace.
aclnnStatus gmmB200NoAllocCheckStatus(aclrtStream stream, int32_t record[4])
{
    using namespace gmm;
    clear_error();
    void *scratch = nullptr;
    cudaError_t ce = scratch_address(&scratch);
    if (ce != cudaSuccess) return fail(ACLNN_ERR_RUNTIME_ERROR, "cannot resolve the built-in scratch array: %s", cudaGetErrorString(ce));
    return gmmB200CheckStatus(scratch, 16, stream, record);
}

}  // extern "C"
