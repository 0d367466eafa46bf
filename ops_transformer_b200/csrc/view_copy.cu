// Strided view <-> contiguous buffer copies.  The aclnn contract lets callers pass non-contiguous views: inputs are made
// contiguous inside the executor and results are copied back into possibly strided outputs (the reference does this with
// l0op::Contiguous / l0op::ViewCopy, e.g. gmm/grouped_matmul/op_host/op_api/aclnn_grouped_matmul.cpp:1640-1667, 1802-1805).
// Here the contiguous copies live in the tail of the caller's workspace and one kernel per tensor moves the elements.
#include "gmm_common.h"

namespace gmm {
namespace {

struct ViewCopyParams {
    const char *src;
    char *dst;
    int rank, elem;
    long long total;
    long long dims[8];
    long long view_stride[8];  // elements
};

// Element i of the contiguous buffer corresponds to the view element with the same row-major coordinates.
template <typename T, bool TO_CONTIGUOUS>
__global__ void __launch_bounds__(256) view_copy_kernel(const ViewCopyParams p)
{
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < p.total; i += (long long)gridDim.x * blockDim.x) {
        long long rem = i, off = 0;
        for (int d = p.rank - 1; d >= 0; --d) {
            const long long c = rem % p.dims[d];
            rem /= p.dims[d];
            off += c * p.view_stride[d];
        }
        if (TO_CONTIGUOUS) reinterpret_cast<T *>(p.dst)[i] = reinterpret_cast<const T *>(p.src)[off];
        else reinterpret_cast<T *>(p.dst)[off] = reinterpret_cast<const T *>(p.src)[i];
    }
}

template <bool TO_CONTIGUOUS>
cudaError_t launch_elem(const ViewCopyParams &p, cudaStream_t stream)
{
    long long blocks = (p.total + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    const unsigned g = (unsigned)blocks;
    switch (p.elem) {
        case 1: view_copy_kernel<uint8_t, TO_CONTIGUOUS><<<g, 256, 0, stream>>>(p); break;
        case 2: view_copy_kernel<uint16_t, TO_CONTIGUOUS><<<g, 256, 0, stream>>>(p); break;
        case 4: view_copy_kernel<uint32_t, TO_CONTIGUOUS><<<g, 256, 0, stream>>>(p); break;
        case 8: view_copy_kernel<unsigned long long, TO_CONTIGUOUS><<<g, 256, 0, stream>>>(p); break;
        default: return cudaErrorInvalidValue;
    }
    return cudaGetLastError();
}

}  // namespace

cudaError_t view_copy_launch(const StagedView &v, void *contiguous, bool to_contiguous, cudaStream_t stream)
{
    ViewCopyParams p;
    p.rank = (int)v.dims.size();
    if (p.rank > 8) return cudaErrorInvalidValue;
    p.elem = v.elem;
    p.total = 1;
    for (int d = 0; d < p.rank; ++d) {
        p.dims[d] = v.dims[d];
        p.view_stride[d] = v.strides[d];
        p.total *= v.dims[d];
    }
    if (p.total == 0) return cudaSuccess;
    if (to_contiguous) {
        p.src = static_cast<const char *>(v.data);
        p.dst = static_cast<char *>(contiguous);
        return launch_elem<true>(p, stream);
    }
    p.src = static_cast<const char *>(contiguous);
    p.dst = static_cast<char *>(v.data);
    return launch_elem<false>(p, stream);
}

}  // namespace gmm
