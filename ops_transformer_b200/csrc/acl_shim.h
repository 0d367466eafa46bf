// Concrete definitions of the opaque aclnn handle types (internal).
#pragma once
#include <cstdarg>
#include <cstdint>
#include <string>
#include <vector>

#include "aclnn/aclnn_base.h"
#include "gmm_common.h"

struct aclTensor {
    std::vector<int64_t> view_dims;
    std::vector<int64_t> strides;   // elements
    int64_t offset = 0;             // elements
    aclDataType dtype = ACL_DT_UNDEFINED;
    aclFormat format = ACL_FORMAT_ND;
    std::vector<int64_t> storage_dims;
    void *data = nullptr;

    size_t rank() const { return view_dims.size(); }
    int64_t dim(size_t i) const { return view_dims[i]; }
    int64_t numel() const
    {
        int64_t n = 1;
        for (int64_t d : view_dims) n *= d;
        return n;
    }
    bool empty() const { return numel() == 0; }
    bool contiguous() const
    {
        int64_t expect = 1;
        for (size_t i = view_dims.size(); i-- > 0;) {
            if (view_dims[i] != 1 && strides[i] != expect) return false;
            expect *= view_dims[i];
        }
        return true;
    }
};

struct aclTensorList {
    std::vector<const aclTensor *> items;
};

struct aclIntArray {
    std::vector<int64_t> values;
};

struct aclOpExecutor {
    enum Kind { kNoop = 0, kGmm = 1, kInitRouting = 2 } kind = kNoop;
    uint32_t magic = 0xac10e8ecu;
    bool consumed = false;
    const char *op_name = "";
    gmm::Problem problem;
    gmm::Plan plan;
    gmm::InitRoutingProblem routing;
    std::vector<gmm::StagedView> staged;   // non-contiguous views with a contiguous copy in the workspace tail
    size_t staged_bytes = 0;
};

namespace gmm {

size_t dtype_size(aclDataType t);
// Stores a printf-style message as the calling thread's most recent error and returns `code`.
aclnnStatus fail(aclnnStatus code, const char *fmt, ...) __attribute__((format(printf, 2, 3)));
void clear_error();
// Element address of a tensor view's first element.
inline void *tensor_ptr(const aclTensor *t)
{
    return static_cast<char *>(t->data) + (size_t)t->offset * dtype_size(t->dtype);
}
aclnnStatus run_executor(const char *op_name, void *workspace, uint64_t workspace_size, aclOpExecutor *executor,
                         aclrtStream stream);

}  // namespace gmm
