// Handle objects of the aclnn-compatible C API (tensors, lists, executors) and the per-thread error text.
// Stand-in for the parts of CANN's closed runtime that callers of the grouped-matmul operators touch
// (usage pattern: gmm/grouped_matmul/examples/test_aclnn_grouped_matmul.cpp:71-110 of the reference).
#include "acl_shim.h"

#include <cstdio>
#include <cstdlib>
#include <mutex>
#include <unordered_set>

namespace gmm {

static thread_local std::string t_last_error;

size_t dtype_size(aclDataType t)
{
    switch (t) {
        case ACL_FLOAT: case ACL_INT32: case ACL_UINT32: return 4;
        case ACL_FLOAT16: case ACL_BF16: case ACL_INT16: case ACL_UINT16: return 2;
        case ACL_INT8: case ACL_UINT8: case ACL_BOOL: return 1;
        case ACL_INT64: case ACL_UINT64: case ACL_DOUBLE: return 8;
        default: return 1;
    }
}

aclnnStatus fail(aclnnStatus code, const char *fmt, ...)
{
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof(buf), fmt, ap);
    va_end(ap);
    t_last_error = buf;
    static const bool verbose = [] {
        const char *e = std::getenv("GMM_B200_LOG");
        return e && e[0] && e[0] != '0';
    }();
    if (verbose) fprintf(stderr, "[gmm_b200] error %d: %s\n", (int)code, buf);
    return code;
}

void clear_error() { t_last_error.clear(); }

// Executors handed out by a first-phase call and not yet run or destroyed.
static std::mutex g_exec_mu;
static std::unordered_set<aclOpExecutor *> g_live_executors;

void register_executor(aclOpExecutor *e)
{
    std::lock_guard<std::mutex> lk(g_exec_mu);
    g_live_executors.insert(e);
}
// Removes the executor from the live set; false if it was not there (already run, destroyed, or never ours).
bool claim_executor(aclOpExecutor *e)
{
    std::lock_guard<std::mutex> lk(g_exec_mu);
    return g_live_executors.erase(e) == 1;
}

bool executor_is_live(aclOpExecutor *e)
{
    std::lock_guard<std::mutex> lk(g_exec_mu);
    return g_live_executors.count(e) == 1;
}

}  // namespace gmm

extern "C" {

aclTensor *aclCreateTensor(const int64_t *viewDims, uint64_t viewDimsNum, aclDataType dataType, const int64_t *stride,
                           int64_t offset, aclFormat format, const int64_t *storageDims, uint64_t storageDimsNum,
                           void *tensorData)
{
    if ((viewDimsNum && !viewDims) || viewDimsNum > 8 || storageDimsNum > 8) return nullptr;
    aclTensor *t = new aclTensor();
    t->view_dims.assign(viewDims, viewDims + viewDimsNum);
    if (stride) {
        t->strides.assign(stride, stride + viewDimsNum);
    } else {
        t->strides.assign(viewDimsNum, 1);
        for (int64_t i = (int64_t)viewDimsNum - 2; i >= 0; --i) t->strides[i] = t->strides[i + 1] * t->view_dims[i + 1];
    }
    t->offset = offset;
    t->dtype = dataType;
    t->format = format;
    if (storageDims) t->storage_dims.assign(storageDims, storageDims + storageDimsNum);
    t->data = tensorData;
    return t;
}

aclnnStatus aclDestroyTensor(const aclTensor *tensor)
{
    delete tensor;
    return ACLNN_SUCCESS;
}

aclTensorList *aclCreateTensorList(const aclTensor *const *value, uint64_t size)
{
    if (size && !value) return nullptr;
    aclTensorList *l = new aclTensorList();
    l->items.assign(value, value + size);
    return l;
}

aclnnStatus aclDestroyTensorList(const aclTensorList *tensorList)
{
    if (tensorList) {
        for (const aclTensor *t : tensorList->items) delete t;
        delete tensorList;
    }
    return ACLNN_SUCCESS;
}

aclIntArray *aclCreateIntArray(const int64_t *value, uint64_t size)
{
    if (size && !value) return nullptr;
    aclIntArray *a = new aclIntArray();
    a->values.assign(value, value + size);
    return a;
}

aclnnStatus aclDestroyIntArray(const aclIntArray *array)
{
    delete array;
    return ACLNN_SUCCESS;
}

aclnnStatus aclDestroyAclOpExecutor(aclOpExecutor *executor)
{
    if (!executor) return ACLNN_ERR_PARAM_NULLPTR;
    if (!gmm::claim_executor(executor)) return gmm::fail(ACLNN_ERR_PARAM_INVALID, "executor is not live (already run or destroyed)");
    delete executor;
    return ACLNN_SUCCESS;
}

const char *aclGetRecentErrMsg(void) { return gmm::t_last_error.c_str(); }

}  // extern "C"
