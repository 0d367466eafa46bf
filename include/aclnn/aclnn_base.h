/*
 * Minimal, source-compatible stand-in for CANN's closed "aclnn/aclnn_base.h" / "acl/acl_base.h", limited to what
 * the grouped-matmul operators and their callers use.  The reference includes the CANN header at
 * gmm/grouped_matmul/op_host/op_api/aclnn_grouped_matmul_v4.h:13 and
 * gmm/grouped_matmul_swiglu_quant/op_host/op_api/aclnn_grouped_matmul_swiglu_quant.h:13; callers use the types the
 * way gmm/grouped_matmul/examples/test_aclnn_grouped_matmul.cpp:71-110 and
 * gmm/grouped_matmul_swiglu_quant/examples/test_aclnn_grouped_matmul_swiglu_quant.cpp:52-73 do.
 *
 * Differences from CANN: the stream is a CUDA stream (cudaStream_t passed as aclrtStream) and device addresses are
 * CUDA device pointers.  Everything is plain C: opaque handles, pointers and sizes.
 */
#ifndef B200_ACLNN_BASE_H
#define B200_ACLNN_BASE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define ACL_FUNC_VISIBILITY __attribute__((visibility("default")))

typedef int32_t aclnnStatus;
typedef void *aclrtStream; /* a cudaStream_t */

typedef struct aclTensor aclTensor;
typedef struct aclTensorList aclTensorList;
typedef struct aclIntArray aclIntArray;
typedef struct aclOpExecutor aclOpExecutor;

/* Return codes: docs/context/aclnn返回码.md:16-116 of the reference. */
#define ACLNN_SUCCESS 0
#define ACLNN_ERR_PARAM_NULLPTR 161001
#define ACLNN_ERR_PARAM_INVALID 161002
#define ACLNN_ERR_RUNTIME_ERROR 361001
#define ACLNN_ERR_INNER 561000
#define ACLNN_ERR_INNER_INFERSHAPE_ERROR 561001
#define ACLNN_ERR_INNER_TILING_ERROR 561002
#define ACLNN_ERR_INNER_FIND_KERNEL_ERROR 561003
#define ACLNN_ERR_INNER_CREATE_EXECUTOR 561101
#define ACLNN_ERR_INNER_NOT_TRANS_EXECUTOR 561102
#define ACLNN_ERR_INNER_NULLPTR 561103

/* Values as in CANN's public acl_base.h. */
typedef enum {
    ACL_DT_UNDEFINED = -1,
    ACL_FLOAT = 0,
    ACL_FLOAT16 = 1,
    ACL_INT8 = 2,
    ACL_INT32 = 3,
    ACL_UINT8 = 4,
    ACL_INT16 = 6,
    ACL_UINT16 = 7,
    ACL_UINT32 = 8,
    ACL_INT64 = 9,
    ACL_UINT64 = 10,
    ACL_DOUBLE = 11,
    ACL_BOOL = 12,
    ACL_BF16 = 27,
    ACL_INT4 = 29
} aclDataType;

typedef enum {
    ACL_FORMAT_UNDEFINED = -1,
    ACL_FORMAT_NCHW = 0,
    ACL_FORMAT_NHWC = 1,
    ACL_FORMAT_ND = 2,
    ACL_FORMAT_NC1HWC0 = 3,
    ACL_FORMAT_FRACTAL_Z = 4,
    ACL_FORMAT_FRACTAL_NZ = 29
} aclFormat;

/* A tensor is a view (dims, strides and offset in elements) over a storage shape at a device address.  The
 * caller keeps ownership of the device memory; the handle only describes it. */
ACL_FUNC_VISIBILITY aclTensor *aclCreateTensor(const int64_t *viewDims, uint64_t viewDimsNum, aclDataType dataType,
                                               const int64_t *stride, int64_t offset, aclFormat format,
                                               const int64_t *storageDims, uint64_t storageDimsNum, void *tensorData);
ACL_FUNC_VISIBILITY aclnnStatus aclDestroyTensor(const aclTensor *tensor);

/* The list takes ownership of the tensor handles passed in; destroying the list destroys them. */
ACL_FUNC_VISIBILITY aclTensorList *aclCreateTensorList(const aclTensor *const *value, uint64_t size);
ACL_FUNC_VISIBILITY aclnnStatus aclDestroyTensorList(const aclTensorList *tensorList);

ACL_FUNC_VISIBILITY aclIntArray *aclCreateIntArray(const int64_t *value, uint64_t size);
ACL_FUNC_VISIBILITY aclnnStatus aclDestroyIntArray(const aclIntArray *array);

/* Releases an executor that was obtained from a GetWorkspaceSize call but never run.  An executor that has been
 * passed to the second-phase call is consumed by it and must not be destroyed or reused. */
ACL_FUNC_VISIBILITY aclnnStatus aclDestroyAclOpExecutor(aclOpExecutor *executor);

/* Text of the most recent error on the calling thread (empty string when none). */
ACL_FUNC_VISIBILITY const char *aclGetRecentErrMsg(void);

#ifdef __cplusplus
}
#endif

#endif /* B200_ACLNN_BASE_H */
