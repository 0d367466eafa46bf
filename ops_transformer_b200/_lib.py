"""ctypes binding of libgmm_b200.so, the C-ABI library that carries the CUDA kernels.

The library is required: importing this module without it raises, there is no CPU fallback.
"""
from __future__ import annotations

import ctypes as C
import os

_PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG, "libgmm_b200.so")

# aclDataType / aclFormat codes (include/aclnn/aclnn_base.h)
ACL_FLOAT, ACL_FLOAT16, ACL_INT8, ACL_INT32, ACL_INT64, ACL_BF16 = 0, 1, 2, 3, 9, 27
ACL_FORMAT_ND, ACL_FORMAT_FRACTAL_NZ = 2, 29

ACLNN_SUCCESS = 0
ACLNN_ERR_PARAM_NULLPTR = 161001
ACLNN_ERR_PARAM_INVALID = 161002
ACLNN_ERR_RUNTIME_ERROR = 361001
ACLNN_ERR_INNER = 561000

# Every symbol the public headers under include/ declare.
EXPORTED_SYMBOLS = [
    "aclCreateTensor", "aclDestroyTensor", "aclCreateTensorList", "aclDestroyTensorList", "aclCreateIntArray",
    "aclDestroyIntArray", "aclDestroyAclOpExecutor", "aclGetRecentErrMsg",
    "aclnnGroupedMatmulV4GetWorkspaceSize", "aclnnGroupedMatmulV4",
    "aclnnGroupedMatmulV5GetWorkspaceSize", "aclnnGroupedMatmulV5",
    "aclnnGroupedMatmulWeightNzGetWorkspaceSize", "aclnnGroupedMatmulWeightNz",
    "aclnnGroupedMatmulFinalizeRoutingWeightNzGetWorkspaceSize", "aclnnGroupedMatmulFinalizeRoutingWeightNz",
    "aclnnGroupedMatmulFinalizeRoutingWeightNzV2GetWorkspaceSize", "aclnnGroupedMatmulFinalizeRoutingWeightNzV2",
    "gmmB200GroupedMatmulFinalizeRouting",
    "aclnnMoeInitRoutingV3GetWorkspaceSize", "aclnnMoeInitRoutingV3",
    "aclnnGroupedMatmulSwigluQuantGetWorkspaceSize", "aclnnGroupedMatmulSwigluQuant",
    "aclnnGroupedMatmulSwigluQuantWeightNZGetWorkspaceSize", "aclnnGroupedMatmulSwigluQuantWeightNZ",
    "gmmB200Version", "gmmB200CheckStatus", "gmmB200SetExecutorOptions", "gmmB200GroupedMatmulW8A8WorkspaceSize", "gmmB200GroupedMatmulW8A8",
    "gmmB200GroupedMatmulSwigluQuantWorkspaceSize", "gmmB200GroupedMatmulSwigluQuant",
    "gmmB200NoAllocScratchBytes", "gmmB200GroupedMatmulSwigluQuantNoAlloc", "gmmB200NoAllocCheckStatus",
    "gmmB200PeerAlloc", "gmmB200PeerFree", "gmmB200PeerExport", "gmmB200PeerImport", "gmmB200PeerRelease", "gmmB200EpDispatch", "gmmB200EpCount", "gmmB200EpRoute", "gmmB200EpInverseMap", "gmmB200EpCombine",
]


class LaunchOptions(C.Structure):
    """gmmB200LaunchOptions (include/gmm_b200.h): per-call CTA cap, timing events, wait bound, abort-path test hook."""
    _fields_ = [("structSize", C.c_uint32), ("maxCtas", C.c_int32), ("startEvent", C.c_void_p), ("stopEvent", C.c_void_p),
                ("waitLimitCycles", C.c_int64), ("testSkipKBlocks", C.c_int32), ("reserved", C.c_int32)]

    def __init__(self, max_ctas: int = 0, start_event=None, stop_event=None, wait_limit_cycles: int = 0, test_skip_k_blocks: int = 0):
        super().__init__(C.sizeof(LaunchOptions), max_ctas, start_event, stop_event, wait_limit_cycles, test_skip_k_blocks, 0)


class LibraryMissing(RuntimeError):
    pass


def _load():
    if not os.path.exists(LIB_PATH):
        raise LibraryMissing(
            f"{LIB_PATH} is missing: build it with `python -m ops_transformer_b200._build` "
            "(nvcc, sm_100a).  There is no CPU fallback.")
    L = C.CDLL(LIB_PATH)
    p, i64, u64, i32 = C.c_void_p, C.c_int64, C.c_uint64, C.c_int32
    L.aclCreateTensor.restype = p
    L.aclCreateTensor.argtypes = [C.POINTER(i64), u64, i32, C.POINTER(i64), i64, i32, C.POINTER(i64), u64, p]
    L.aclDestroyTensor.argtypes = [p]
    L.aclCreateTensorList.restype = p
    L.aclCreateTensorList.argtypes = [C.POINTER(p), u64]
    L.aclDestroyTensorList.argtypes = [p]
    L.aclCreateIntArray.restype = p
    L.aclCreateIntArray.argtypes = [C.POINTER(i64), u64]
    L.aclDestroyIntArray.argtypes = [p]
    L.aclDestroyAclOpExecutor.argtypes = [p]
    L.aclGetRecentErrMsg.restype = C.c_char_p
    L.aclnnGroupedMatmulV4GetWorkspaceSize.argtypes = [p] * 12 + [i64] * 4 + [p] * 3 + [C.POINTER(u64), C.POINTER(p)]
    L.aclnnGroupedMatmulV4.argtypes = [p, u64, p, p]
    L.aclnnGroupedMatmulV5GetWorkspaceSize.argtypes = [p] * 12 + [i64] * 4 + [p] * 4 + [C.POINTER(u64), C.POINTER(p)]
    L.aclnnGroupedMatmulV5.argtypes = [p, u64, p, p]
    L.aclnnGroupedMatmulWeightNzGetWorkspaceSize.argtypes = [p] * 12 + [i64] * 4 + [p, i64] + [p] * 3 + [C.POINTER(u64), C.POINTER(p)]
    L.aclnnGroupedMatmulWeightNz.argtypes = [p, u64, p, p]
    f32, b8 = C.c_float, C.c_bool
    po = C.POINTER(LaunchOptions)
    L.aclnnGroupedMatmulFinalizeRoutingWeightNzGetWorkspaceSize.argtypes = [p] * 9 + [i64, f32, i64, b8, b8, i64, p, C.POINTER(u64), C.POINTER(p)]
    L.aclnnGroupedMatmulFinalizeRoutingWeightNz.argtypes = [p, u64, p, p]
    L.aclnnGroupedMatmulFinalizeRoutingWeightNzV2GetWorkspaceSize.argtypes = [p] * 12 + [i64, f32, i64, b8, b8, i64, p, p, C.POINTER(u64), C.POINTER(p)]
    L.aclnnGroupedMatmulFinalizeRoutingWeightNzV2.argtypes = [p, u64, p, p]
    L.aclnnMoeInitRoutingV3GetWorkspaceSize.argtypes = [p] * 4 + [i64] * 5 + [b8, i64, p, i64] + [p] * 4 + [C.POINTER(u64), C.POINTER(p)]
    L.aclnnMoeInitRoutingV3.argtypes = [p, u64, p, p]
    L.gmmB200GroupedMatmulFinalizeRouting.argtypes = [p, p, i32, p, i32, p, p, p, i64, i32, p, i64, i64, f32, p, p, i32, i64, i64, i64, i64, p, i64, p, u64, p,
                                                      C.POINTER(LaunchOptions)]
    L.aclnnGroupedMatmulSwigluQuantWeightNZGetWorkspaceSize.argtypes = [p] * 10 + [C.POINTER(u64), C.POINTER(p)]
    L.aclnnGroupedMatmulSwigluQuantWeightNZ.argtypes = [p, u64, p, p]
    L.aclnnGroupedMatmulSwigluQuantGetWorkspaceSize.argtypes = [p] * 10 + [C.POINTER(u64), C.POINTER(p)]
    L.aclnnGroupedMatmulSwigluQuant.argtypes = [p, u64, p, p]
    L.gmmB200CheckStatus.argtypes = [p, u64, p, C.POINTER(i32)]
    L.gmmB200SetExecutorOptions.argtypes = [p, po]
    L.gmmB200GroupedMatmulW8A8WorkspaceSize.argtypes = [i64, i64, i64, i64, i32, C.POINTER(u64)]
    L.gmmB200GroupedMatmulW8A8.argtypes = [p, p, p, i32, p, p, i32, p, i64, i32, i64, i64, i64, i64, i32, i32, p, p, i32, i64, p, i32, p, u64, p, po]
    L.gmmB200GroupedMatmulSwigluQuantWorkspaceSize.argtypes = [i64, i64, i64, i64, C.POINTER(u64)]
    L.gmmB200GroupedMatmulSwigluQuant.argtypes = [p, p, p, i32, p, p, i64, i64, i64, i64, i64, i32, p, p, p, u64, p, po]
    L.gmmB200PeerAlloc.argtypes = [u64, C.POINTER(p)]
    L.gmmB200PeerFree.argtypes = [p]
    L.gmmB200PeerExport.argtypes = [p, p]
    L.gmmB200PeerImport.argtypes = [p, C.POINTER(p)]
    L.gmmB200PeerRelease.argtypes = [p]
    L.gmmB200EpDispatch.argtypes = [p, p, p, p, i64, i64, i64, C.POINTER(p), C.POINTER(p), i32, p, p, i32, p]
    L.gmmB200EpCount.argtypes = [p, i64, i32, p, p, p]
    L.gmmB200EpRoute.argtypes = [p, p, p, i64, i32, i32, i32, i32, i64, i64, i64, p, p, p, p, p, p, p]
    L.gmmB200EpInverseMap.argtypes = [p, p, i64, i64, i64, p, p, p]
    L.gmmB200EpCombine.argtypes = [p, p, p, p, i64, i32, i64, i64, p]
    L.gmmB200NoAllocScratchBytes.restype = u64
    L.gmmB200GroupedMatmulSwigluQuantNoAlloc.argtypes = [p, p, p, i32, p, p, i64, i64, i64, i64, i64, p, p, p]
    L.gmmB200NoAllocCheckStatus.argtypes = [p, C.POINTER(i32)]
    return L


_LIB = None


def lib():
    global _LIB
    if _LIB is None:
        _LIB = _load()
    return _LIB


def last_error() -> str:
    return lib().aclGetRecentErrMsg().decode("utf-8", "replace")
