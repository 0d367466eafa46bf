"""B200-native grouped int8 GEMM operators behind the aclnn two-phase C API.

``grouped_matmul_v4`` and ``grouped_matmul_swiglu_quant`` mirror the reference operators
``aclnnGroupedMatmulV4`` (W8A8 per-token mode) and ``aclnnGroupedMatmulSwigluQuant``; both go through the
C-ABI library ``libgmm_b200.so`` and run hand-written sm_100a kernels.  There is no CPU fallback.
"""
from .acl import (AclnnError, grouped_matmul_swiglu_quant, grouped_matmul_v4, check_status, format_cast_nz,  # noqa: F401
                  grouped_matmul_finalize_routing, grouped_matmul_finalize_routing_flat, moe_init_routing_v3)  # noqa: F401
from ._lib import ACL_FORMAT_FRACTAL_NZ, ACL_FORMAT_ND, LIB_PATH, LaunchOptions, lib  # noqa: F401
