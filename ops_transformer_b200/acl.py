"""Host-side mirror of the reference operator interface on top of the C ABI.

``grouped_matmul_v4`` follows aclnnGroupedMatmulV4 (gmm/grouped_matmul/op_host/op_api/aclnn_grouped_matmul_v4.h:66-86
of the reference) and ``grouped_matmul_swiglu_quant`` follows aclnnGroupedMatmulSwigluQuant
(gmm/grouped_matmul_swiglu_quant/op_host/op_api/aclnn_grouped_matmul_swiglu_quant.h:37-52): same argument
names and meaning, same two-phase sequence (GetWorkspaceSize -> allocate -> launch on a stream), same status
codes raised as ``AclnnError``.  torch is used for device memory and streams only.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional, Sequence

import torch

from . import _lib
from ._lib import (ACL_BF16, ACL_FLOAT, ACL_FLOAT16, ACL_FORMAT_ND, ACL_INT8, ACL_INT32, ACL_INT64, ACLNN_SUCCESS)

_DTYPES = {
    torch.float32: ACL_FLOAT, torch.float16: ACL_FLOAT16, torch.int8: ACL_INT8, torch.int32: ACL_INT32,
    torch.int64: ACL_INT64, torch.bfloat16: ACL_BF16,
}


class AclnnError(RuntimeError):
    """A non-zero aclnnStatus.  ``status`` holds the code, the text comes from aclGetRecentErrMsg."""

    def __init__(self, status: int, where: str):
        self.status = int(status)
        super().__init__(f"{where} failed with aclnnStatus {status}: {_lib.last_error()}")


def _i64(values: Sequence[int]):
    return (C.c_int64 * len(values))(*values)


def create_tensor(t: torch.Tensor, fmt: int = ACL_FORMAT_ND, dtype: Optional[int] = None) -> int:
    """aclCreateTensor over a torch tensor's view (dims, strides, device address).  The caller destroys it."""
    dims = list(t.shape)
    strides = list(t.stride())
    code = _DTYPES[t.dtype] if dtype is None else dtype
    h = _lib.lib().aclCreateTensor(_i64(dims), len(dims), code, _i64(strides), 0, fmt, _i64(dims), len(dims),
                                   C.c_void_p(t.data_ptr()))
    if not h:
        raise MemoryError("aclCreateTensor returned null")
    return h


def create_tensor_list(tensors: Sequence[torch.Tensor]) -> int:
    """aclCreateTensorList; the list owns its tensor handles (aclDestroyTensorList frees them)."""
    hs = [create_tensor(t) for t in tensors]
    arr = (C.c_void_p * len(hs))(*hs)
    h = _lib.lib().aclCreateTensorList(arr, len(hs))
    if not h:
        raise MemoryError("aclCreateTensorList returned null")
    return h


class _Workspace:
    """One growing device buffer per device, reused across calls like a framework's workspace pool."""

    def __init__(self):
        self._buf = {}

    def get(self, device: torch.device, nbytes: int) -> Optional[torch.Tensor]:
        if nbytes == 0:
            return None
        key = (device.type, device.index)
        b = self._buf.get(key)
        if b is None or b.numel() < nbytes:
            b = torch.empty(int(nbytes), dtype=torch.uint8, device=device)
            self._buf[key] = b
        return b


_WS = _Workspace()


def _stream_handle(stream) -> int:
    if stream is None:
        stream = torch.cuda.current_stream()
    return int(stream.cuda_stream)


def check_status(workspace: Optional[torch.Tensor], stream=None) -> None:
    """Synchronise the stream and raise if a kernel recorded a problem in the workspace status word."""
    rec = (C.c_int32 * 4)()
    ptr = C.c_void_p(workspace.data_ptr()) if workspace is not None else None
    size = workspace.numel() if workspace is not None else 0
    rc = _lib.lib().gmmB200CheckStatus(ptr, size, C.c_void_p(_stream_handle(stream)), rec)
    if rc != ACLNN_SUCCESS:
        raise AclnnError(rc, "gmmB200CheckStatus")


def grouped_matmul_v4(x: torch.Tensor, weight: torch.Tensor, scale: Optional[torch.Tensor],
                      per_token_scale: Optional[torch.Tensor], group_list: torch.Tensor, *,
                      bias: Optional[torch.Tensor] = None, split_item: int = 3, group_type: int = 0,
                      group_list_type: int = 0, act_type: int = 0, out: Optional[torch.Tensor] = None,
                      out_dtype: torch.dtype = torch.bfloat16, stream=None, workspace: Optional[torch.Tensor] = None,
                      return_workspace: bool = False, out_row_index: Optional[torch.Tensor] = None,
                      out_peers: Optional[Sequence[int]] = None):
    """y = bf16((x @ weight[e]) * scale[e] * per_token_scale) per expert row range (W8A8), or the raw int32
    accumulators when ``out_dtype`` is torch.int32.  Rows not covered by ``group_list`` keep their contents.
    ``out_row_index`` (int64 [M], an extension of this library) scatters result row r to row out_row_index[r]; it
    goes through the flat entry point gmmB200GroupedMatmulW8A8."""
    L = _lib.lib()
    if out is None and not out_peers:
        out = torch.empty((x.shape[0], weight.shape[2]), dtype=out_dtype, device=x.device)
    if out_row_index is not None:
        return _grouped_matmul_flat(x, weight, scale, per_token_scale, group_list, bias, group_list_type, act_type, out,
                                    out_row_index, stream, workspace, return_workspace, out_peers)
    lists = []
    try:
        hx = create_tensor_list([x]); lists.append(hx)
        hw = create_tensor_list([weight]); lists.append(hw)
        hb = None
        if bias is not None:
            hb = create_tensor_list([bias]); lists.append(hb)
        hs = None
        if scale is not None:
            hs = create_tensor_list([scale]); lists.append(hs)
        hp = None
        if per_token_scale is not None:
            hp = create_tensor_list([per_token_scale]); lists.append(hp)
        hy = create_tensor_list([out]); lists.append(hy)
        hg = create_tensor(group_list)
        try:
            ws_size = C.c_uint64(0)
            ex = C.c_void_p(0)
            rc = L.aclnnGroupedMatmulV4GetWorkspaceSize(hx, hw, hb, hs, None, None, None, hp, hg, None, None, None,
                                                        split_item, group_type, group_list_type, act_type, hy, None, None,
                                                        C.byref(ws_size), C.byref(ex))
            if rc != ACLNN_SUCCESS:
                raise AclnnError(rc, "aclnnGroupedMatmulV4GetWorkspaceSize")
            if workspace is None:
                workspace = _WS.get(x.device, ws_size.value)
            elif workspace.numel() < ws_size.value:
                L.aclDestroyAclOpExecutor(ex)
                raise ValueError(f"workspace of {workspace.numel()} bytes is smaller than the {ws_size.value} required")
            wptr = C.c_void_p(workspace.data_ptr()) if workspace is not None else None
            rc = L.aclnnGroupedMatmulV4(wptr, ws_size.value, ex, C.c_void_p(_stream_handle(stream)))
            if rc != ACLNN_SUCCESS:
                raise AclnnError(rc, "aclnnGroupedMatmulV4")
        finally:
            L.aclDestroyTensor(hg)
    finally:
        for h in lists:
            L.aclDestroyTensorList(h)
    return (out, workspace) if return_workspace else out


def _grouped_matmul_flat(x, weight, scale, per_token_scale, group_list, bias, group_list_type, act_type, out, out_row_index,
                         stream, workspace, return_workspace, out_peers=None):
    """Flat entry point.  ``out_peers`` (device addresses, one [rows, N] bf16 buffer per GPU) makes out_row_index hold
    (gpu << 40) | row; ``out`` may then be None."""
    L = _lib.lib()
    M, K = x.shape
    E, _, N = weight.shape
    trans = (not weight.is_contiguous()) and weight.transpose(1, 2).is_contiguous()
    for t in (x, scale, per_token_scale, group_list, bias, out, out_row_index):
        if t is not None and not t.is_contiguous():
            raise ValueError("the flat entry point needs contiguous tensors")
    if out_row_index.dtype != torch.int64 or out_row_index.numel() != M:
        raise ValueError("out_row_index must be int64 [M]")
    ydt = _DTYPES[out.dtype] if out is not None else ACL_BF16
    n_peers = len(out_peers) if out_peers else 0
    peers = (C.c_void_p * max(n_peers, 1))(*[C.c_void_p(a) for a in (out_peers or [])])
    size = C.c_uint64(0)
    rc = L.gmmB200GroupedMatmulW8A8WorkspaceSize(M, K, N, E, ydt, C.byref(size))
    if rc != ACLNN_SUCCESS:
        raise AclnnError(rc, "gmmB200GroupedMatmulW8A8WorkspaceSize")
    if workspace is None:
        workspace = _WS.get(x.device, size.value)
    p = lambda t: C.c_void_p(t.data_ptr()) if t is not None else None  # noqa: E731
    rc = L.gmmB200GroupedMatmulW8A8(p(x), p(weight), p(scale), _DTYPES[scale.dtype] if scale is not None else 0, p(per_token_scale),
                                    p(bias), _DTYPES[bias.dtype] if bias is not None else 0, p(group_list), group_list.numel(),
                                    group_list_type, M, K, N, E, int(trans), act_type, p(out_row_index), peers if n_peers else None, n_peers, p(out), ydt, p(workspace),
                                    workspace.numel(), C.c_void_p(_stream_handle(stream)))
    if rc != ACLNN_SUCCESS:
        raise AclnnError(rc, "gmmB200GroupedMatmulW8A8")
    return (out, workspace) if return_workspace else out


def grouped_matmul_swiglu_quant(x: torch.Tensor, weight: torch.Tensor, weight_scale: torch.Tensor, x_scale: torch.Tensor,
                                group_list: torch.Tensor, *, bias: Optional[torch.Tensor] = None,
                                offset: Optional[torch.Tensor] = None, output: Optional[torch.Tensor] = None,
                                output_scale: Optional[torch.Tensor] = None, stream=None,
                                workspace: Optional[torch.Tensor] = None, return_workspace: bool = False):
    """(output int8 [M, N/2], output_scale fp32 [M]) = per-token int8 requant of SwiGLU of the dequantised grouped
    GEMM.  ``group_list`` holds running totals.  Rows at and beyond group_list[-1] keep their contents."""
    L = _lib.lib()
    M = x.shape[0]
    N = weight_scale.shape[1] if weight_scale.dim() == 2 else 0
    if output is None:
        output = torch.empty((M, N // 2), dtype=torch.int8, device=x.device)
    if output_scale is None:
        output_scale = torch.empty((M,), dtype=torch.float32, device=x.device)
    handles = []
    try:
        def mk(t):
            if t is None:
                return None
            h = create_tensor(t)
            handles.append(h)
            return h
        hx, hw, hb, ho = mk(x), mk(weight), mk(bias), mk(offset)
        hws, hxs, hg, hq, hqs = mk(weight_scale), mk(x_scale), mk(group_list), mk(output), mk(output_scale)
        ws_size = C.c_uint64(0)
        ex = C.c_void_p(0)
        rc = L.aclnnGroupedMatmulSwigluQuantGetWorkspaceSize(hx, hw, hb, ho, hws, hxs, hg, hq, hqs, None, C.byref(ws_size),
                                                             C.byref(ex))
        if rc != ACLNN_SUCCESS:
            raise AclnnError(rc, "aclnnGroupedMatmulSwigluQuantGetWorkspaceSize")
        if workspace is None:
            workspace = _WS.get(x.device, ws_size.value)
        elif workspace.numel() < ws_size.value:
            L.aclDestroyAclOpExecutor(ex)
            raise ValueError(f"workspace of {workspace.numel()} bytes is smaller than the {ws_size.value} required")
        wptr = C.c_void_p(workspace.data_ptr()) if workspace is not None else None
        rc = L.aclnnGroupedMatmulSwigluQuant(wptr, ws_size.value, ex, C.c_void_p(_stream_handle(stream)))
        if rc != ACLNN_SUCCESS:
            raise AclnnError(rc, "aclnnGroupedMatmulSwigluQuant")
    finally:
        for h in handles:
            L.aclDestroyTensor(h)
    return (output, output_scale, workspace) if return_workspace else (output, output_scale)
