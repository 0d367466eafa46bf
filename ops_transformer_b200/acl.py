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
from ._lib import LaunchOptions  # noqa: F401  (re-exported: the per-call options of include/gmm_b200.h)
from ._lib import (ACL_BF16, ACL_FLOAT, ACL_FLOAT16, ACL_FORMAT_FRACTAL_NZ, ACL_FORMAT_ND, ACL_INT8, ACL_INT32, ACL_INT64,
                   ACLNN_SUCCESS)

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


def create_tensor(t: torch.Tensor, fmt: int = ACL_FORMAT_ND, dtype: Optional[int] = None,
                  view_dims: Optional[Sequence[int]] = None) -> int:
    """aclCreateTensor over a torch tensor's view (dims, strides, device address).  The caller destroys it.
    ``view_dims``: the tensor is the storage (its shape becomes the storage shape) and is viewed with these dimensions,
    as a FRACTAL_NZ weight is: storage [E, N/32, K/16, 16, 32], view [E, K, N]."""
    storage = list(t.shape)
    if view_dims is None:
        dims, strides = storage, list(t.stride())
    else:
        dims = list(view_dims)
        strides = [1] * len(dims)
        for i in range(len(dims) - 2, -1, -1):
            strides[i] = strides[i + 1] * dims[i + 1]
    code = _DTYPES[t.dtype] if dtype is None else dtype
    h = _lib.lib().aclCreateTensor(_i64(dims), len(dims), code, _i64(strides), 0, fmt, _i64(storage), len(storage),
                                   C.c_void_p(t.data_ptr()))
    if not h:
        raise MemoryError("aclCreateTensor returned null")
    return h


def format_cast_nz(weight: torch.Tensor) -> torch.Tensor:
    """int8 [E, K, N] -> the FRACTAL_NZ storage [E, N/32, K/16, 16, 32] (a copy; K % 16 == 0, N % 32 == 0): element
    (k, n) moves to [n // 32, k // 16, k % 16, n % 32].  What a caller of the reference does once per weight with its
    framework's format cast before calling the WeightNZ operators; a set-up step, not part of the hot path."""
    E, K, N = weight.shape
    if K % 16 or N % 32:
        raise ValueError("FRACTAL_NZ needs K % 16 == 0 and N % 32 == 0")
    return weight.reshape(E, K // 16, 16, N // 32, 32).permute(0, 3, 1, 2, 4).contiguous()


def create_tensor_list(tensors: Sequence[torch.Tensor], fmt: int = ACL_FORMAT_ND) -> int:
    """aclCreateTensorList; the list owns its tensor handles (aclDestroyTensorList frees them)."""
    hs = [create_tensor(t, fmt) for t in tensors]
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
        err = AclnnError(rc, "gmmB200CheckStatus")
        err.record = tuple(int(v) for v in rec)   # (code, CTA, waiting role, detail)
        raise err


def _apply_options(executor, options: Optional[LaunchOptions], where: str) -> None:
    """Attach per-call options to a live executor (between the two phases)."""
    if options is None:
        return
    rc = _lib.lib().gmmB200SetExecutorOptions(executor, C.byref(options))
    if rc != ACLNN_SUCCESS:
        _lib.lib().aclDestroyAclOpExecutor(executor)
        raise AclnnError(rc, where + ": gmmB200SetExecutorOptions")


def grouped_matmul_v4(x: torch.Tensor, weight: torch.Tensor, scale: Optional[torch.Tensor],
                      per_token_scale: Optional[torch.Tensor], group_list: torch.Tensor, *,
                      bias: Optional[torch.Tensor] = None, split_item: int = 3, group_type: int = 0,
                      group_list_type: int = 0, act_type: int = 0, out: Optional[torch.Tensor] = None,
                      out_dtype: torch.dtype = torch.bfloat16, stream=None, workspace: Optional[torch.Tensor] = None,
                      return_workspace: bool = False, out_row_index: Optional[torch.Tensor] = None,
                      out_peers: Optional[Sequence[int]] = None, weight_format: int = ACL_FORMAT_ND,
                      api: str = "V4", tuning_config: Optional[Sequence[int]] = None, quant_group_size: int = 0,
                      options: Optional[LaunchOptions] = None, out_rows: int = 0):
    """y = bf16(act((x @ weight[e]) * scale[e] * per_token_scale)) per expert row range (W8A8), a float16 result with
    ``out_dtype`` torch.float16, or the raw int32 accumulators with torch.int32.  Rows not covered by ``group_list``
    keep their contents.  ``weight_format`` ACL_FORMAT_FRACTAL_NZ: ``weight`` is the 5-D storage of ``format_cast_nz``.
    ``api`` picks the entry point: "V4", "V5" (adds ``tuning_config``) or "WeightNz" (adds ``quant_group_size`` and
    treats the weight as FRACTAL_NZ) - aclnn_grouped_matmul_v5.h:49-58, aclnn_grouped_matmul_weight_nz.h:50-59 of the
    reference.  ``out_row_index`` (int64 [M], an extension of this library) scatters result row r to row
    out_row_index[r]; it goes through the flat entry point gmmB200GroupedMatmulW8A8.  ``options``: per-call
    ``LaunchOptions`` (CTA cap, timing events)."""
    L = _lib.lib()
    nz = weight_format == ACL_FORMAT_FRACTAL_NZ or api == "WeightNz"
    if out is None and not out_peers:
        n_out = weight.shape[1] * 32 if (nz and weight.dim() == 5) else weight.shape[2]
        out = torch.empty((x.shape[0], n_out), dtype=out_dtype, device=x.device)
    if out_row_index is not None:
        return _grouped_matmul_flat(x, weight, scale, per_token_scale, group_list, bias, group_list_type, act_type, out,
                                    out_row_index, stream, workspace, return_workspace, out_peers, nz, options, out_rows)
    lists = []
    tuning = None
    try:
        hx = create_tensor_list([x]); lists.append(hx)
        hw = create_tensor_list([weight], ACL_FORMAT_FRACTAL_NZ if nz else ACL_FORMAT_ND); lists.append(hw)
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
            if tuning_config is not None:
                tuning = L.aclCreateIntArray(_i64(list(tuning_config)), len(tuning_config))
            head = (hx, hw, hb, hs, None, None, None, hp, hg, None, None, None, split_item, group_type, group_list_type, act_type)
            tail = (hy, None, None, C.byref(ws_size), C.byref(ex))
            if api == "V4":
                rc = L.aclnnGroupedMatmulV4GetWorkspaceSize(*head, *tail)
            elif api == "V5":
                rc = L.aclnnGroupedMatmulV5GetWorkspaceSize(*head, tuning, *tail)
            elif api == "WeightNz":
                rc = L.aclnnGroupedMatmulWeightNzGetWorkspaceSize(*head, tuning, quant_group_size, *tail)
            else:
                raise ValueError(f"unknown api {api!r}")
            if rc != ACLNN_SUCCESS:
                raise AclnnError(rc, f"aclnnGroupedMatmul{api}GetWorkspaceSize")
            if workspace is None:
                workspace = _WS.get(x.device, ws_size.value)
            elif workspace.numel() < ws_size.value:
                L.aclDestroyAclOpExecutor(ex)
                raise ValueError(f"workspace of {workspace.numel()} bytes is smaller than the {ws_size.value} required")
            wptr = C.c_void_p(workspace.data_ptr()) if workspace is not None else None
            _apply_options(ex, options, "aclnnGroupedMatmul" + api)
            rc = getattr(L, "aclnnGroupedMatmul" + api)(wptr, ws_size.value, ex, C.c_void_p(_stream_handle(stream)))
            if rc != ACLNN_SUCCESS:
                raise AclnnError(rc, "aclnnGroupedMatmul" + api)
        finally:
            L.aclDestroyTensor(hg)
            if tuning:
                L.aclDestroyIntArray(tuning)
    finally:
        for h in lists:
            L.aclDestroyTensorList(h)
    return (out, workspace) if return_workspace else out


def _grouped_matmul_flat(x, weight, scale, per_token_scale, group_list, bias, group_list_type, act_type, out, out_row_index,
                         stream, workspace, return_workspace, out_peers=None, nz=False, options=None, out_rows=0):
    """Flat entry point.  ``out_peers`` (device addresses, one [rows, N] bf16 buffer per GPU) makes out_row_index hold
    (gpu << 40) | row; ``out`` may then be None.  ``out_rows``: rows of ``out`` / of every peer buffer (0 = taken from
    ``out``, unbounded without it); rows scattered outside are skipped and reported by ``check_status``."""
    L = _lib.lib()
    M, K = x.shape
    if nz and weight.dim() == 5:
        E, N = weight.shape[0], weight.shape[1] * 32
    else:
        E, _, N = weight.shape
    trans = 2 if nz else int((not weight.is_contiguous()) and weight.transpose(1, 2).is_contiguous())
    for t in (x, scale, per_token_scale, group_list, bias, out, out_row_index):
        if t is not None and not t.is_contiguous():
            raise ValueError("the flat entry point needs contiguous tensors")
    if out_row_index.dtype != torch.int64 or out_row_index.numel() != M:
        raise ValueError("out_row_index must be int64 [M]")
    ydt = _DTYPES[out.dtype] if out is not None else ACL_BF16
    if not out_rows and out is not None:
        out_rows = out.shape[0]
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
                                    group_list_type, M, K, N, E, trans, act_type, p(out_row_index), peers if n_peers else None, n_peers, out_rows, p(out), ydt, p(workspace),
                                    workspace.numel(), C.c_void_p(_stream_handle(stream)), C.byref(options) if options is not None else None)
    if rc != ACLNN_SUCCESS:
        raise AclnnError(rc, "gmmB200GroupedMatmulW8A8")
    return (out, workspace) if return_workspace else out


def grouped_matmul_swiglu_quant(x: torch.Tensor, weight: torch.Tensor, weight_scale: torch.Tensor, x_scale: torch.Tensor,
                                group_list: torch.Tensor, *, bias: Optional[torch.Tensor] = None,
                                offset: Optional[torch.Tensor] = None, output: Optional[torch.Tensor] = None,
                                output_scale: Optional[torch.Tensor] = None, stream=None,
                                workspace: Optional[torch.Tensor] = None, return_workspace: bool = False,
                                weight_format: int = ACL_FORMAT_ND, api: str = "", options: Optional[LaunchOptions] = None):
    """(output int8 [M, N/2], output_scale fp32 [M]) = per-token int8 requant of SwiGLU of the dequantised grouped
    GEMM.  ``group_list`` holds running totals.  Rows at and beyond group_list[-1] keep their contents.
    ``weight_format`` ACL_FORMAT_FRACTAL_NZ: ``weight`` is the 5-D storage of ``format_cast_nz``; ``api`` "WeightNZ"
    calls aclnnGroupedMatmulSwigluQuantWeightNZ (aclnn_grouped_matmul_swiglu_quant_weight_nz.h:37-54 of the reference),
    which takes the storage as FRACTAL_NZ whatever the format says."""
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
        hx, hb, ho = mk(x), mk(bias), mk(offset)
        hw = create_tensor(weight, weight_format)
        handles.append(hw)
        hws, hxs, hg, hq, hqs = mk(weight_scale), mk(x_scale), mk(group_list), mk(output), mk(output_scale)
        ws_size = C.c_uint64(0)
        ex = C.c_void_p(0)
        name = "aclnnGroupedMatmulSwigluQuant" + api
        rc = getattr(L, name + "GetWorkspaceSize")(hx, hw, hb, ho, hws, hxs, hg, hq, hqs, None, C.byref(ws_size), C.byref(ex))
        if rc != ACLNN_SUCCESS:
            raise AclnnError(rc, name + "GetWorkspaceSize")
        if workspace is None:
            workspace = _WS.get(x.device, ws_size.value)
        elif workspace.numel() < ws_size.value:
            L.aclDestroyAclOpExecutor(ex)
            raise ValueError(f"workspace of {workspace.numel()} bytes is smaller than the {ws_size.value} required")
        wptr = C.c_void_p(workspace.data_ptr()) if workspace is not None else None
        _apply_options(ex, options, name)
        rc = getattr(L, name)(wptr, ws_size.value, ex, C.c_void_p(_stream_handle(stream)))
        if rc != ACLNN_SUCCESS:
            raise AclnnError(rc, name)
    finally:
        for h in handles:
            L.aclDestroyTensor(h)
    return (output, output_scale, workspace) if return_workspace else (output, output_scale)


def grouped_matmul_finalize_routing(x: torch.Tensor, weight_nz: torch.Tensor, scale: torch.Tensor, group_list: torch.Tensor,
                                    row_index: torch.Tensor, batch: int, *, bias: Optional[torch.Tensor] = None,
                                    pertoken_scale: Optional[torch.Tensor] = None, shared_input: Optional[torch.Tensor] = None,
                                    logit: Optional[torch.Tensor] = None, shared_input_weight: float = 1.0,
                                    shared_input_offset: int = 0, group_list_type: int = 1, out: Optional[torch.Tensor] = None,
                                    view_3d: bool = True, api: str = "", tuning_config: Optional[Sequence[int]] = None,
                                    stream=None, workspace: Optional[torch.Tensor] = None, return_workspace: bool = False,
                                    options: Optional[LaunchOptions] = None):
    """aclnnGroupedMatmulFinalizeRoutingWeightNz (``api`` "") or ...WeightNzV2 (``api`` "V2"): W8A8 grouped GEMM whose fp32
    result rows, weighted by ``logit``, are added into row ``row_index[i]`` of ``out`` [batch, N] on top of the weighted
    ``shared_input`` rows (gmm/grouped_matmul_finalize_routing/op_host/op_api/aclnn_grouped_matmul_finalize_routing_weight_nz.h:48-64
    of the reference).  ``weight_nz`` is the FRACTAL_NZ storage [E, N/32, K/16, 16, 32] (``format_cast_nz``); with
    ``view_3d`` it is described to the operator as the reference's callers do, a view [E, K, N] over that storage."""
    L = _lib.lib()
    E, n1, k1 = weight_nz.shape[0], weight_nz.shape[1], weight_nz.shape[2]
    N, K = n1 * 32, k1 * 16
    if out is None:
        out = torch.empty((batch, N), dtype=torch.float32, device=x.device)
    handles = []
    tuning = None
    try:
        def mk(t, **kw):
            if t is None:
                return None
            h = create_tensor(t, **kw)
            handles.append(h)
            return h
        hx = mk(x)
        hw = mk(weight_nz, fmt=ACL_FORMAT_FRACTAL_NZ, view_dims=[E, K, N] if view_3d else None)
        hs, hb, hp, hg = mk(scale), mk(bias), mk(pertoken_scale), mk(group_list)
        hsh, hl, hr, hy = mk(shared_input), mk(logit), mk(row_index), mk(out)
        ws_size = C.c_uint64(0)
        ex = C.c_void_p(0)
        name = "aclnnGroupedMatmulFinalizeRoutingWeightNz" + api
        if api == "V2":
            if tuning_config is not None:
                tuning = L.aclCreateIntArray(_i64(list(tuning_config)), len(tuning_config))
            rc = L.aclnnGroupedMatmulFinalizeRoutingWeightNzV2GetWorkspaceSize(
                hx, hw, hs, hb, None, None, None, hp, hg, hsh, hl, hr, 0, shared_input_weight, shared_input_offset, False, False,
                group_list_type, tuning, hy, C.byref(ws_size), C.byref(ex))
        else:
            rc = L.aclnnGroupedMatmulFinalizeRoutingWeightNzGetWorkspaceSize(
                hx, hw, hs, hb, hp, hg, hsh, hl, hr, 0, shared_input_weight, shared_input_offset, False, False, group_list_type,
                hy, C.byref(ws_size), C.byref(ex))
        if rc != ACLNN_SUCCESS:
            raise AclnnError(rc, name + "GetWorkspaceSize")
        if workspace is None:
            workspace = _WS.get(x.device, ws_size.value)
        elif workspace.numel() < ws_size.value:
            L.aclDestroyAclOpExecutor(ex)
            raise ValueError(f"workspace of {workspace.numel()} bytes is smaller than the {ws_size.value} required")
        wptr = C.c_void_p(workspace.data_ptr()) if workspace is not None else None
        _apply_options(ex, options, name)
        rc = getattr(L, name)(wptr, ws_size.value, ex, C.c_void_p(_stream_handle(stream)))
        if rc != ACLNN_SUCCESS:
            raise AclnnError(rc, name)
    finally:
        for h in handles:
            L.aclDestroyTensor(h)
        if tuning:
            L.aclDestroyIntArray(tuning)
    return (out, workspace) if return_workspace else out


def grouped_matmul_finalize_routing_flat(x, weight, weight_layout, scale, group_list, row_index, out, *, bias=None,
                                         pertoken_scale=None, shared_input=None, logit=None, shared_input_weight=1.0,
                                         shared_input_offset=0, group_list_type=1, stream=None, workspace=None, options=None):
    """gmmB200GroupedMatmulFinalizeRouting: the same operator without handles; ``weight_layout`` 0 takes the ND [E, K, N]
    weight (the faster layout here), 2 the FRACTAL_NZ storage."""
    L = _lib.lib()
    M, K = x.shape
    if weight_layout == 2:
        E, N = weight.shape[0], weight.shape[1] * 32
    else:
        E, _, N = weight.shape
    if workspace is None:
        workspace = _WS.get(x.device, 256)
    p = lambda t: C.c_void_p(t.data_ptr()) if t is not None else None  # noqa: E731
    rc = L.gmmB200GroupedMatmulFinalizeRouting(
        p(x), p(weight), weight_layout, p(scale), _DTYPES[scale.dtype], p(bias), p(pertoken_scale), p(group_list),
        group_list.numel(), group_list_type, p(shared_input), 0 if shared_input is None else shared_input.shape[0],
        shared_input_offset, shared_input_weight, p(logit), p(row_index), _DTYPES[row_index.dtype], M, K, N, E, p(out),
        out.shape[0], p(workspace), workspace.numel(), C.c_void_p(_stream_handle(stream)),
        C.byref(options) if options is not None else None)
    if rc != ACLNN_SUCCESS:
        raise AclnnError(rc, "gmmB200GroupedMatmulFinalizeRouting")
    return out


def moe_init_routing_v3(x: torch.Tensor, expert_idx: torch.Tensor, *, expert_num: int, active_expert_range: Sequence[int],
                        quant_mode: int = 1, scale: Optional[torch.Tensor] = None, offset: Optional[torch.Tensor] = None,
                        active_num: Optional[int] = None, expert_capacity: int = 0, drop_pad_mode: int = 0,
                        expert_tokens_num_type: int = 1, expert_tokens_num_flag: bool = True, row_idx_type: int = 1,
                        outputs=None, stream=None, workspace: Optional[torch.Tensor] = None):
    """aclnnMoeInitRoutingV3 (moe/moe_init_routing_v3/op_host/op_api/aclnn_moe_init_routing_v3.h:24-47 of the reference):
    returns (expandedX, expandedRowIdx, expertTokensCountOrCumsum, expandedScale).  With ``quant_mode`` 1 expandedX is int8
    and expandedScale the per-row scale, i.e. the x / per-token scale of the grouped GEMM operators."""
    L = _lib.lib()
    n, h = x.shape
    k = expert_idx.shape[1]
    start, end = active_expert_range
    if outputs is None:
        ex = torch.empty((n * k, h), dtype=torch.int8 if quant_mode == 1 else x.dtype, device=x.device)
        ri = torch.empty((n * k,), dtype=torch.int32, device=x.device)
        cnt = torch.empty((end - start,) if expert_tokens_num_type == 1 else (expert_num, 2), dtype=torch.int64, device=x.device)
        es = torch.empty((n * k,), dtype=torch.float32, device=x.device)
    else:
        ex, ri, cnt, es = outputs
    handles = []
    rng = L.aclCreateIntArray(_i64(list(active_expert_range)), len(active_expert_range))
    try:
        def mk(t):
            if t is None:
                return None
            hh = create_tensor(t)
            handles.append(hh)
            return hh
        hx, hi, hs, ho, hex_, hri, hc, hes = (mk(t) for t in (x, expert_idx, scale, offset, ex, ri, cnt, es))
        ws_size = C.c_uint64(0)
        exr = C.c_void_p(0)
        rc = L.aclnnMoeInitRoutingV3GetWorkspaceSize(hx, hi, hs, ho, n * k if active_num is None else active_num, expert_capacity,
                                                     expert_num, drop_pad_mode, expert_tokens_num_type, expert_tokens_num_flag,
                                                     quant_mode, rng, row_idx_type, hex_, hri, hc, hes, C.byref(ws_size), C.byref(exr))
        if rc != ACLNN_SUCCESS:
            raise AclnnError(rc, "aclnnMoeInitRoutingV3GetWorkspaceSize")
        if workspace is None:
            workspace = _WS.get(x.device, ws_size.value)
        wptr = C.c_void_p(workspace.data_ptr()) if workspace is not None else None
        rc = L.aclnnMoeInitRoutingV3(wptr, ws_size.value, exr, C.c_void_p(_stream_handle(stream)))
        if rc != ACLNN_SUCCESS:
            raise AclnnError(rc, "aclnnMoeInitRoutingV3")
    finally:
        for hh in handles:
            L.aclDestroyTensor(hh)
        L.aclDestroyIntArray(rng)
    return ex, ri, cnt, es
