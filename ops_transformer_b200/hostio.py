"""Host-resident activations: the grouped operators with the row tensors in pinned host memory.

A caller whose token rows live in host memory pays PCIe for them on every call; the operator itself is 5-10 times
shorter than the copies.  ``HostPipelinedGroupedOp`` splits the call by experts (groups are independent: contiguous rows,
their own weight slice) and runs the pieces as a three-stage pipeline on three streams - host-to-device copy of piece
i+1, the operator on piece i, device-to-host copy of the results of piece i-1 - so that both directions of the link and
the GPU work at the same time.  Every piece goes through the same aclnn two-phase entry points as a whole call
(``acl.grouped_matmul_swiglu_quant`` / ``acl.grouped_matmul_v4``); weights and scales stay resident on the device.

Rows not covered by ``group_list`` are neither copied nor written (the operators leave them untouched as well).
"""
from __future__ import annotations

from typing import Optional

import numpy as np
import torch

import ctypes as C

from . import _lib, acl


class HostPipelinedGroupedOp:
    """``op``: "swiglu_quant" (outputs int8 [M, N/2] + fp32 [M]) or "gmm" (bf16 [M, N])."""

    def __init__(self, op: str, weight: torch.Tensor, weight_scale: torch.Tensor, max_rows: int, pieces: int = 4):
        if op not in ("swiglu_quant", "gmm"):
            raise ValueError(op)
        self.op = op
        self.w, self.ws = weight, weight_scale
        self.dev = weight.device
        if weight.dim() == 5:   # FRACTAL_NZ [E, N/32, K/16, 16, 32] (acl.format_cast_nz); pieces slice it by experts all the same
            self.E, self.N, self.K = int(weight.shape[0]), int(weight.shape[1]) * 32, int(weight.shape[2]) * 16
            self.wkw = {"weight_format": _lib.ACL_FORMAT_FRACTAL_NZ}
        else:
            self.E, self.K, self.N = (int(v) for v in weight.shape)
            self.wkw = {}
        self.pieces = max(1, min(pieces, self.E))
        self.s_in, self.s_op, self.s_out = (torch.cuda.Stream(self.dev) for _ in range(3))
        self.dx = torch.empty((max_rows, self.K), dtype=torch.int8, device=self.dev)
        self.dxs = torch.empty((max_rows,), dtype=torch.float32, device=self.dev)
        self.dgl = torch.empty((self.E,), dtype=torch.int64, device=self.dev)
        self.hgl = torch.empty((self.E,), dtype=torch.int64).pin_memory()
        if op == "swiglu_quant":
            self.out0 = torch.empty((max_rows, self.N // 2), dtype=torch.int8, device=self.dev)
            self.out1 = torch.empty((max_rows,), dtype=torch.float32, device=self.dev)
        else:
            self.out0 = torch.empty((max_rows, self.N), dtype=torch.bfloat16, device=self.dev)
            self.out1 = None
        # one workspace sized for a call over all rows serves every piece (the pieces run in order on one stream)
        size = C.c_uint64(0)
        L = _lib.lib()
        if op == "swiglu_quant":
            rc = L.gmmB200GroupedMatmulSwigluQuantWorkspaceSize(max_rows, self.K, self.N, self.E, C.byref(size))
        else:
            rc = L.gmmB200GroupedMatmulW8A8WorkspaceSize(max_rows, self.K, self.N, self.E, _lib.ACL_BF16, C.byref(size))
        if rc != 0:
            raise acl.AclnnError(rc, "workspace size")
        self.workspace = torch.empty(int(size.value) + 4096, dtype=torch.uint8, device=self.dev)

    def run(self, x_host: torch.Tensor, x_scale_host: torch.Tensor, counts: np.ndarray, out0_host: torch.Tensor,
            out1_host: Optional[torch.Tensor] = None) -> None:
        """x_host int8 [M, K], x_scale_host fp32 [M], outputs: pinned host tensors.  ``counts``: rows per expert (host).
        Returns when the results are in the host tensors."""
        counts = np.asarray(counts, np.int64)
        E = self.E
        bounds = [round(i * E / self.pieces) for i in range(self.pieces + 1)]
        starts = np.concatenate([[0], np.cumsum(counts)])
        # per-piece running totals, rebased to the piece's first row, uploaded in one small copy
        for p in range(self.pieces):
            e0, e1 = bounds[p], bounds[p + 1]
            self.hgl[e0:e1] = torch.from_numpy(np.cumsum(counts[e0:e1]))
        cur = torch.cuda.current_stream(self.dev)
        for s in (self.s_in, self.s_op, self.s_out):
            s.wait_stream(cur)
        with torch.cuda.stream(self.s_in):
            self.dgl.copy_(self.hgl, non_blocking=True)
        for p in range(self.pieces):
            e0, e1 = bounds[p], bounds[p + 1]
            r0, r1 = int(starts[e0]), int(starts[e1])
            if r1 == r0:
                continue
            with torch.cuda.stream(self.s_in):
                self.dx[r0:r1].copy_(x_host[r0:r1], non_blocking=True)
                self.dxs[r0:r1].copy_(x_scale_host[r0:r1], non_blocking=True)
                ev_in = torch.cuda.Event()
                ev_in.record(self.s_in)
            with torch.cuda.stream(self.s_op):
                self.s_op.wait_event(ev_in)
                if self.op == "swiglu_quant":
                    acl.grouped_matmul_swiglu_quant(
                        self.dx[r0:r1], self.w[e0:e1], self.ws[e0:e1], self.dxs[r0:r1], self.dgl[e0:e1], output=self.out0[r0:r1],
                        output_scale=self.out1[r0:r1], stream=self.s_op, workspace=self.workspace, **self.wkw)
                else:
                    acl.grouped_matmul_v4(
                        self.dx[r0:r1], self.w[e0:e1], self.ws[e0:e1], self.dxs[r0:r1], self.dgl[e0:e1], out=self.out0[r0:r1],
                        stream=self.s_op, workspace=self.workspace, **self.wkw)
                ev_op = torch.cuda.Event()
                ev_op.record(self.s_op)
            with torch.cuda.stream(self.s_out):
                self.s_out.wait_event(ev_op)
                out0_host[r0:r1].copy_(self.out0[r0:r1], non_blocking=True)
                if self.out1 is not None and out1_host is not None:
                    out1_host[r0:r1].copy_(self.out1[r0:r1], non_blocking=True)
        self.s_out.synchronize()
        self.s_op.synchronize()
