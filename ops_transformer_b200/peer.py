"""Device buffers that every rank of a single-node process group can write into.

Each rank allocates one buffer with the library's allocator, exports a CUDA IPC handle, and opens the handles of
all other ranks.  ``ptrs[r]`` is then the device address of rank r's buffer as seen from this process (the local one
for r == rank).  The memory behind ``ptrs[rank]`` can also be viewed as a torch tensor.
"""
from __future__ import annotations

import ctypes as C
from typing import List

import torch
import torch.distributed as dist

from . import _lib


class _RawCudaMemory:
    """Exposes raw device memory through __cuda_array_interface__ so that torch can wrap it without a copy."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3}


class PeerBuffer:
    def __init__(self, nbytes: int, group=None):
        L = _lib.lib()
        self.nbytes = int(nbytes)
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        p = C.c_void_p(0)
        if L.gmmB200PeerAlloc(self.nbytes, C.byref(p)) != 0:
            raise RuntimeError(_lib.last_error())
        self.local_ptr = int(p.value)
        self.ptrs: List[int] = [0] * self.world
        self.ptrs[self.rank] = self.local_ptr
        self._imported: List[int] = []
        if self.world > 1:
            handle = (C.c_ubyte * 64)()
            if L.gmmB200PeerExport(C.c_void_p(self.local_ptr), handle) != 0:
                raise RuntimeError(_lib.last_error())
            handles = [None] * self.world
            dist.all_gather_object(handles, bytes(handle), group=group)
            for r, h in enumerate(handles):
                if r == self.rank:
                    continue
                q = C.c_void_p(0)
                buf = (C.c_ubyte * 64).from_buffer_copy(h)
                if L.gmmB200PeerImport(buf, C.byref(q)) != 0:
                    raise RuntimeError(f"rank {self.rank}: cannot open rank {r}'s buffer: {_lib.last_error()}")
                self.ptrs[r] = int(q.value)
                self._imported.append(int(q.value))
        self._raw = _RawCudaMemory(self.local_ptr, self.nbytes)
        self.bytes_tensor = torch.as_tensor(self._raw, device=torch.device("cuda", torch.cuda.current_device()))

    def view(self, dtype: torch.dtype, shape) -> torch.Tensor:
        n = 1
        for d in shape:
            n *= int(d)
        nb = n * torch.empty((), dtype=dtype).element_size()
        return self.bytes_tensor[:nb].view(dtype).view(*shape)

    def ptr_array(self):
        return (C.c_void_p * self.world)(*[C.c_void_p(p) for p in self.ptrs])

    def close(self):
        L = _lib.lib()
        for p in self._imported:
            L.gmmB200PeerRelease(C.c_void_p(p))
        self._imported = []
        if self.local_ptr:
            self.bytes_tensor = None
            L.gmmB200PeerFree(C.c_void_p(self.local_ptr))
            self.local_ptr = 0
