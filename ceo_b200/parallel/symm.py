"""Peer-mapped ("symmetric") device buffers for in-kernel collectives.

Each rank allocates the same-sized buffer with a plain ``cudaMalloc`` (through the kernel
library, outside PyTorch's caching allocator so the allocation is a whole IPC-exportable
block), publishes its CUDA IPC handle through the process group, and opens every peer's
handle.  The result is, on every rank, a list of ``world`` device pointers - this rank's own
memory and its peers' memory over NVLink - that kernels take as a pointer table.

The reference only wraps ``cudaDeviceEnablePeerAccess`` and never calls it
(src/runtime/cuda.zig:519-527, src/runtime/main.zig:310-318).
"""
from __future__ import annotations

import ctypes

import torch
import torch.distributed as dist

from ..ops import _lib

_DT = {torch.float32: "<f4", torch.bfloat16: None, torch.int32: "<i4", torch.uint8: "|u1"}


class _RawCuda:
    """Exposes a raw device allocation to torch through ``__cuda_array_interface__``."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1",
                                         "data": (ptr, False), "version": 3, "strides": None}


class SymmetricBuffer:
    """``nbytes`` of device memory on every rank of ``group``, mapped on all of them."""

    def __init__(self, nbytes: int, group=None, zero: bool = True):
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.nbytes = (nbytes + 255) // 256 * 256
        L = _lib.lib()
        out = ctypes.c_void_p()
        _lib.check(L.ceo_dev_malloc(ctypes.byref(out), self.nbytes), "ceo_dev_malloc")
        self.local_ptr = out.value
        self._raw = _RawCuda(self.local_ptr, self.nbytes)
        self.bytes = torch.as_tensor(self._raw, device=torch.device("cuda",
                                                                     torch.cuda.current_device()))
        if zero:
            self.bytes.zero_()
        torch.cuda.synchronize()
        self.ptrs = [self.local_ptr]
        self._opened = []
        if self.world > 1:
            h = ctypes.create_string_buffer(64)
            _lib.check(L.ceo_ipc_get_handle(self.local_ptr, h), "ceo_ipc_get_handle")
            handles = [None] * self.world
            dist.all_gather_object(handles, bytes(h.raw), group=group)
            self.ptrs = []
            for r, hb in enumerate(handles):
                if r == self.rank:
                    self.ptrs.append(self.local_ptr)
                    continue
                p = ctypes.c_void_p()
                _lib.check(L.ceo_ipc_open(ctypes.create_string_buffer(hb, 64), ctypes.byref(p)),
                           "ceo_ipc_open")
                self.ptrs.append(p.value)
                self._opened.append(p.value)
            dist.barrier(group=group)
        self._table = (ctypes.c_void_p * 8)(*([p for p in self.ptrs] + [None] * (8 - self.world)))

    def table(self, byte_offset: int = 0):
        """ctypes array of the per-rank pointers (optionally offset) for a kernel call."""
        if byte_offset == 0:
            return self._table
        return (ctypes.c_void_p * 8)(*([p + byte_offset for p in self.ptrs] +
                                       [None] * (8 - self.world)))

    def view(self, dtype: torch.dtype, numel: int, byte_offset: int = 0) -> torch.Tensor:
        """A typed tensor over this rank's local part of the buffer."""
        nb = numel * torch.empty((), dtype=dtype).element_size()
        assert byte_offset % 16 == 0 and byte_offset + nb <= self.nbytes
        return self.bytes[byte_offset:byte_offset + nb].view(dtype)

    def close(self):
        L = _lib.lib()
        for p in self._opened:
            L.ceo_ipc_close(p)
        self._opened = []
        if self.local_ptr:
            self.bytes = None
            torch.cuda.synchronize()
            L.ceo_dev_free(self.local_ptr)
            self.local_ptr = None
