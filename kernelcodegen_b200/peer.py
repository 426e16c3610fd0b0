"""Peer-visible device buffers for the fused all-gather of C (one process per GPU, one node).

Every rank allocates its full C buffer through `kcg_peer_alloc`, the 64-byte handles travel
over `torch.distributed` (any backend: they are plain bytes), and each rank maps the others'
buffers with `kcg_peer_open`.  The GEMM epilogue then stores each finished tile into the local
buffer and into every peer's buffer (plain unicast stores over NVLink; no collective
kernel), so that when all ranks' kernels have finished every rank holds the whole of C.
"""
from __future__ import annotations

import ctypes
from typing import List

import torch
import torch.distributed as dist

from . import capi


class _CudaBuffer:
    """Exposes a raw device allocation to torch through __cuda_array_interface__."""

    def __init__(self, ptr: int, shape, typestr: str):
        self.__cuda_array_interface__ = {"shape": tuple(shape), "typestr": typestr, "data": (ptr, False), "version": 3,
                                         "strides": None}


class PeerMatrix:
    """A [rows, cols] bf16 or f32 matrix on this rank's GPU that the other ranks can store into."""

    def __init__(self, rows: int, cols: int, dtype: torch.dtype, device: torch.device, group=None):
        self.lib = capi.load()
        self.group = group
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rows, self.cols, self.dtype, self.device = rows, cols, dtype, device
        self.itemsize = torch.empty((), dtype=dtype).element_size()
        nbytes = rows * cols * self.itemsize
        ptr = ctypes.c_void_p()
        handle = ctypes.create_string_buffer(64)
        with torch.cuda.device(device):
            capi.check(self.lib.kcg_peer_alloc(nbytes, ctypes.byref(ptr), handle), "kcg_peer_alloc")
        self.ptr = ptr.value
        # torch views the same memory; bf16 has no array-interface typestr, so view through int16
        if dtype == torch.bfloat16:
            raw = torch.as_tensor(_CudaBuffer(self.ptr, (rows, cols), "<i2"), device=device)
            self.tensor = raw.view(torch.bfloat16)
        else:
            self.tensor = torch.as_tensor(_CudaBuffer(self.ptr, (rows, cols), "<f4"), device=device)
        self.peer_ptrs: List[int] = []      # base pointers of the other ranks' buffers, rank order rotated
        self._opened: List[int] = []
        if self.world > 1:
            handles = [None] * self.world
            dist.all_gather_object(handles, bytes(handle.raw), group=group)
            for step in range(1, self.world):
                peer = (self.rank + step) % self.world
                out = ctypes.c_void_p()
                hb = ctypes.create_string_buffer(handles[peer], 64)
                with torch.cuda.device(device):
                    capi.check(self.lib.kcg_peer_open(hb, ctypes.byref(out)), "kcg_peer_open")
                self.peer_ptrs.append(out.value)
                self._opened.append(out.value)

    def peer_row_ptrs(self, row_lo: int) -> List[int]:
        """Peers' addresses of row `row_lo` (where this rank's row block lands in their copies)."""
        off = row_lo * self.cols * self.itemsize
        return [p + off for p in self.peer_ptrs]

    def close(self) -> None:
        torch.cuda.synchronize(self.device)
        if dist.is_initialized() and self.world > 1:
            dist.barrier(group=self.group)  # nobody unmaps while a peer may still store
        for p in self._opened:
            self.lib.kcg_peer_close(p)
        self._opened = []
        if dist.is_initialized() and self.world > 1:
            dist.barrier(group=self.group)
        if self.ptr:
            self.tensor = None
            self.lib.kcg_peer_free(self.ptr)
            self.ptr = 0
