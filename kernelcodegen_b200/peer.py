"""Peer-visible device buffers for the fused all-gather of C (one process per GPU, one node).

Every rank holds its own full copy of C.  The GEMM epilogue delivers each finished tile of this
rank's row block to all copies, and publishes a completion flag when the launch, and with it all
its stores, has finished; a consumer waits for the other ranks' flags with a bounded
device-side wait instead of a collective.  Two ways of making the copies reachable:

  "symmetric"  torch symmetric memory (CUDA virtual-memory handles exchanged by torch).  When the
               node's NVSwitch supports multicast, the allocation also has a multicast address:
               the epilogue then stores every 16 bytes once (`multimem.st`) and the switch
               replicates them to all ranks, instead of one store per rank.
  "ipc"        `kcg_peer_alloc` / `kcg_peer_open` (CUDA IPC handles, plain bytes that travel over
               torch.distributed): plain unicast stores to every peer.

Nothing here runs a collective on the data path.
"""
from __future__ import annotations

import ctypes
from typing import List, Optional

import torch
import torch.distributed as dist

from . import capi, ops, sharding

FLAG_STRIDE_WORDS = 32          # one 128-byte line per source rank


class _CudaBuffer:
    """Exposes a raw device allocation to torch through __cuda_array_interface__."""

    def __init__(self, ptr: int, shape, typestr: str):
        self.__cuda_array_interface__ = {"shape": tuple(shape), "typestr": typestr, "data": (ptr, False), "version": 3,
                                         "strides": None}


class _IpcBuffer:
    """`nbytes` of device memory the other ranks can store into (CUDA IPC)."""

    def __init__(self, nbytes: int, device: torch.device, group, rank: int, world: int):
        self.lib = capi.load()
        self.device, self.group, self.world = device, group, world
        ptr = ctypes.c_void_p()
        handle = ctypes.create_string_buffer(64)
        with torch.cuda.device(device):
            capi.check(self.lib.kcg_peer_alloc(nbytes, ctypes.byref(ptr), handle), "kcg_peer_alloc")
        self.ptr = ptr.value
        self.ptrs: List[int] = [0] * world      # address of every rank's buffer as seen from this rank
        self.ptrs[rank] = self.ptr
        self._opened: List[int] = []
        if world > 1:
            handles = [None] * world
            dist.all_gather_object(handles, bytes(handle.raw), group=group)
            for peer in range(world):
                if peer == rank:
                    continue
                out = ctypes.c_void_p()
                hb = ctypes.create_string_buffer(handles[peer], 64)
                with torch.cuda.device(device):
                    capi.check(self.lib.kcg_peer_open(hb, ctypes.byref(out)), "kcg_peer_open")
                self.ptrs[peer] = out.value
                self._opened.append(out.value)

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
            self.lib.kcg_peer_free(self.ptr)
            self.ptr = 0


class PeerMatrix:
    """A [rows, cols] bf16 or f32 matrix on this rank's GPU that the other ranks' kernels store into,
    with one completion flag per source rank.

    `backend`: "ipc", "symmetric", or "auto" (symmetric memory when torch offers it for this group,
    else IPC).  `store`, when given (a torch.distributed store), is used for a host-side check-in of
    all ranks before any buffer is mapped: a rank that never arrives raises `sharding.PeerTimeout`
    (KCG_PEER_TIMEOUT) on the host, before a kernel could ever wait for it.
    """

    def __init__(self, rows: int, cols: int, dtype: torch.dtype, device: torch.device, group=None,
                 backend: str = "ipc", store=None, checkin_timeout_s: float = 60.0):
        self.group = group
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        if store is not None:
            sharding.check_in(store, self.rank, self.world, step=f"peer-matrix/{rows}x{cols}", timeout_s=checkin_timeout_s)
        self.rows, self.cols, self.dtype, self.device = rows, cols, dtype, device
        self.itemsize = torch.empty((), dtype=dtype).element_size()
        self.mc_ptr = 0
        self._hdl = self._fhdl = None
        self._ipc: Optional[_IpcBuffer] = None
        self._fipc: Optional[_IpcBuffer] = None
        want_symm = backend in ("symmetric", "auto") and self.world > 1
        if want_symm:
            try:
                self._init_symmetric()
            except Exception:
                if backend == "symmetric":
                    raise
                want_symm = False
        if not want_symm:
            self._init_ipc()
        self.backend = "symmetric" if want_symm else "ipc"
        self.flags.zero_()
        torch.cuda.synchronize(device)
        if dist.is_initialized() and self.world > 1:
            dist.barrier(group=group)       # every rank's flags are zero before anybody signals

    # -- set-up ---------------------------------------------------------------------------------
    def _init_symmetric(self) -> None:
        import torch.distributed._symmetric_memory as symm

        grp = self.group if self.group is not None else dist.group.WORLD
        self.tensor = symm.empty((self.rows, self.cols), dtype=self.dtype, device=self.device)
        self._hdl = symm.rendezvous(self.tensor, grp)
        self.ptr = self.tensor.data_ptr()
        self._c_ptrs = [int(p) for p in self._hdl.buffer_ptrs]
        self.mc_ptr = int(self._hdl.multicast_ptr or 0)
        self.flags = symm.empty((self.world * FLAG_STRIDE_WORDS,), dtype=torch.int32, device=self.device)
        self._fhdl = symm.rendezvous(self.flags, grp)
        self._f_ptrs = [int(p) for p in self._fhdl.buffer_ptrs]

    def _init_ipc(self) -> None:
        nbytes = self.rows * self.cols * self.itemsize
        self._ipc = _IpcBuffer(nbytes, self.device, self.group, self.rank, self.world)
        self.ptr = self._ipc.ptr
        # torch views the same memory; bf16 has no array-interface typestr, so view through int16
        if self.dtype == torch.bfloat16:
            raw = torch.as_tensor(_CudaBuffer(self.ptr, (self.rows, self.cols), "<i2"), device=self.device)
            self.tensor = raw.view(torch.bfloat16)
        else:
            self.tensor = torch.as_tensor(_CudaBuffer(self.ptr, (self.rows, self.cols), "<f4"), device=self.device)
        self._c_ptrs = list(self._ipc.ptrs)
        self._fipc = _IpcBuffer(self.world * FLAG_STRIDE_WORDS * 4, self.device, self.group, self.rank, self.world)
        self.flags = torch.as_tensor(_CudaBuffer(self._fipc.ptr, (self.world * FLAG_STRIDE_WORDS,), "<i4"), device=self.device)
        self._f_ptrs = list(self._fipc.ptrs)

    # -- addresses handed to the GEMM launch --------------------------------------------------------
    @property
    def peer_ptrs(self) -> List[int]:
        """Base addresses of the other ranks' copies, rank order rotated to start after this rank."""
        return [self._c_ptrs[(self.rank + s) % self.world] for s in range(1, self.world)]

    def peer_row_ptrs(self, row_lo: int) -> List[int]:
        """Peers' addresses of row `row_lo` (where this rank's row block lands in their copies)."""
        off = row_lo * self.cols * self.itemsize
        return [p + off for p in self.peer_ptrs]

    def mc_row_ptr(self, row_lo: int) -> int:
        """Multicast address of row `row_lo` (0 when the copies are not bound to a multicast object)."""
        return self.mc_ptr + row_lo * self.cols * self.itemsize if self.mc_ptr else 0

    def done_flag_ptrs(self) -> List[int]:
        """This rank's slot in every rank's flag array (its own first): what a launch signals."""
        order = [self.rank] + [(self.rank + s) % self.world for s in range(1, self.world)]
        return [self._f_ptrs[r] + self.rank * FLAG_STRIDE_WORDS * 4 for r in order]

    def store_args(self, row_lo: int, value: int, multicast: bool = True) -> dict:
        """Keyword arguments for ops.matmul that make the launch deliver its row block to every
        copy and publish `value` in this rank's flag slots afterwards."""
        kw = {"done_flags": self.done_flag_ptrs(), "done_value": value}
        mc = self.mc_row_ptr(row_lo) if multicast else 0
        if mc:
            kw["mc"] = mc
        else:
            kw["peers"] = self.peer_row_ptrs(row_lo)
        return kw

    # -- completion ---------------------------------------------------------------------------------
    def wait(self, value: int, max_polls: int = 0) -> None:
        """Queues on the current stream a bounded wait until every rank's flag has reached `value`."""
        ops.peer_wait(self.flags.data_ptr(), self.world, FLAG_STRIDE_WORDS, value, self.device, max_polls)

    def close(self) -> None:
        torch.cuda.synchronize(self.device)
        if self._ipc is not None:
            self.tensor = None
            self.flags = None
            self._ipc.close()
            self._fipc.close()
            self._ipc = self._fipc = None
        else:
            if dist.is_initialized() and self.world > 1:
                dist.barrier(group=self.group)  # nobody releases the mapping while a peer may still store
            torch.cuda.synchronize(self.device)
            self._hdl = self._fhdl = None
            self.tensor = None
            self.flags = None
        self.ptr = 0
