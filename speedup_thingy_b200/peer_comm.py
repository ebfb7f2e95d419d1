"""Gradient exchange of the data-parallel step over NVLink peer memory.

One process per GPU on one node.  Every rank allocates its gradient buffer and a small flag array through the
library (``rte_peer_alloc``: plain device allocations with an inter-process handle), plus a staging buffer of the
same size, sends the 64-byte handles to the other ranks over the existing process group, and maps theirs with its own
device current (``rte_peer_open``).  From then on a bucket is summed across ranks by ONE kernel per rank
(``rte_peer_allreduce_sum_f32``: plain peer stores, sums in rank order, bounded waits) instead of a library collective.  The kernel takes no host-side state
per call, so it can be captured into the step's CUDA graph.
"""
from __future__ import annotations

import ctypes as C
import os

import torch

from . import _abi as A


class _DeviceArray:
    """Lets ``torch.as_tensor`` wrap a library allocation without copying (CUDA array interface, version 3)."""

    def __init__(self, ptr: int, numel: int, typestr: str):
        self.__cuda_array_interface__ = {"shape": (numel,), "typestr": typestr, "data": (ptr, False), "version": 3,
                                         "strides": None, "stream": None}


class PeerMemory:
    """One zero-filled device allocation of this rank that the other ranks can map."""

    def __init__(self, ops, nbytes: int):
        self.ops, self.nbytes = ops, int(nbytes)
        ptr, handle = A.c_vp(), C.create_string_buffer(A.IPC_HANDLE_BYTES)
        with torch.cuda.device(ops.device):
            A.check(ops.lib.rte_peer_alloc(self.nbytes, C.byref(ptr), handle), "rte_peer_alloc")
        self.ptr, self.handle = int(ptr.value), handle.raw

    def tensor(self, dtype: torch.dtype) -> torch.Tensor:
        """The allocation as a flat tensor (a view: it keeps this object alive, not the other way round)."""
        typestr = {torch.float32: "<f4", torch.int32: "<i4"}[dtype]
        t = torch.as_tensor(_DeviceArray(self.ptr, self.nbytes // 4, typestr), device=self.ops.device)
        t._rte_owner = self
        return t

    def free(self) -> None:
        if self.ptr:
            with torch.cuda.device(self.ops.device):
                A.check(self.ops.lib.rte_peer_free(A.c_vp(self.ptr)), "rte_peer_free")
            self.ptr = 0


class PeerAllReduce:
    """`buffer_mem`: this rank's PeerMemory holding the float32 gradient buffer (same size on every rank); slices of it
    are exchanged in place."""

    def __init__(self, ops, buffer_mem: PeerMemory, process_group):
        import torch.distributed as dist

        self.ops, self.pg, self.buffer_mem = ops, process_group, buffer_mem
        self.world, self.rank = dist.get_world_size(process_group), dist.get_rank(process_group)
        if not 2 <= self.world <= A.COMM_MAX_RANKS:
            raise ValueError(f"PeerAllReduce handles 2..{A.COMM_MAX_RANKS} ranks of one node")
        dev = ops.device
        self.flag_mem = PeerMemory(ops, A.COMM_MAX_SLOTS * 2 * A.COMM_MAX_RANKS * 4)
        # where the peers push their values of this rank's parts (a part's row may overhang a range by 4 * ranks floats)
        self.stage_mem = PeerMemory(ops, buffer_mem.nbytes + 4 * A.COMM_MAX_RANKS * 4)
        self.epoch = torch.zeros(A.COMM_MAX_SLOTS, dtype=torch.int32, device=dev)
        self.done_count = torch.zeros(A.COMM_MAX_SLOTS * 2, dtype=torch.int32, device=dev)
        torch.cuda.synchronize(dev)
        mine = (buffer_mem.handle, self.stage_mem.handle, self.flag_mem.handle, buffer_mem.nbytes, int(dev.index or 0))
        gathered: list = [None] * self.world
        dist.all_gather_object(gathered, mine, group=process_group)
        self._mapped: list[int] = []               # peers' allocations mapped into this process
        comm = A.PeerComm()
        with torch.cuda.device(dev):               # the mappings must be opened with THIS rank's device current
            for q, (buf_h, stage_h, flag_h, nbytes, owner_dev) in enumerate(gathered):
                if nbytes != buffer_mem.nbytes:
                    raise ValueError("every rank's gradient buffer must have the same size")
                if q == self.rank:
                    comm.buf[q], comm.stage[q], comm.flags[q] = buffer_mem.ptr, self.stage_mem.ptr, self.flag_mem.ptr
                    continue
                for h, field in ((buf_h, comm.buf), (stage_h, comm.stage), (flag_h, comm.flags)):
                    p = A.c_vp()
                    A.check(ops.lib.rte_peer_open(h, owner_dev, C.byref(p)), "rte_peer_open")
                    self._mapped.append(int(p.value))
                    field[q] = int(p.value)
        comm.epoch, comm.done_count = self.epoch.data_ptr(), self.done_count.data_ptr()
        comm.world, comm.rank = self.world, self.rank
        self._comm = comm
        dist.barrier(group=process_group)          # everybody has mapped everybody before the first exchange
        self.max_ctas = int(os.environ.get("RTE_PEER_CTAS", "64"))      # CTAs of one exchange (the rest of the SMs keep computing)

    def all_reduce_(self, lo: int, hi: int, slot: int) -> None:
        """buffer[lo:hi] <- sum over ranks, in place, on the current stream.  Every rank must issue the same calls in
        the same order; `slot` (< 64) must differ between exchanges that can be in flight at the same time."""
        if lo % 4 or hi % 4 or not 0 <= lo < hi <= self.buffer_mem.nbytes // 4:
            raise ValueError("exchanged ranges must lie inside the buffer and start and end on multiples of 4 floats")
        o = self.ops
        o._call("rte_peer_allreduce_sum_f32", C.byref(self._comm), lo, hi - lo, slot % A.COMM_MAX_SLOTS, self.max_ctas,
                C.c_void_p(o.status.data_ptr()), o.stream)

    def close(self) -> None:
        """Unmaps the peers' memory (call after the last exchange has completed on every rank; a barrier belongs between
        this and the owners' `PeerMemory.free`)."""
        with torch.cuda.device(self.ops.device):
            for p in self._mapped:
                A.check(self.ops.lib.rte_peer_close(A.c_vp(p)), "rte_peer_close")
        self._mapped.clear()
