"""Peer-mapped memory and the exchange descriptors of a model cut over the GPUs of one box (one process a GPU).

The exchange itself is device code (csrc/tp.cuh): producers store every finished element, marked with its hop's
sequence number, into every rank's copy of an activation vector; consumers read their local copy and take each word
once it carries the mark. This module sets that up: a `PeerHeap` is one allocation of the same size and layout on every
rank, each rank's mapped into every process (CUDA IPC handles handed round through the process group at set-up; plain
pointers when the "ranks" are engines of one process, which is how a single GPU exercises the N-rank data path in
lockstep); `carve` hands out equal offsets on every rank; `send_desc` builds the C-ABI's descriptor.
"""

from __future__ import annotations

import ctypes as C
from typing import Any

import torch

from . import capi
from .capi import Send, call


class PeerHeap:
    """`nbytes` of zeroed device memory on this rank plus every rank's heap as mapped here: base[r] + offset is rank r's
    copy of whatever lies at `offset`"""

    def __init__(self, nbytes: int, rank: int = 0, world: int = 1):
        self.nbytes, self.rank, self.world = int(nbytes), rank, world
        p = C.c_void_p()
        call("btb_b200_peer_alloc", self.nbytes, C.byref(p))
        self.local = int(p.value)
        self.base: list[int] = [0] * world
        self.base[rank] = self.local
        self._opened: list[int] = []
        self._top = 0

    # -- connecting the ranks ------------------------------------------------------------------------------------------
    def connect_processes(self, group: Any = None) -> None:
        """one process a GPU: every rank's IPC handle to every rank through the process group, then opened"""
        if self.world == 1:
            return
        import torch.distributed as dist

        h = (C.c_ubyte * 64)()
        call("btb_b200_peer_handle", self.local, h)
        handles: list[Any] = [None] * self.world
        dist.all_gather_object(handles, bytes(h), group=group)
        for r, hb in enumerate(handles):
            if r == self.rank:
                continue
            p = C.c_void_p()
            call("btb_b200_peer_open", (C.c_ubyte * 64)(*hb), C.byref(p))
            self.base[r] = int(p.value)
            self._opened.append(int(p.value))
        dist.barrier(group=group)

    @staticmethod
    def connect_engines(heaps: list["PeerHeap"]) -> None:
        """the ranks are engines of ONE process on one GPU (the lockstep emulation): their heaps are plain pointers"""
        for h in heaps:
            h.base = [o.local for o in heaps]

    def close(self) -> None:
        for p in self._opened:
            capi.lib().btb_b200_peer_close(p)
        self._opened = []
        if self.local:
            capi.lib().btb_b200_peer_free(self.local)
            self.local = 0

    # -- layout --------------------------------------------------------------------------------------------------------
    def carve(self, nbytes: int, align: int = 256) -> int:
        """the next `nbytes` of the heap (the same offset on every rank, as long as every rank carves in the same order)"""
        off = (self._top + align - 1) // align * align
        if off + nbytes > self.nbytes:
            raise MemoryError(f"the peer heap holds {self.nbytes} bytes, asked for {off + nbytes}")
        self._top = off + nbytes
        return off

    def tensor(self, off: int, shape: tuple, dtype: torch.dtype) -> torch.Tensor:
        """this rank's copy of the region at `off` as a torch tensor (no copy; the heap must outlive it)"""
        n = 1
        for d in shape:
            n *= int(d)
        nbytes = n * torch.empty(0, dtype=dtype).element_size()

        class _Mem:
            __cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (self.local + off, False), "version": 2}

        return torch.as_tensor(_Mem(), device="cuda").view(dtype).reshape(shape)

    # -- descriptors ---------------------------------------------------------------------------------------------------
    def send_desc(self, buf_off: int, stride: int, offset: int, pass_ptr: int, per_pass: int, base: int) -> Send:
        s = Send()
        for r in range(self.world):
            s.out[r] = self.base[r] + buf_off
        s.n, s.stride, s.offset = self.world, int(stride), int(offset)
        s.pass_, s.per_pass, s.base = pass_ptr, int(per_pass), int(base)
        return s
