"""Exchange arenas in peer memory for the sequence-parallel attention (one process per GPU).

Each rank owns one device allocation ("arena": a library header with arrival flags and epoch
counters, then the buffers the other ranks store into) and maps every other rank's arena
through CUDA IPC.  The q/k/v assembly kernel then writes each head group directly into the
arena of the rank that will run attention on it, and the attention kernel writes each query
row directly into the arena of the rank that owns that token — the two head all-to-alls of
Ulysses happen inside the producing kernels, as plain stores over NVLink, ordered by the
library's signal / wait kernels.  Nothing here reads peer memory.
"""
from __future__ import annotations

import ctypes
from ctypes import c_void_p

import torch
import torch.distributed as dist

from .. import _lib


class _DeviceBytes:
    """Zero-copy view of a raw device allocation for torch.as_tensor."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {
            "shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 2, "strides": None,
        }


class PeerArena:
    """This rank's arena plus the mapped arenas of all ranks of `group`.

    Collective: every rank of the group must construct it with the same `nbytes`, in the same
    order relative to other collectives."""

    def __init__(self, nbytes: int, group=None):
        lib = _lib.load()
        self.group = group
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)
        if self.world > 8:
            raise NotImplementedError("peer exchange is built for at most 8 ranks on one box")
        self.header = lib.fluxb_peer_header_bytes()
        self.nbytes = self.header + ((nbytes + 255) // 256) * 256
        own = c_void_p()
        _lib.check(lib.fluxb_peer_alloc(self.nbytes, ctypes.byref(own)), launches=False)
        self._own = own.value
        handle = ctypes.create_string_buffer(64)
        _lib.check(lib.fluxb_peer_export(self._own, handle), launches=False)
        handles: list = [None] * self.world
        dist.all_gather_object(handles, bytes(handle.raw), group=group)
        self.ptrs: list[int] = []
        self._opened: list[int] = []
        for r, h in enumerate(handles):
            if r == self.rank:
                self.ptrs.append(self._own)
                continue
            p = c_void_p()
            _lib.check(lib.fluxb_peer_open(ctypes.create_string_buffer(h, 64), ctypes.byref(p)), launches=False)
            self.ptrs.append(p.value)
            self._opened.append(p.value)
        self.c_ptrs = (c_void_p * self.world)(*self.ptrs)
        dev = torch.cuda.current_device()
        self.local = torch.as_tensor(_DeviceBytes(self._own, self.nbytes), device=f"cuda:{dev}")
        # Every rank has mapped every arena before anyone stores into one.
        dist.barrier(group=group)

    def local_view(self, offset: int, shape, dtype) -> torch.Tensor:
        """Tensor over this rank's arena, `offset` bytes after the header."""
        n = 1
        for s in shape:
            n *= s
        nbytes = n * torch.empty((), dtype=dtype).element_size()
        start = self.header + offset
        assert start + nbytes <= self.nbytes, "view exceeds the arena"
        return self.local[start : start + nbytes].view(dtype).view(*shape)

    def address(self, rank: int, offset: int) -> int:
        """Address, in this process, of byte `offset` (after the header) of `rank`'s arena."""
        return self.ptrs[rank] + self.header + offset

    def signal(self, barrier: int) -> None:
        _lib.check(_lib.load().fluxb_peer_signal(self.c_ptrs, self.world, self.rank, barrier, _lib.stream_handle()))

    def wait(self, barrier: int) -> None:
        _lib.check(_lib.load().fluxb_peer_wait(self.c_ptrs, self.world, self.rank, barrier, _lib.stream_handle()))

    def close(self) -> None:
        """Collective teardown: unmap the peers' arenas, then free the own one."""
        lib = _lib.load()
        torch.cuda.synchronize()
        dist.barrier(group=self.group)
        for p in self._opened:
            lib.fluxb_peer_close(p)
        self._opened = []
        dist.barrier(group=self.group)
        if self._own:
            self.local = None
            lib.fluxb_peer_free(self._own)
            self._own = 0
