"""Symmetric device memory: every rank allocates an arena of the same size and
maps every other rank's arena into its own address space through CUDA IPC, so
kernels can store payloads and flags straight into a peer GPU over NVLink.

Handles travel through ``torch.distributed`` (object all-gather on the job's
process group); the memory itself comes from ``cudaMalloc`` inside the native
library because a caching allocator's blocks cannot always be exported."""
from __future__ import annotations

import ctypes as C

import torch
import torch.distributed as dist

from .._native import lib as _lib
from . import comm


class SymmetricArena:
    def __init__(self, nbytes: int, group=None):
        self.nbytes = (int(nbytes) + 4095) // 4096 * 4096
        self.size, self.rank = comm.size(), comm.rank()
        self.group = group
        L = _lib.cuda()
        p = C.c_void_p()
        _lib.check(L.hp_cuda_arena_alloc(self.nbytes, C.byref(p)), "arena alloc")
        self.local = p.value
        self.ptrs = [None] * self.size
        self.ptrs[self.rank] = self.local
        self._opened = []
        if self.size > 1:
            hb = L.hp_cuda_ipc_handle_bytes()
            buf = C.create_string_buffer(hb)
            _lib.check(L.hp_cuda_ipc_export(self.local, buf), "ipc export")
            handles = [None] * self.size
            dist.all_gather_object(handles, bytes(buf.raw), group=group)
            for q, h in enumerate(handles):
                if q == self.rank:
                    continue
                pp = C.c_void_p()
                _lib.check(L.hp_cuda_ipc_open(C.create_string_buffer(h, hb), C.byref(pp)),
                           f"ipc open rank {q}")
                self.ptrs[q] = pp.value
                self._opened.append(pp.value)
            dist.barrier(group=group)
        self._cursor = 0

    def carve(self, nbytes: int):
        """Reserve `nbytes` at the same offset on every rank; returns per-rank addresses."""
        off = self._cursor
        self._cursor += (int(nbytes) + 255) // 256 * 256
        if self._cursor > self.nbytes:
            raise MemoryError("symmetric arena exhausted")
        return [p + off for p in self.ptrs]

    def close(self):
        L = _lib.cuda()
        if self.local is None:
            return
        torch.cuda.synchronize()
        if self.size > 1:
            dist.barrier(group=self.group)
        for p in self._opened:
            L.hp_cuda_ipc_close(p)
        self._opened = []
        if self.size > 1:
            dist.barrier(group=self.group)
        L.hp_cuda_arena_free(self.local)
        self.local = None
