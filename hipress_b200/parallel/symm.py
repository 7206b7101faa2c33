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
        self.size, self.rank = comm.group_size(group), comm.group_rank(group)
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
        self._guards = []

    GUARD_BYTES = 256
    GUARD_WORD = 0x5AFEC0DE

    def carve(self, nbytes: int):
        """Reserve `nbytes` at the same offset on every rank; returns per-rank
        addresses.  Every region is followed by a guard block of canary words in
        this rank's arena; :meth:`check_guards` reports a region that was overrun
        (by a local kernel or by a peer's stores)."""
        off = self._cursor
        size = (int(nbytes) + 255) // 256 * 256
        self._cursor += size + self.GUARD_BYTES
        if self._cursor > self.nbytes:
            raise MemoryError("symmetric arena exhausted")
        self._guards.append(off + size)
        g = self._view(off + size, self.GUARD_BYTES // 4)
        g.fill_(self.GUARD_WORD)
        return [p + off for p in self.ptrs]

    def _view(self, offset: int, words: int) -> torch.Tensor:
        """int32 tensor over a piece of the local arena (no copy)."""
        class _Arr:  # minimal __cuda_array_interface__ carrier
            pass
        a = _Arr()
        a.__cuda_array_interface__ = {"shape": (words,), "typestr": "<i4",
                                      "data": (self.local + offset, False), "version": 3}
        return torch.as_tensor(a, device=torch.device("cuda", torch.cuda.current_device()))

    def check_guards(self):
        """Raises if any guard block behind a carved region was overwritten."""
        torch.cuda.synchronize()
        bad = []
        for i, off in enumerate(self._guards):
            g = self._view(off, self.GUARD_BYTES // 4)
            if not bool((g == self.GUARD_WORD).all()):
                bad.append(i)
        if bad:
            raise RuntimeError(f"symmetric arena: regions {bad} were overrun (guard words changed)")

    def close(self, collective: bool = True):
        """Unmap the peers' arenas and free this rank's.  ``collective`` (the normal
        shutdown): every rank of the group calls it, and barriers keep a rank from
        freeing memory a peer's kernel may still store into.  ``collective=False`` is
        for the survivors of a changed membership: the group the arena was built on
        no longer exists, so no barrier can run; the caller guarantees that no kernel
        of any surviving rank is in flight (recovery happens between steps)."""
        L = _lib.cuda()
        if self.local is None:
            return
        torch.cuda.synchronize()
        if collective and self.size > 1:
            dist.barrier(group=self.group)
        for p in self._opened:
            L.hp_cuda_ipc_close(p)
        self._opened = []
        if collective and self.size > 1:
            dist.barrier(group=self.group)
        L.hp_cuda_arena_free(self.local)
        self.local = None
