"""Python face of the fused sparse kernels (csrc/cuda/fused_sparse.cu): a DGC /
GradDrop bucket is synchronised by ONE persistent cooperative launch that selects,
stores (index, value) pairs into peer GPUs' inboxes, re-selects (at the owner for
PS, at every hop for the ring) and scatters the result -- no NCCL call."""
from __future__ import annotations

import ctypes as C

import torch

from .._native import lib as _lib
from ..ops.algorithms import DGC, AlgSpec
from .simulate import chunk_elems

_bound = False


def _bind():
    global _bound
    L = _lib.cuda()
    if not _bound:
        L.hp_fused_sparse_layout.restype = C.c_int
        L.hp_fused_sparse_layout.argtypes = [C.c_float, C.POINTER(C.c_uint64), C.c_int, C.c_int,
                                             C.POINTER(C.c_uint64), C.POINTER(C.c_uint64),
                                             C.POINTER(C.c_uint64)]
        L.hp_cuda_fused_sparse_ps.restype = C.c_int
        sig = [C.c_int, C.c_float, C.c_float, C.POINTER(_lib.HpSeg), C.POINTER(C.c_void_p), C.c_int,
               C.POINTER(_lib.HpComm), C.c_void_p, C.c_int, C.c_void_p]
        L.hp_cuda_fused_sparse_ps.argtypes = sig
        L.hp_cuda_fused_sparse_ring.restype = C.c_int
        L.hp_cuda_fused_sparse_ring.argtypes = sig
        _bound = True
    return L


class FusedSparseBucket:
    """One bucket (<= 40 tensors) of a top-k algorithm on the PS or ring topology."""

    def __init__(self, spec: AlgSpec, sizes, nranks: int, rank: int, *, ctas: int = 0,
                 emulate: bool = False, timeout_s: float = 2.0, topology: str = "ps"):
        self.topology = topology.lower()
        if not spec.sparse:
            raise ValueError("FusedSparseBucket handles dgc / graddrop")
        self.spec, self.sizes = spec, [int(s) for s in sizes]
        self.nranks, self.rank, self.ctas, self.emulate = nranks, rank, int(ctas), emulate
        self.timeout_ns = int(timeout_s * 1e9)
        self.epoch = 0
        L = _bind()
        arr = (C.c_uint64 * len(self.sizes))(*self.sizes)
        ib, fw, wb = C.c_uint64(), C.c_uint64(), C.c_uint64()
        _lib.check(L.hp_fused_sparse_layout(spec.ratio, arr, len(self.sizes), nranks, C.byref(ib),
                                            C.byref(fw), C.byref(wb)), "sparse layout")
        self.inbox_bytes, self.flag_words, self.ws_bytes = ib.value, fw.value, wb.value
        self._segs = (_lib.HpSeg * len(self.sizes))()
        self._us = (C.c_void_p * len(self.sizes))()
        self._comm = _lib.HpComm()
        self.ws = None
        self.status = None

    def region_bytes(self) -> int:
        return (self.inbox_bytes + 255) // 256 * 256 + (self.flag_words * 4 + 255) // 256 * 256

    def bind(self, region_ptrs, status: torch.Tensor, device):
        ioff = (self.inbox_bytes + 255) // 256 * 256
        self.inbox_ptrs = [int(p) for p in region_ptrs]
        self.flag_ptrs = [int(p) + ioff for p in region_ptrs]
        self.status = status
        nr = self.nranks if self.emulate else 1
        self.ws = torch.zeros(self.ws_bytes * nr // 4, dtype=torch.int32, device=device)
        return self

    def bind_local(self, device):
        nr = self.nranks if self.emulate else 1
        assert self.emulate or self.nranks == 1
        self._arena = torch.zeros(nr * self.region_bytes(), dtype=torch.uint8, device=device)
        base = self._arena.data_ptr()
        status = torch.zeros(4 * nr, dtype=torch.int32, device=device)
        return self.bind([base + q * self.region_bytes() for q in range(nr)], status, device)

    def chunk_elems(self, i: int) -> int:
        return chunk_elems(self.sizes[i], self.nranks)

    def launch_ptrs(self, g_ptrs, acc_ptrs, u_ptrs, out_ptrs, sr_ptrs, *, strides=(0, 0, 0, 0),
                    stream=None):
        """Addresses per tensor: gradient, accumulator (DGC v / GradDrop residual),
        DGC momentum (or None), output, server accumulator of the owned chunk.
        strides (emulation): element strides between ranks of g, state, out, sr."""
        L = _bind()
        nseg = len(self.sizes)
        for i in range(nseg):
            s = self._segs[i]
            s.g, s.r, s.out, s.sr, s.n, s.id = g_ptrs[i], acc_ptrs[i], out_ptrs[i], sr_ptrs[i], \
                self.sizes[i], i
            self._us[i] = u_ptrs[i] if u_ptrs is not None else None
        cm = self._comm
        self.epoch = self.epoch % 0x7FFFFFFE + 1     # 31 bits: the top bit of a flag is a mark
        cm.nranks, cm.rank, cm.emulate = self.nranks, self.rank, 1 if self.emulate else 0
        cm.epoch, cm.timeout_ns = self.epoch, self.timeout_ns
        for q in range(self.nranks):
            cm.inbox[q] = self.inbox_ptrs[q]
            cm.flags[q] = self.flag_ptrs[q]
        cm.status = self.status.data_ptr()
        cm.trace = None
        cm.emu_stride_g, cm.emu_stride_r, cm.emu_stride_out, cm.emu_stride_sr = strides
        sp = self.spec
        us = self._us if sp.alg == DGC else None
        fn = L.hp_cuda_fused_sparse_ps if self.topology == "ps" else L.hp_cuda_fused_sparse_ring
        rc = fn(sp.alg, sp.ratio, sp.momentum, self._segs, us, nseg, C.byref(cm), self.ws.data_ptr(),
                self.ctas, _lib.stream_ptr(stream))
        _lib.check(rc, "fused sparse launch")

    def last_phase_times(self):
        """Device-side profile of the last launch (rank 0 of an emulated launch): the
        time in ms, from the kernel's start, at which CTA 0 left each phase barrier,
        and last its own end.  %globaltimer stamps written by the kernel."""
        WS_WORDS, STAMPS = 3 * 4096 + 16, 8      # kWsWords, kCtlStamps of the kernels
        nseg = len(self.sizes)
        ctl = (nseg * self.nranks + nseg) * WS_WORDS
        w = self.ws[ctl:ctl + 128].cpu().tolist()
        gen = w[1]
        st = [(x & 0xFFFFFFFF) for x in w[STAMPS:STAMPS + min(gen + 2, 128 - STAMPS)]]
        self.last_marks = [((x & 0xFFFFFFFF) - st[0]) % (1 << 32) * 1e-6 for x in w[64:72]]
        return [((x - st[0]) & 0xFFFFFFFF) * 1e-6 for x in st[1:]]

    def check_status(self):
        from .fused import HipressTimeoutError, decode_status
        words = self.status.cpu().tolist()
        bad = [(i // 4, w & 0xFFFFFFFF) for i, w in enumerate(words) if w != 0]
        if bad:
            self.status.zero_()
            raise HipressTimeoutError("; ".join(f"rank {r}: {decode_status(w)}" for r, w in bad))


def setup_engine_buckets(engine, fused_buckets) -> bool:
    """Called by GradSyncEngine for a sparse algorithm with the fused backend.
    Returns False when there is nothing to set up."""
    cfg = engine.cfg
    if not fused_buckets:
        return False
    from .symm import SymmetricArena
    impls = [FusedSparseBucket(engine.comp.spec, [s.n for s in b.segs], engine.N, engine.R,
                               ctas=0, timeout_s=cfg.timeout_s, topology=cfg.topology)
             for b in fused_buckets]
    total = sum(i.region_bytes() + 512 for i in impls) + 4096
    engine.arena = SymmetricArena(total, engine.group)
    engine.status = torch.zeros(4, dtype=torch.int32, device=engine.device)
    for b, impl in zip(fused_buckets, impls):
        impl.bind(engine.arena.carve(impl.region_bytes()), engine.status, engine.device)
        b.impl = impl
        b.stream = engine.comm_stream
        for s in b.segs:  # PS: the owner always needs an accumulator for the summed payloads
            sst = s.entry.server_state[s.part]
            if cfg.topology == "ps" and "residual" not in sst:
                sst["residual"] = torch.zeros(chunk_elems(s.n, engine.N), dtype=torch.float32,
                                              device=engine.device)
                sst["_scratch"] = True
    engine._status_host = torch.zeros(4, dtype=torch.int32).pin_memory()
    engine._status_event = None
    return True
