"""Python face of the fused CaSync kernels (csrc/cuda/fused_dense.cu).

:class:`FusedDenseBucket` owns the symmetric inbox / flag regions of one bucket of
tensors and launches ONE persistent kernel per synchronisation that performs
encode, peer-to-peer transfer and decode-aggregate for every tensor of the bucket.
With ``emulate=N`` a single GPU plays all N ranks in one cooperative launch
(gridDim.y = N): kernels that wait on one another must not run as separate
launches on one GPU, so this is how the multi-rank protocol is tested on one GPU.
"""
from __future__ import annotations

import ctypes as C

import torch

from .._native import lib as _lib
from ..ops.algorithms import AlgSpec
from .simulate import chunk_elems

TOPOLOGIES = {"ring": _lib.TOPO_RING, "ps": _lib.TOPO_PS}
TRACE_PHASES = 20                    # HP_TRACE_PHASES / HP_TRACE_WORDS of capi.h
TRACE_WORDS = 4 + 2 * TRACE_PHASES


class HipressTimeoutError(RuntimeError):
    """A bounded device-side wait expired (a peer never produced its flag)."""


def decode_status(word: int) -> str:
    if word == 0:
        return "ok"
    if word & 0x20000000 and not word & 0x80000000:
        return f"debug build: a payload index left its inbox at site {word & 0xFFFF} (recorded and skipped)"
    phase = (word >> 16) & 0x3FFF
    slot = (word >> 8) & 0xFF
    cta = word & 0xFF
    what = "a peer gave up first (its input never arrived)" if word & 0x40000000 else "timeout"
    return f"{what} phase={phase} slot={slot} cta={cta}"


class FusedDenseBucket:
    """One bucket = up to 40 tensors synchronised by one launch.

    ``inbox_ptrs`` / ``flag_ptrs``: per-rank device addresses of this bucket's
    regions as mapped into this process (from a symmetric arena), ``status``: a
    local int32 tensor of 4 words per emulated rank.
    """

    def __init__(self, spec: AlgSpec, topology: str, sizes, nranks: int, rank: int, *,
                 ctas: int = 64, emulate: bool = False, timeout_s: float = 2.0, trace: bool = False):
        self.trace_enabled = trace
        self.trace = None
        if spec.sparse:
            raise ValueError("FusedDenseBucket handles onebit / tbq / terngrad")
        self.spec, self.topo = spec, TOPOLOGIES[topology.lower()]
        self.sizes = [int(s) for s in sizes]
        self.nranks, self.rank, self.ctas, self.emulate = nranks, rank, int(ctas), emulate
        self.timeout_ns = int(timeout_s * 1e9)
        self.epoch = 0
        L = _lib.cuda()
        arr = (C.c_uint64 * len(self.sizes))(*self.sizes)
        ib, sb, tt = C.c_uint64(), C.c_uint64(), C.c_uint32()
        _lib.check(L.hp_fused_dense_layout(self.topo, spec.alg, spec.bits, arr, len(self.sizes),
                                           nranks, C.byref(ib), C.byref(sb), C.byref(tt)), "layout")
        self.inbox_bytes, self.slot_bytes, self.tiles_total = ib.value, sb.value, tt.value
        phases = 2 * nranks + (1 if self.topo == _lib.TOPO_PS else 0)
        self.ctas = max(1, min(self.ctas, self.tiles_total * phases))   # never more CTAs than work items
        self.inbox_ptrs = None
        self.status = None
        self._segs = (_lib.HpSeg * len(self.sizes))()
        self._comm = _lib.HpComm()

    # -- memory -----------------------------------------------------------
    def region_bytes(self) -> int:
        """Bytes this bucket needs in every rank's symmetric arena."""
        return (self.inbox_bytes + 255) // 256 * 256

    def bind(self, region_ptrs, status: torch.Tensor):
        """region_ptrs[q]: address of rank q's region for this bucket."""
        self.inbox_ptrs = [int(p) for p in region_ptrs]
        self.status = status
        if self.trace_enabled:
            nr = self.nranks if self.emulate else 1
            self.trace = torch.zeros(TRACE_WORDS * nr, dtype=torch.int64, device=status.device)
            self._trace_init = torch.tensor(([-1] + [0] * (TRACE_WORDS - 1)) * nr, dtype=torch.int64,
                                            device=status.device)
        return self

    def bind_local(self, device):
        """Emulation / single rank: allocate the regions of all ranks locally."""
        nr = self.nranks if self.emulate else 1
        assert self.emulate or self.nranks == 1
        self._arena = torch.zeros(nr * self.region_bytes(), dtype=torch.uint8, device=device)
        base = self._arena.data_ptr()
        status = torch.zeros(4 * nr, dtype=torch.int32, device=device)
        return self.bind([base + q * self.region_bytes() for q in range(nr)], status)

    def chunk_elems(self, i: int) -> int:
        return chunk_elems(self.sizes[i], self.nranks)

    def enable_trace(self, on: bool = True):
        """Switch the device-side phase trace on or off for the following launches
        (the bucket must be bound)."""
        if not on:
            self.trace = None
            return
        if self.trace is None:
            nr = self.nranks if self.emulate else 1
            dev = self.status.device
            self.trace = torch.zeros(TRACE_WORDS * nr, dtype=torch.int64, device=dev)
            self._trace_init = torch.tensor(([-1] + [0] * (TRACE_WORDS - 1)) * nr, dtype=torch.int64,
                                            device=dev)

    # -- launch -----------------------------------------------------------
    def launch(self, grads, residuals=None, outs=None, server_residuals=None, *, step=0, salt=0,
               tensor_ids=None, stream=None):
        """grads[i]: fp32 tensor of sizes[i] elements (emulation: shape [N, sizes[i]]
        with the same row stride for every tensor class).  The averaged result is
        written to outs[i] (default: in place)."""
        L = _lib.cuda()
        nseg = len(self.sizes)
        outs = outs if outs is not None else grads
        cm = self._comm
        for i in range(nseg):
            s = self._segs[i]
            g = grads[i]
            s.g = g.data_ptr()
            s.r = residuals[i].data_ptr() if residuals is not None and residuals[i] is not None else None
            s.out = outs[i].data_ptr()
            s.sr = (server_residuals[i].data_ptr()
                    if server_residuals is not None and server_residuals[i] is not None else None)
            s.n = self.sizes[i]
            s.id = tensor_ids[i] if tensor_ids is not None else i
        self.epoch = self.epoch % 0x7FFFFFFE + 1     # 31 bits: the top bit of the wire word is a mark
        cm.nranks, cm.rank, cm.emulate = self.nranks, self.rank, 1 if self.emulate else 0
        cm.epoch, cm.timeout_ns = self.epoch, self.timeout_ns
        for q in range(self.nranks):
            cm.inbox[q] = self.inbox_ptrs[q]
            cm.flags[q] = None      # the dense kernels signal inside the payload slots
        cm.status = self.status.data_ptr()
        self._arm_trace(cm, stream)
        if self.emulate:
            def stride(ts):
                if ts is None or ts[0] is None:
                    return 0
                st = ts[0].stride(0)
                assert all(t.stride(0) == st for t in ts if t is not None)
                return st
            cm.emu_stride_g = stride(grads)
            cm.emu_stride_r = stride(residuals)
            cm.emu_stride_out = stride(outs)
            cm.emu_stride_sr = stride(server_residuals)
        sp = self.spec
        rc = L.hp_cuda_fused_dense(self.topo, sp.alg, sp.bits, self._segs, nseg, C.byref(cm),
                                   sp.threshold, sp.seed, step, salt, self.ctas,
                                   _lib.stream_ptr(stream))
        _lib.check(rc, "fused dense launch")

    def launch_ptrs(self, g_ptrs, r_ptrs, out_ptrs, sr_ptrs, *, step=0, salt=0, tensor_ids=None,
                    stream=None):
        """Same as :meth:`launch` from raw device addresses (one per tensor; None = absent)."""
        L = _lib.cuda()
        nseg = len(self.sizes)
        cm = self._comm
        for i in range(nseg):
            s = self._segs[i]
            s.g, s.r, s.out, s.sr = g_ptrs[i], r_ptrs[i], out_ptrs[i], sr_ptrs[i]
            s.n = self.sizes[i]
            s.id = tensor_ids[i] if tensor_ids is not None else i
        self.epoch = self.epoch % 0x7FFFFFFE + 1     # 31 bits: the top bit of the wire word is a mark
        cm.nranks, cm.rank, cm.emulate = self.nranks, self.rank, 0
        cm.epoch, cm.timeout_ns = self.epoch, self.timeout_ns
        for q in range(self.nranks):
            cm.inbox[q] = self.inbox_ptrs[q]
            cm.flags[q] = None      # the dense kernels signal inside the payload slots
        cm.status = self.status.data_ptr()
        self._arm_trace(cm, stream)
        sp = self.spec
        rc = L.hp_cuda_fused_dense(self.topo, sp.alg, sp.bits, self._segs, nseg, C.byref(cm),
                                   sp.threshold, sp.seed, step, salt, self.ctas,
                                   _lib.stream_ptr(stream))
        _lib.check(rc, "fused dense launch")

    def _arm_trace(self, cm, stream):
        if self.trace is None:
            cm.trace = None
            return
        if stream is not None:
            with torch.cuda.stream(stream):
                self.trace.copy_(self._trace_init)
        else:
            self.trace.copy_(self._trace_init)
        cm.trace = self.trace.data_ptr()

    def last_trace(self):
        """Device-side timing of the last launch, per rank played by it:
        (encode phases ms, whole kernel ms) from %globaltimer stamps."""
        if self.trace is None:
            return None
        t = self.trace.cpu().view(-1, TRACE_WORDS)
        return [((int(r[1]) - int(r[0])) * 1e-6, (int(r[2]) - int(r[0])) * 1e-6) for r in t]

    def last_trace_phases(self):
        """Per rank played by the last launch: for every phase (ring: N hops then N
        gathers; PS: N pushes, the server pass, N pulls) the time, in ms from the
        first CTA's start, at which the last CTA finished it, and the mean time a CTA
        spent polling for its input in that phase."""
        if self.trace is None:
            return None
        phases = 2 * self.nranks + (1 if self.topo == _lib.TOPO_PS else 0)
        out = []
        for r in self.trace.cpu().view(-1, TRACE_WORDS):
            t0 = int(r[0])
            out.append([{"phase": p, "end_ms": (int(r[4 + p]) - t0) * 1e-6,
                         "mean_poll_ms": int(r[4 + TRACE_PHASES + p]) * 1e-6 / self.ctas}
                        for p in range(min(phases, TRACE_PHASES))])
        return out

    def check_status(self):
        """Synchronising read of the status words; raises on a recorded timeout."""
        words = self.status.cpu().tolist()
        bad = [(i // 4, w & 0xFFFFFFFF) for i, w in enumerate(words) if w != 0]
        if bad:
            self.status.zero_()
            raise HipressTimeoutError(
                "; ".join(f"rank {r}: {decode_status(w)}" for r, w in bad))
