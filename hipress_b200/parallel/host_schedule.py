"""CaSync ring and PS schedules over a message transport (``torch.distributed``
point-to-point + all-gather), built from the decoupled primitives encode / decode
/ merge / send / recv.

This is (a) the path CPU ranks use (gloo), (b) the *unfused* compressed baseline
on GPUs (separate encode and decode kernels around NCCL calls), and (c) the
behavioural twin of the fused kernels: same chunking, hop order, summation order
and division by N as :mod:`hipress_b200.parallel.simulate`.  All tensors of a
bucket share one message per hop (the reference's "bulk synchronisation").

Reference parity: CaSync-Ring / CaSync-PS, ``--topo Ring|PS``
(README.md:45,51 of mark14wu/hipress); cost shape src/SeCoPa/SeCoPa.py:75-103.
"""
from __future__ import annotations

import os
from dataclasses import dataclass, field

import torch
import torch.distributed as dist

from .._native import lib as _lib
from ..ops.compressor import Compressor, PayloadError
from .simulate import chunk_elems, chunk_range


@dataclass
class SegView:
    """One segment (a tensor or one partition of it) as flat fp32 views."""
    g: torch.Tensor                      # gradient, averaged result is written here
    state: dict                          # name -> flat view, same length as g
    server_state: dict = field(default_factory=dict)  # owner-side state, chunk_elems long
    seg_id: int = 0


class HostSchedule:
    def __init__(self, comp: Compressor, topology: str, group=None, verify: bool | None = None):
        """``verify``: check the header, sizes and indices of every received chunk
        payload before it is decoded and raise ``PayloadError`` naming hop and
        source (a corrupted or misrouted message must not be folded into the
        gradients).  Default: on for host tensors, where the check reads 16 bytes
        in place; off for device tensors (it would copy and synchronise) unless
        HIPRESS_VERIFY=1."""
        self.comp, self.topology, self.group = comp, topology.lower(), group
        self.verify = verify
        self.N = dist.get_world_size(group) if dist.is_initialized() else 1
        self.R = dist.get_rank(group) if dist.is_initialized() else 0
        self._bufs = {}
        self._ws = None
        self._ws_n = 0

    # ---------------------------------------------------------------- helpers
    def _layout(self, segs):
        """Byte offset and capacity of every segment's chunk payload in a message."""
        offs, total = [], 0
        for s in segs:
            ch = chunk_elems(s.g.numel(), self.N)
            if self.comp.spec.sparse:
                kmax = self.comp.kmax(ch)
                nb = int(_lib.cpu().hp_sparse_payload_bytes(kmax))
            else:
                kmax = None
                nb = self.comp.payload_bytes(ch)
            offs.append((total, nb, kmax))
            total += (nb + 127) // 128 * 128
        return offs, max(total, 16)

    def _buf(self, key, nbytes, device):
        b = self._bufs.get(key)
        if b is None or b.numel() < nbytes or b.device != device:
            b = torch.zeros(nbytes, dtype=torch.uint8, device=device)
            self._bufs[key] = b
        return b[:nbytes]

    def _verify(self, segs, offs, msg, chunk, what):
        """Integrity check of one received message: every segment's payload for `chunk`."""
        on = self.verify
        if on is None:
            on = (not msg.is_cuda) or os.environ.get("HIPRESS_VERIFY") == "1"
        if not on:
            return
        for s, (o, nb, kmax) in zip(segs, offs):
            lo, hi = chunk_range(s.g.numel(), self.N, chunk)
            if hi <= lo:
                continue
            try:
                self.comp.check_payload(msg[o:o + nb], hi - lo, kmax=kmax)
            except PayloadError as e:
                raise PayloadError(f"rank {self.R}, {what}, segment {s.seg_id}: {e}") from None

    def _global(self, r):
        return r if self.group is None else dist.get_global_rank(self.group, r)

    def _exchange(self, send, dst, recv, src):
        ops = [dist.P2POp(dist.isend, send, self._global(dst), group=self.group),
               dist.P2POp(dist.irecv, recv, self._global(src), group=self.group)]
        for w in dist.batch_isend_irecv(ops):
            w.wait()

    def _encode_chunk(self, s: SegView, c, hop, incoming, out, kmax, step, salt):
        comp, N, R = self.comp, self.N, self.R
        lo, hi = chunk_range(s.g.numel(), N, c)
        if hi <= lo:
            return
        g = s.g[lo:hi]
        st = {k: v[lo:hi] for k, v in s.state.items()}
        if comp.spec.sparse:
            acc = st["accum_v"] if "accum_v" in st else st["residual"]
            if incoming is not None:
                comp.decode(incoming, acc, accumulate=True, kmax=kmax)
            if g.is_cuda and (self._ws is None or self._ws_n < g.numel()):
                self._ws, self._ws_n = comp.new_workspace(g.device, g.numel()), g.numel()
            comp.encode(g, st, out=out, update=True, kmax=kmax, workspace=self._ws)
        else:
            comp.encode(g, st, incoming=incoming, out=out, step=step,
                        salt=salt + R * 256 + hop, tensor_id=s.seg_id, elem_offset=lo)

    def _decode_chunk(self, s: SegView, c, payload, kmax):
        lo, hi = chunk_range(s.g.numel(), self.N, c)
        if hi > lo:
            self.comp.decode(payload, s.g[lo:hi], scale=1.0 / self.N, kmax=kmax)

    # ------------------------------------------------------------------- sync
    def sync(self, segs, step=0, salt=0):
        if self.topology == "ring":
            self._ring(segs, step, salt)
        else:
            self._ps(segs, step, salt)

    def _ring(self, segs, step, salt):
        N, R = self.N, self.R
        dev = segs[0].g.device
        offs, total = self._layout(segs)
        send = [self._buf(("s", i), total, dev) for i in range(2)]
        recv = [self._buf(("r", i), total, dev) for i in range(2)]
        cur = None
        for hop in range(N):
            c = (R - hop) % N
            out = send[hop & 1]
            inc = recv[hop & 1] if hop > 0 else None
            if inc is not None:
                self._verify(segs, offs, inc, c, f"ring hop {hop} from rank {(R - 1) % N}")
            for s, (o, nb, kmax) in zip(segs, offs):
                self._encode_chunk(s, c, hop, None if inc is None else inc[o:o + nb],
                                   out[o:o + nb], kmax, step, salt)
            cur = out
            if hop < N - 1:
                self._exchange(out, (R + 1) % N, recv[(hop + 1) & 1], (R - 1) % N)
        if N > 1:
            gathered = [self._buf(("g", q), total, dev) for q in range(N)]
            dist.all_gather(gathered, cur.contiguous(), group=self.group)
        else:
            gathered = [cur]
        for src in range(N):
            c = (src + 1) % N
            if src != R:
                self._verify(segs, offs, gathered[src], c, f"ring gather from rank {src}")
            for s, (o, nb, kmax) in zip(segs, offs):
                self._decode_chunk(s, c, gathered[src][o:o + nb], kmax)

    def _ps(self, segs, step, salt):
        N, R = self.N, self.R
        comp = self.comp
        dev = segs[0].g.device
        offs, total = self._layout(segs)
        push = [self._buf(("p", j), total, dev) for j in range(N)]
        inbox = [self._buf(("i", q), total, dev) for q in range(N)]
        for j in range(N):
            for s, (o, nb, kmax) in zip(segs, offs):
                self._encode_chunk(s, j, 0, None, push[j][o:o + nb], kmax, step, salt)
        if N > 1:
            ops = []
            for d in range(1, N):
                ops.append(dist.P2POp(dist.isend, push[(R + d) % N], self._global((R + d) % N),
                                      group=self.group))
                ops.append(dist.P2POp(dist.irecv, inbox[(R - d) % N], self._global((R - d) % N),
                                      group=self.group))
            works = dist.batch_isend_irecv(ops)
            inbox[R].copy_(push[R])
            for w in works:
                w.wait()
        else:
            inbox[0] = push[0]
        pull = self._buf(("pull",), total, dev)
        for q in range(N):
            if q != R:
                self._verify(segs, offs, inbox[q], R, f"PS push from rank {q}")
        for s, (o, nb, kmax) in zip(segs, offs):
            lo, hi = chunk_range(s.g.numel(), N, R)
            if hi <= lo:
                continue
            m = hi - lo
            sst = {k: v[:m] for k, v in s.server_state.items()}
            if comp.spec.sparse:
                acc = sst["residual"] if "residual" in sst else torch.zeros(m, device=dev)
                for q in range(N):
                    comp.decode(inbox[q][o:o + nb], acc, accumulate=True, kmax=kmax)
                if acc.is_cuda and (self._ws is None or self._ws_n < m):
                    self._ws, self._ws_n = comp.new_workspace(dev, m), m
                comp.encode(acc, {"residual": acc}, out=pull[o:o + nb], update=False, kmax=kmax,
                            workspace=self._ws)
            else:
                acc = torch.empty(m, dtype=torch.float32, device=dev)
                for q in range(N):
                    comp.decode(inbox[q][o:o + nb], acc, accumulate=q > 0)
                comp.encode(acc, sst, out=pull[o:o + nb], step=step, salt=salt + R * 256 + 1,
                            tensor_id=s.seg_id, elem_offset=lo)
        if N > 1:
            gathered = [self._buf(("g", q), total, dev) for q in range(N)]
            dist.all_gather(gathered, pull.contiguous(), group=self.group)
        else:
            gathered = [pull]
        for j in range(N):
            if j != R:
                self._verify(segs, offs, gathered[j], j, f"PS pull from rank {j}")
            for s, (o, nb, kmax) in zip(segs, offs):
                self._decode_chunk(s, j, gathered[j][o:o + nb], kmax)
