"""Tensor-level compression primitives (CompLL's run-time face).

:class:`Compressor` offers the decoupled primitives CaSync composes — ``encode``
(optionally merging an incoming payload: recv -> decode -> merge -> encode),
``decode`` and ``decode``-accumulate — on CPU tensors (C++ oracle) and on CUDA
tensors (sm_100a kernels) with identical wire formats.  The fused ring / PS
kernels do not go through this class; they share its device code and are checked
against it.

Reference parity: the generated ops are in-place pairs
``Encode(gradient, compressed, params)`` / ``Decode(compressed, gradient)``
(src/CompLL/GCGen/output/TernGradEncode/TernGradEncode.cc:10-24).
"""
from __future__ import annotations

import torch

from .._native import lib as _lib
from .algorithms import AlgSpec, DGC, get_algorithm

TILE = 4096


def _c(t):
    return None if t is None else t.data_ptr()


class PayloadError(RuntimeError):
    """A received payload does not match the format its receiver expects."""


class Compressor:
    def __init__(self, spec: AlgSpec | str, **overrides):
        self.spec = get_algorithm(spec, **overrides) if isinstance(spec, str) else spec

    # ------------------------------------------------------------------ sizes
    def kmax(self, n: int) -> int:
        return int(_lib.cpu().hp_sparse_k(n, self.spec.ratio)) if self.spec.sparse else 0

    def payload_bytes(self, n: int) -> int:
        L = _lib.cpu()
        if self.spec.sparse:
            return int(L.hp_sparse_payload_bytes(self.kmax(n)))
        return int(L.hp_dense_payload_bytes(self.spec.alg, self.spec.bits, n))

    def new_state(self, n: int, device) -> dict:
        return {k: torch.zeros(n, dtype=torch.float32, device=device) for k in self.spec.state_names()}

    def new_workspace(self, device, n: int | None = None):
        """Scratch of the sparse CUDA encoder: radix histograms and counters, plus
        (when the tensor size ``n`` is given) room for the candidate list that lets
        the encoder read the array once instead of three times after the update."""
        if self.spec.sparse and torch.device(device).type == "cuda":
            L = _lib.cuda()
            nb = int(L.hp_sparse_workspace_bytes()) if n is None else \
                int(L.hp_sparse_workspace_bytes_for(self.kmax(n)))
            return torch.zeros((nb + 3) // 4, dtype=torch.int32, device=device)
        return None

    # ----------------------------------------------------------------- encode
    def encode(self, g, state=None, *, incoming=None, out=None, step=0, salt=0, tensor_id=0,
               elem_offset=0, update=True, workspace=None, kmax=None, stream=None, max_ctas=0):
        """Compress ``g`` (fp32, contiguous, 1-D view).

        dense : x = g (+ decode(incoming)) (+ residual); payload = Q(x); residual = x - Q^-1.
        sparse: state update with g when ``update``; incoming pairs are added into
                the accumulator; exact top-k of the accumulator is sent and zeroed.
        ``state`` is the dict from :meth:`new_state` (views of it for chunks).
        """
        sp = self.spec
        n = g.numel()
        state = state or {}
        if out is None:
            nb = self.payload_bytes(n) if kmax is None else int(_lib.cpu().hp_sparse_payload_bytes(kmax))
            out = torch.empty(nb, dtype=torch.uint8, device=g.device)
        if n == 0:
            return out
        assert g.dtype == torch.float32 and g.is_contiguous()
        if sp.sparse:
            return self._encode_sparse(g, state, incoming, out, update, workspace, kmax, stream, max_ctas)
        r = state.get("residual") if sp.error_feedback else None
        if g.is_cuda:
            L = _lib.cuda()
            rc = L.hp_cuda_dense_encode(sp.alg, sp.bits, _c(g), _c(r), _c(incoming), _c(out), n,
                                        sp.threshold, sp.seed, step, salt, tensor_id, elem_offset,
                                        max_ctas, _lib.stream_ptr(stream))
        else:
            rc = _lib.cpu().hp_cpu_dense_encode(sp.alg, sp.bits, _c(g), _c(r), _c(incoming), _c(out),
                                                n, sp.threshold, sp.seed, step, salt, tensor_id,
                                                elem_offset)
        _lib.check(rc, f"{sp.name} encode", device_call=g.is_cuda)
        return out

    def _encode_sparse(self, g, state, incoming, out, update, workspace, kmax, stream, max_ctas):
        sp = self.spec
        n = g.numel()
        k = self.kmax(n)
        kmax = k if kmax is None else kmax
        a = state["accum_v"] if "accum_v" in state else state["residual"]
        u = state.get("momentum_u")
        if g.is_cuda:
            L = _lib.cuda()
            sptr = _lib.stream_ptr(stream)
            ws = workspace if workspace is not None else self.new_workspace(g.device, n)
            if incoming is not None:
                # the accumulator must hold the updated local value before the merge
                raise ValueError("merge incoming sparse payloads with decode(accumulate=True) "
                                 "after update_state(); then call encode(update=False)")
            rc = L.hp_cuda_sparse_encode(sp.alg, _c(g), _c(a), _c(u), n, k, kmax, sp.momentum,
                                         1 if update else 0, _c(out), _c(ws), ws.numel() * 4, max_ctas,
                                         sptr)
            _lib.check(rc, f"{sp.name} encode")
            return out
        L = _lib.cpu()
        if update:
            if sp.alg == DGC:
                L.hp_cpu_dgc_update(_c(g), _c(u), _c(a), n, sp.momentum)
            else:
                L.hp_cpu_acc_update(_c(g), _c(a), n)
        if incoming is not None:
            raise ValueError("merge incoming sparse payloads with decode(accumulate=True)")
        rc = L.hp_cpu_sparse_select(sp.alg, _c(a), _c(u), n, k, _c(out), kmax)
        _lib.check(rc, f"{sp.name} select", device_call=False)
        return out

    def update_state(self, g, state, stream=None):
        """Sparse algorithms only: apply the state update without selecting
        (DGC: u = m*u + g, v += u; GradDrop: r += g)."""
        sp = self.spec
        assert sp.sparse
        n = g.numel()
        if n == 0:
            return
        a = state["accum_v"] if sp.alg == DGC else state["residual"]
        if g.is_cuda:
            # plain torch ops: this path is only used by the unfused baseline
            if sp.alg == DGC:
                u = state["momentum_u"]
                u.mul_(sp.momentum).add_(g)
                a.add_(u)
            else:
                a.add_(g)
            return
        L = _lib.cpu()
        if sp.alg == DGC:
            L.hp_cpu_dgc_update(_c(g), _c(state["momentum_u"]), _c(a), n, sp.momentum)
        else:
            L.hp_cpu_acc_update(_c(g), _c(a), n)

    # ----------------------------------------------------------------- decode
    def decode(self, payload, out, *, scale=1.0, accumulate=False, kmax=None, stream=None, max_ctas=0):
        """out = (out if accumulate else 0) + decode(payload) * scale."""
        sp = self.spec
        n = out.numel()
        if n == 0:
            return out
        assert out.dtype == torch.float32 and out.is_contiguous()
        if sp.sparse:
            kmax = self.kmax(n) if kmax is None else kmax
            if out.is_cuda:
                rc = _lib.cuda().hp_cuda_sparse_decode(_c(payload), _c(out), n, kmax, scale,
                                                       1 if accumulate else 0, _lib.stream_ptr(stream))
            else:
                rc = _lib.cpu().hp_cpu_sparse_decode(_c(payload), _c(out), n, kmax, scale,
                                                     1 if accumulate else 0)
        elif out.is_cuda:
            rc = _lib.cuda().hp_cuda_dense_decode(sp.alg, sp.bits, _c(payload), _c(out), n,
                                                  sp.threshold, scale, 1 if accumulate else 0,
                                                  max_ctas, _lib.stream_ptr(stream))
        else:
            rc = _lib.cpu().hp_cpu_dense_decode(sp.alg, sp.bits, _c(payload), _c(out), n,
                                                sp.threshold, scale, 1 if accumulate else 0)
        _lib.check(rc, f"{sp.name} decode", device_call=out.is_cuda)
        return out

    _PAYLOAD_FAULTS = {1: "buffer shorter than the format needs", 2: "algorithm id", 3: "bit width",
                       4: "element count", 5: "tile size or flags", 6: "pair count above capacity",
                       7: "pair index out of range"}

    def check_payload(self, payload, n, kmax=None):
        """Integrity check of a received payload against what this compressor would
        have produced for ``n`` elements (header fields, sizes, sparse indices);
        raises :class:`PayloadError` naming the first mismatch.  The payload is read
        on the host: for a CUDA tensor this copies and synchronises, so the host
        transport verifies device payloads only when asked to."""
        sp = self.spec
        p = payload if not payload.is_cuda else payload.cpu()
        p = p.contiguous()
        if sp.sparse:
            kmax = self.kmax(n) if kmax is None else kmax
            rc = _lib.cpu().hp_payload_check(_c(p), p.numel(), sp.alg, 0, n, kmax)
        else:
            rc = _lib.cpu().hp_payload_check(_c(p), p.numel(), sp.alg, sp.bits, n, 0)
        if rc:
            raise PayloadError(f"{sp.name} payload for {n} elements is corrupt: "
                               f"{self._PAYLOAD_FAULTS.get(rc, rc)}")


def sparse_pairs(payload: torch.Tensor, kmax: int):
    """(indices, values) of a sparse payload, sorted by index (host tensors)."""
    p = payload.detach().cpu()
    k = int(p[12:16].view(torch.int32).item())
    off = 16 + (4 * kmax + 15) // 16 * 16
    idx = p[16:16 + 4 * k].view(torch.int32).to(torch.int64) & 0xFFFFFFFF
    val = p[off:off + 4 * k].view(torch.float32)
    order = torch.argsort(idx)
    return idx[order], val[order]
