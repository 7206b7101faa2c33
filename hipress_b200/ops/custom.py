"""User-defined compression algorithms in the synchronisation runtime.

The reference's workflow for a new algorithm is: write it in the CompLL DSL,
generate the operator pair, register it with the framework, select it with
``--comp-alg`` (README.md:190-277 of mark14wu/hipress).  Here the last two steps are

    enc, dec = load_op("MyEncode"), load_op("MyDecode")       # or any callables
    hp.register_algorithm("mine", encode=enc, decode=dec,
                          payload_bytes=lambda n: 10 + (n + 3) // 4,
                          encode_args=(2,), error_feedback=True)
    hp.DistributedOptimizer(opt, named, algorithm="mine", topology="ring")

``encode(gradient, compressed, *encode_args, seed=...)`` fills the uint8 payload from
a flat fp32 tensor and ``decode(compressed, gradient, *decode_args)`` overwrites a flat
fp32 tensor with the decoded values (the signatures of the DSL's TernGrad pair).
Registered algorithms run through the schedule built from decoupled primitives
(encode / decode / merge / send / recv): ring and PS, CPU and CUDA tensors, any
world size.  Merging, error feedback and the owner-side re-encode are composed
around the two operators, so the algorithm itself stays a plain encode/decode pair.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable

import torch


@dataclass(frozen=True)
class CustomSpec:
    name: str
    error_feedback: bool = True
    sparse: bool = False
    dense: bool = True
    ratio: float = 0.0
    momentum: float = 0.0
    alg: int = 0
    bits: int = 0

    def state_names(self):
        return ("residual",) if self.error_feedback else ()


class CustomCompressor:
    """The part of :class:`~hipress_b200.ops.Compressor`'s interface the host
    schedule uses, on top of a user-supplied encode/decode pair."""

    def __init__(self, name: str, encode: Callable, decode: Callable, payload_bytes: Callable,
                 encode_args=(), decode_args=(), error_feedback: bool = True, seeded: bool = True):
        self.spec = CustomSpec(name, error_feedback)
        self._enc, self._dec, self._nbytes = encode, decode, payload_bytes
        self._ea, self._da, self._seeded = tuple(encode_args), tuple(decode_args), seeded
        self._tmp: dict = {}

    # ------------------------------------------------------------- interface
    def payload_bytes(self, n: int) -> int:
        return int(self._nbytes(int(n)))

    def kmax(self, n: int) -> int:
        return 0

    def new_state(self, n: int, device) -> dict:
        return {k: torch.zeros(n, dtype=torch.float32, device=device) for k in self.spec.state_names()}

    def new_workspace(self, device, n):
        return None

    def check_payload(self, payload, n, kmax=None):
        """The payload layout belongs to the user's operators: nothing to verify."""

    def _scratch(self, key, n, device):
        t = self._tmp.get((key, device))
        if t is None or t.numel() < n:
            t = torch.empty(n, dtype=torch.float32, device=device)
            self._tmp[(key, device)] = t
        return t[:n]

    def encode(self, g, state=None, *, incoming=None, out=None, step=0, salt=0, tensor_id=0,
               elem_offset=0, **_):
        """x = g (+ decode(incoming)) (+ residual); payload = Q(x); residual = x - Q^-1(payload)."""
        n = g.numel()
        if out is None:
            out = torch.empty(self.payload_bytes(n), dtype=torch.uint8, device=g.device)
        if n == 0:
            return out
        # operators may derive the element count from the buffer length (the DSL's
        # extract does): hand them exactly the bytes of an n-element payload
        nb = self.payload_bytes(n)
        pay = out[:nb]
        x = self._scratch("x", n, g.device)
        x.copy_(g.reshape(-1))
        if incoming is not None:
            d = self._scratch("d", n, g.device)
            self._dec(incoming[:nb], d, *self._da)
            x.add_(d)
        r = (state or {}).get("residual") if self.spec.error_feedback else None
        if r is not None:
            x.add_(r)
        kw = {}
        if self._seeded:  # one independent random stream per (step, rank/hop, tensor, chunk)
            kw["seed"] = ((int(step) * 1000003 + int(salt)) * 1000003 + int(tensor_id)) * 1000003 \
                + int(elem_offset) & ((1 << 63) - 1)
        self._enc(x, pay, *self._ea, **kw)
        if r is not None:
            d = self._scratch("d", n, g.device)
            self._dec(pay, d, *self._da)
            torch.sub(x, d, out=r)
        return out

    def decode(self, payload, out, *, scale=1.0, accumulate=False, kmax=None, **_):
        """out = (out if accumulate else 0) + decode(payload) * scale."""
        n = out.numel()
        if n == 0:
            return out
        payload = payload[:self.payload_bytes(n)]
        if not accumulate and scale == 1.0 and out.is_contiguous():
            self._dec(payload, out, *self._da)
            return out
        d = self._scratch("d", n, out.device)
        self._dec(payload, d, *self._da)
        if accumulate:
            out.add_(d, alpha=scale)
        else:
            torch.mul(d, scale, out=out)
        return out


_REGISTRY: dict = {}


def register_algorithm(name: str, *, encode: Callable, decode: Callable, payload_bytes: Callable,
                       encode_args=(), decode_args=(), error_feedback: bool = True,
                       seeded: bool = True) -> None:
    """Make ``algorithm=name`` available to DistributedOptimizer / GradSyncEngine.
    ``seeded``: the encoder takes a ``seed=`` keyword (CompLL bindings do)."""
    key = name.lower()
    from .algorithms import ALIASES, _TABLE
    if key in _TABLE or key in ALIASES or key in ("none", ""):
        raise ValueError(f"{name!r} is a built-in algorithm name")
    _REGISTRY[key] = dict(name=key, encode=encode, decode=decode, payload_bytes=payload_bytes,
                          encode_args=encode_args, decode_args=decode_args,
                          error_feedback=error_feedback, seeded=seeded)


def unregister_algorithm(name: str) -> None:
    _REGISTRY.pop(name.lower(), None)


def custom_compressor(name: str) -> CustomCompressor | None:
    """A fresh compressor for a registered name, or ``None``."""
    kw = _REGISTRY.get((name or "").lower())
    return None if kw is None else CustomCompressor(**kw)
