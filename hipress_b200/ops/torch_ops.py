"""The compression primitives as PyTorch custom operators (``torch.ops.hipress.*``),
the counterpart of the reference's torch extension (deps/torch-hipress-extension,
"use pytorch extension to power pytorch", README.md:92-96,111 of
mark14wu/hipress; its symbol names are not published, so these are our own).

    payload = torch.ops.hipress.encode(g, residual, "tbq", 0.01, 2, 0, 0)
    torch.ops.hipress.decode(payload, out, "tbq", 0.01, 2, 1.0, False)

CPU tensors run the C++ oracle, CUDA tensors the sm_100a kernels; both mutate their
state / output arguments in place like the reference's zero-output ops.
"""
from __future__ import annotations

import torch

from .compressor import Compressor

_cache: dict = {}


def _comp(alg: str, param: float, bits: int) -> Compressor:
    key = (alg, float(param), int(bits))
    c = _cache.get(key)
    if c is None:
        kw = {}
        if alg == "tbq":
            kw["threshold"] = param
        elif alg in ("dgc", "graddrop"):
            kw["ratio"] = param
        if alg == "terngrad" and bits:
            kw["bitwidth"] = bits
        c = _cache[key] = Compressor(alg, **kw)
    return c


@torch.library.custom_op("hipress::encode", mutates_args=("state",))
def encode(g: torch.Tensor, state: torch.Tensor, alg: str, param: float, bits: int, step: int,
           tensor_id: int) -> torch.Tensor:
    """Dense algorithms (onebit, tbq, terngrad).  `state` is the residual (an empty
    tensor for algorithms without error feedback).  Returns the payload bytes."""
    c = _comp(alg, param, bits)
    if c.spec.sparse:
        raise ValueError("use hipress::encode_topk for dgc / graddrop")
    st = {"residual": state} if state.numel() else {}
    return c.encode(g.reshape(-1), st, step=step, tensor_id=tensor_id)


@encode.register_fake
def _(g, state, alg, param, bits, step, tensor_id):
    return g.new_empty(_comp(alg, param, bits).payload_bytes(g.numel()), dtype=torch.uint8)


@torch.library.custom_op("hipress::encode_topk", mutates_args=("accum", "momentum"))
def encode_topk(g: torch.Tensor, accum: torch.Tensor, momentum: torch.Tensor, alg: str,
                ratio: float) -> torch.Tensor:
    """dgc (accum = v, momentum = u) or graddrop (accum = residual, momentum empty)."""
    c = _comp(alg, ratio, 0)
    st = {"accum_v": accum, "momentum_u": momentum} if alg == "dgc" else {"residual": accum}
    return c.encode(g.reshape(-1), st)


@encode_topk.register_fake
def _(g, accum, momentum, alg, ratio):
    return g.new_empty(_comp(alg, ratio, 0).payload_bytes(g.numel()), dtype=torch.uint8)


@torch.library.custom_op("hipress::decode", mutates_args=("out",))
def decode(payload: torch.Tensor, out: torch.Tensor, alg: str, param: float, bits: int, scale: float,
           accumulate: bool) -> None:
    """out = (out if accumulate else 0) + decode(payload) * scale, any algorithm."""
    _comp(alg, param, bits).decode(payload, out.view(-1), scale=scale, accumulate=accumulate)
