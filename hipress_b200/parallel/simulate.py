"""Lock-step simulation of the CaSync ring and PS schedules for N ranks in one
process, built only from :class:`~hipress_b200.ops.Compressor` primitives.

It defines the exact arithmetic of one synchronisation (which chunk is merged at
which hop, in which order payloads are summed, where the division by N happens)
and is what the fused kernels and the multi-process host schedule are tested
against.  Cost shape per gradient follows the reference planner: ring = N
encodes, N decodes, N-1 merges (src/SeCoPa/SeCoPa.py:92-103); PS = gather +
broadcast with a server-side re-encode (src/SeCoPa/SeCoPa.py:75-89).
"""
from __future__ import annotations

import torch

from ..ops.compressor import TILE, Compressor


def chunk_elems(n: int, nranks: int) -> int:
    """Elements per chunk: ceil(n / nranks) rounded up to whole tiles."""
    per = (n + nranks - 1) // nranks
    return (per + TILE - 1) // TILE * TILE


def chunk_range(n: int, nranks: int, c: int):
    ch = chunk_elems(n, nranks)
    lo = min(n, c * ch)
    return lo, min(n, lo + ch)


def _slice_state(state, lo, hi):
    return {k: v[lo:hi] for k, v in state.items()}


def simulate_ring(comp: Compressor, grads, states, *, step=0, salt=0, tensor_id=0):
    """grads[r], states[r]: rank r's gradient and compressor state (updated in
    place).  Returns the list of averaged gradients, identical on every rank."""
    N = len(grads)
    n = grads[0].numel()
    sp = comp.spec
    dev = grads[0].device
    inv = 1.0 / N
    pay = [[None] * N for _ in range(N)]  # pay[r][hop]
    for hop in range(N):
        for r in range(N):
            c = (r - hop) % N
            lo, hi = chunk_range(n, N, c)
            if hi <= lo:
                continue
            g = grads[r][lo:hi]
            st = _slice_state(states[r], lo, hi)
            inc = pay[(r - 1) % N][hop - 1] if hop > 0 else None
            if sp.sparse:
                # merge first, then state update + selection in one encode
                acc = st["accum_v"] if "accum_v" in st else st["residual"]
                if inc is not None:
                    comp.decode(inc, acc, accumulate=True)
                pay[r][hop] = comp.encode(g, st, update=True)
            else:
                pay[r][hop] = comp.encode(g, st, incoming=inc, step=step,
                                          salt=salt + r * 256 + hop, tensor_id=tensor_id,
                                          elem_offset=lo)
    outs = [torch.zeros(n, dtype=torch.float32, device=dev) for _ in range(N)]
    for r in range(N):
        for src in range(N):
            c = (src + 1) % N
            lo, hi = chunk_range(n, N, c)
            if hi > lo:
                comp.decode(pay[src][N - 1], outs[r][lo:hi], scale=inv)
    return outs


def simulate_ps(comp: Compressor, grads, states, server_states, *, step=0, salt=0, tensor_id=0):
    """server_states[r]: state dict of rank r for the chunk it owns (length =
    chunk_elems), or an empty dict for no server-side error feedback."""
    N = len(grads)
    n = grads[0].numel()
    sp = comp.spec
    dev = grads[0].device
    inv = 1.0 / N
    push = [[None] * N for _ in range(N)]  # push[src][owner]
    for r in range(N):
        for j in range(N):
            lo, hi = chunk_range(n, N, j)
            if hi <= lo:
                continue
            st = _slice_state(states[r], lo, hi)
            if sp.sparse:
                push[r][j] = comp.encode(grads[r][lo:hi], st, update=True)
            else:
                push[r][j] = comp.encode(grads[r][lo:hi], st, step=step, salt=salt + r * 256,
                                         tensor_id=tensor_id, elem_offset=lo)
    pull = [None] * N
    for j in range(N):
        lo, hi = chunk_range(n, N, j)
        if hi <= lo:
            continue
        m = hi - lo
        sst = {k: v[:m] for k, v in server_states[j].items()}
        if sp.sparse:
            # server accumulator = server-side residual; no momentum on the server
            acc = sst["residual"] if "residual" in sst else torch.zeros(m, device=dev)
            for q in range(N):
                comp.decode(push[q][j], acc, accumulate=True)
            pull[j] = comp.encode(acc, {"residual": acc}, update=False)
        else:
            acc = torch.empty(m, dtype=torch.float32, device=dev)
            for q in range(N):
                comp.decode(push[q][j], acc, accumulate=q > 0)
            pull[j] = comp.encode(acc, sst, step=step, salt=salt + j * 256 + 1,
                                  tensor_id=tensor_id, elem_offset=lo)
    outs = [torch.zeros(n, dtype=torch.float32, device=dev) for _ in range(N)]
    for r in range(N):
        for j in range(N):
            lo, hi = chunk_range(n, N, j)
            if hi > lo:
                comp.decode(pull[j], outs[r][lo:hi], scale=inv)
    return outs
