"""Run-time correctness evidence for a multi-GPU job, cheap enough to run at the end
of a benchmark:

* :func:`replicas_identical` -- every rank holds bit-identical parameters;
* :func:`one_step_check`     -- on one extra step, what the compressed
  synchronisation delivered plus what the ranks kept back as error-feedback state
  equals the exact mean of the ranks' gradients.

The second check rests on the conservation law of error feedback.  Every rank feeds
``g_k + r_k`` into the schedule (``m*u_k + g_k`` on top of the accumulator for DGC's
momentum correction); every encode, at any hop and at a PS owner, keeps its
quantisation or selection error in a residual.  So, summed over ranks,

    sum_k input_k  =  N * delivered  +  sum_k (r_k' - r_k)  +  (owner residual changes)

and ``delivered + mean(delta state)`` must equal the exact mean up to fp32 rounding,
whatever the algorithm dropped on the wire.  TernGrad keeps no residual (it is
unbiased instead), so for it the figure is the relative quantisation error itself.

The reference has no counterpart: it ships no test or self-check of any kind
(the only ``assert`` statements of mark14wu/hipress are parser invariants,
src/CompLL/GCGen/tree.py:34-102).
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from ..parallel import comm
from ..parallel.engine import _flat
from ..parallel.simulate import chunk_range


def parameter_checksum(model: torch.nn.Module, buffers: bool = False) -> int:
    """64-bit wrap-around sum of the raw bits of every parameter (and, on request,
    buffer).  Buffers are left out by default: batch-norm running statistics follow each
    rank's own data and are not synchronised, here as under Horovod."""
    tot = torch.zeros((), dtype=torch.int64, device=next(model.parameters()).device)
    for t in list(model.parameters()) + (list(model.buffers()) if buffers else []):
        if t.numel() == 0:
            continue
        flat = t.detach().contiguous().view(-1)
        if flat.element_size() == 4:
            tot += flat.view(torch.int32).to(torch.int64).sum()
        elif flat.element_size() == 2:
            tot += flat.view(torch.int16).to(torch.int64).sum()
        elif flat.element_size() == 8:
            tot += flat.view(torch.int64).sum()
        else:
            tot += flat.view(torch.uint8).to(torch.int64).sum()
    return int(tot.item())


def replicas_identical(model: torch.nn.Module, buffers: bool = False) -> bool:
    """True when every rank's parameters have the same checksum."""
    mine = parameter_checksum(model, buffers)
    if comm.size() == 1:
        return True
    every = [None] * comm.size()
    dist.all_gather_object(every, mine)
    return all(c == every[0] for c in every)


def _sum_over_ranks(t: torch.Tensor, group=None) -> torch.Tensor:
    if comm.size() > 1:
        dist.all_reduce(t, group=group)
    return t


@torch.no_grad()
def _snapshot(engine):
    """Clones of every compressor state tensor (per entry, and per PS segment)."""
    snap = {}
    for e in engine.entries:
        snap[e.name] = ({k: v.clone() for k, v in e.state.items()},
                        [{k: v.clone() for k, v in sst.items() if torch.is_tensor(v)}
                         for sst in e.server_state])
    return snap


def one_step_check(job, x, y) -> dict:
    """Runs one more training step's forward and backward on (x, y) twice: once with
    ``torch.autograd.grad`` (no hooks fire, so the raw local gradients are seen) and
    once through the engine.  Returns ``one_step_rel_err`` =
    ||delivered + mean(delta state) - exact mean|| / ||exact mean|| over all
    compressed gradients, ``plain_rel_err`` the same for the uncompressed ones, and
    the element counts.  No optimizer step is taken; compressor state advances by one
    step as it would in training."""
    import torch.nn.functional as F
    opt = job.optimizer
    eng = opt.engine
    N = eng.world
    model = job.model
    if eng.outer is not None:
        return {"one_step_rel_err": None, "note": "not defined for the hierarchical mode"}
    was_training = model.training
    model.eval()            # no batch-norm statistics update, same function both times
    params = [e.param for e in eng.entries]

    def loss_fn():
        with torch.autocast(job.device.type, dtype=job.dtype, enabled=job.dtype != torch.float32):
            if job.kind == "image":
                return F.cross_entropy(model(x).float(), y)
            return model(x, y)

    opt.zero_grad(set_to_none=True)
    raw = torch.autograd.grad(loss_fn(), params, allow_unused=True)
    raw = [torch.zeros_like(p) if g is None else g.detach().float() for p, g in zip(params, raw)]
    spec = eng.comp.spec if eng.compress else None
    before = _snapshot(eng)
    opt.zero_grad(set_to_none=True)
    loss_fn().backward()
    eng.synchronize()
    if eng.on_cuda:
        torch.cuda.synchronize()
    num = den = pnum = pden = 0.0
    n_comp = n_plain = 0
    fused_entries = {id(e) for b in eng.buckets if b.fused for e in b.entries}
    for e, g in zip(eng.entries, raw):
        pg = e.param.grad.detach()
        cl = pg.dim() == 4 and not pg.is_contiguous() and pg.is_contiguous(memory_format=torch.channels_last)
        g = g.contiguous(memory_format=torch.channels_last) if cl else g.contiguous()
        delivered, flat = _flat(pg).float(), _flat(g)   # the engine works in the gradient's memory order
        if id(e) not in fused_entries:
            exact = _sum_over_ranks(flat.clone(), eng.world_group) / N
            pnum += float((delivered - exact).double().pow(2).sum())
            pden += float(exact.double().pow(2).sum())
            n_plain += e.numel
            continue
        st0, sst0 = before[e.name]
        target = flat.clone()
        if spec is not None and "momentum_u" in e.state:       # DGC: the schedule carries m*u + g
            target = spec.momentum * st0["momentum_u"] + flat
        key = "accum_v" if "accum_v" in e.state else ("residual" if "residual" in e.state else None)
        kept = torch.zeros_like(target)
        if key is not None:
            kept += e.state[key] - st0[key]
        segs = [s for b in eng.buckets if b.fused for s in b.segs if s.entry is e]
        for s in segs:
            if not e.server_state:
                continue
            sst = e.server_state[s.part]
            if "residual" in sst and "residual" in sst0[s.part]:
                lo, hi = chunk_range(s.n, eng.N, eng.R)
                if hi > lo:
                    d = sst["residual"][:hi - lo] - (0 if sst.get("_scratch") else sst0[s.part]["residual"][:hi - lo])
                    kept[s.lo + lo:s.lo + hi] += d
        exact = _sum_over_ranks(target, eng.world_group) / N
        kept = _sum_over_ranks(kept, eng.world_group) / N
        num += float((delivered + kept - exact).double().pow(2).sum())
        den += float(exact.double().pow(2).sum())
        n_comp += e.numel
    opt.zero_grad(set_to_none=True)
    model.train(was_training)
    return {"one_step_rel_err": (num / den) ** 0.5 if den > 0 else None,
            "plain_rel_err": (pnum / pden) ** 0.5 if pden > 0 else None,
            "compressed_elems": n_comp, "plain_elems": n_plain}
