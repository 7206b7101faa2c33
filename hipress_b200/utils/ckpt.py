"""Checkpoint / resume.

Layout (Horovod / torch convention: rank 0 owns the replicated state):

    <dir>/model.pt            {'model', 'optimizer', 'epoch', 'step', 'config'}   written by rank 0
    <dir>/rank{r}.pt          {'compressor_state': {param_name: {'residual' | 'momentum_u' |
                               'accum_v' | 'server_residual.<part>': fp32 tensor, 'step': int}}}

Compressor state is rank-local error memory, keyed by parameter name like the
reference keys its plans by gradient name (src/SeCoPa/input.txt of
mark14wu/hipress).  It is dropped with a warning when the world size or the
algorithm changed.  The reference ships no checkpoint code or flag; this layout is
the least surprising one for its Horovod lineage.
"""
from __future__ import annotations

import os
from pathlib import Path

import torch

from ..parallel import comm


def save_checkpoint(directory, model, optimizer, *, epoch=0, step=0, extra=None):
    d = Path(directory)
    d.mkdir(parents=True, exist_ok=True)
    inner = getattr(optimizer, "optimizer", optimizer)
    if getattr(optimizer, "engine", None) is not None:
        # nothing is written while a device-side wait has expired or a region of the
        # symmetric arena was overrun: raises HipressTimeoutError / RuntimeError
        optimizer.engine.check()
    if comm.rank() == 0:
        tmp = d / "model.pt.tmp"
        torch.save({"model": model.state_dict(), "optimizer": inner.state_dict(), "epoch": epoch,
                    "step": step, "config": dict(vars(optimizer.config)) if hasattr(optimizer, "config")
                    else {}, "extra": extra}, tmp)
        os.replace(tmp, d / "model.pt")
    if hasattr(optimizer, "engine"):
        tmp = d / f"rank{comm.rank()}.pt.tmp"
        torch.save({"compressor_state": optimizer.engine.state_dict()}, tmp)
        os.replace(tmp, d / f"rank{comm.rank()}.pt")
    comm.barrier()


def load_checkpoint(directory, model, optimizer, map_location=None) -> dict:
    """Restores model, optimizer and (when compatible) compressor state; returns
    {'epoch', 'step', 'extra'}.  Every rank reads model.pt, so all start identical."""
    d = Path(directory)
    ck = torch.load(d / "model.pt", map_location=map_location or "cpu", weights_only=False)
    model.load_state_dict(ck["model"])
    inner = getattr(optimizer, "optimizer", optimizer)
    inner.load_state_dict(ck["optimizer"])
    if hasattr(optimizer, "_relink"):
        optimizer._relink()
    mine = d / f"rank{comm.rank()}.pt"
    if hasattr(optimizer, "engine"):
        if mine.exists():
            st = torch.load(mine, map_location="cpu", weights_only=False)
            optimizer.engine.load_state_dict(st["compressor_state"])
        else:
            import logging
            logging.getLogger("hipress").warning(
                "no compressor state for rank %d in %s; residuals start at zero", comm.rank(), d)
    return {"epoch": ck.get("epoch", 0), "step": ck.get("step", 0), "extra": ck.get("extra")}
