"""Recovery after a peer left or died: the survivors agree on the new membership
through the job's key-value store, tear the process group down and form a smaller
one, then rebuild their optimizers (compressor state is rank-local error memory
and is dropped when the world size changes) and continue, usually from the last
checkpoint.  Everything happens on the host, between steps, with nothing in flight
on any GPU.

Nearest upstream analogue: Elastic Horovod; the reference tree has no such code.
"""
from __future__ import annotations

import datetime
import logging
import os
import time

import torch
import torch.distributed as dist

from . import comm

log = logging.getLogger("hipress")


def survivors_rendezvous(store, old_rank: int, old_world: int, dead, *, generation: int,
                         timeout_s: float = 30.0, prefix: str = "hipress"):
    """Every survivor calls this with the same `dead` set (from PeerFailure.ranks) and
    `generation` (a counter that grows with every recovery).  Returns (new_rank,
    new_world): survivors keep their relative order."""
    dead = set(dead)
    alive = [r for r in range(old_world) if r not in dead]
    if old_rank not in alive:
        raise RuntimeError("a rank that was declared dead cannot rejoin")
    key = f"{prefix}/gen{generation}"
    store.add(f"{key}/joined", 1)
    t0 = time.time()
    while int(store.add(f"{key}/joined", 0)) < len(alive):
        if time.time() - t0 > timeout_s:
            raise TimeoutError(f"only {int(store.add(key + '/joined', 0))} of {len(alive)} survivors "
                               "reached the rendezvous")
        time.sleep(0.02)
    return alive.index(old_rank), len(alive)


def reform_process_group(new_rank: int, new_world: int, *, port: int, backend: str | None = None,
                         timeout_s: float = 60.0):
    """Destroys the current process group and creates one of the new size on
    127.0.0.1:`port` (all survivors must pass the same fresh port)."""
    if dist.is_initialized():
        # abort rather than drain: collectives with the dead rank would never finish
        try:
            dist.destroy_process_group()
        except Exception as e:  # pragma: no cover - best effort
            log.warning("destroy_process_group: %s", e)
    comm._state.update(init=False, own_pg=False)
    comm._state.pop("hier", None)   # the machine layout is rediscovered for the new membership
    os.environ.update(RANK=str(new_rank), WORLD_SIZE=str(new_world), MASTER_ADDR="127.0.0.1",
                      MASTER_PORT=str(port))
    if new_world > 1:
        be = backend or ("nccl" if torch.cuda.is_available() else "gloo")
        dist.init_process_group(be, rank=new_rank, world_size=new_world,
                                timeout=datetime.timedelta(seconds=timeout_s))
        comm._state.update(own_pg=True)
    comm._state.update(init=True, rank=new_rank, size=new_world)
    return new_rank, new_world
