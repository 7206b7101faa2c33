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


def _parse_set(text) -> set:
    text = text.decode() if isinstance(text, bytes) else text
    return {int(x) for x in text.split(",") if x != ""}


def survivors_rendezvous(store, old_rank: int, old_world: int, dead, *, generation: int,
                         timeout_s: float = 30.0, prefix: str = "hipress"):
    """Every survivor calls this with the peers IT saw fail (PeerFailure.ranks) and the
    same `generation` (a counter that grows with every recovery).  The survivors need
    not have seen the same failures: each publishes its own set in the job's store, and
    the membership everyone adopts is built from the union of the published sets --
    a rank waits until every rank that is alive by the union has published, and
    widens the union with whatever those ranks reported (two peers that fail close
    together, or a departure one rank read from the store and another only noticed
    as a missed heartbeat, no longer split the survivors).  The first rank to finish
    records the result under ``final``; a rank that arrives at a different one adopts
    the union and goes round again.  Returns (new_rank, new_world): survivors keep
    their relative order."""
    key = f"{prefix}/gen{generation}"
    union = set(dead)
    if old_rank in union:
        raise RuntimeError("a rank that was declared dead cannot rejoin")
    store.set(f"{key}/dead/{old_rank}", ",".join(map(str, sorted(union))))
    t0 = time.time()
    while True:
        # widen the union with the reports of every rank that is alive by it
        grew = True
        missing = []
        while grew:
            grew = False
            missing = []
            for r in range(old_world):
                if r in union or r == old_rank:
                    continue
                if store.check([f"{key}/dead/{r}"]):
                    more = _parse_set(store.get(f"{key}/dead/{r}")) - union
                    if more:
                        union |= more
                        grew = True
                else:
                    missing.append(r)
        if old_rank in union:
            raise RuntimeError(f"rank {old_rank} was declared dead by a peer and cannot rejoin")
        if not missing:
            mine = ",".join(map(str, sorted(union)))
            agreed = store.compare_set(f"{key}/final", "", mine)
            agreed = agreed.decode() if isinstance(agreed, bytes) else agreed
            if agreed == mine:
                break
            other = _parse_set(agreed)
            if other <= union:            # somebody finished with less: it will notice and come back
                store.set(f"{key}/final", mine)
                break
            union |= other
            continue
        if time.time() - t0 > timeout_s:
            raise TimeoutError(f"survivors {missing} never reached the rendezvous "
                               f"(declared dead so far: {sorted(union)})")
        time.sleep(0.02)
    alive = [r for r in range(old_world) if r not in union]
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
