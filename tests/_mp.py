"""Helpers to run a function as several ranks (child processes) on this machine."""
import os
import socket
import tempfile

import torch
import torch.multiprocessing as mp


def free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _entry(rank, world, port, fn, outdir, backend, args, env):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank),
                      WORLD_SIZE=str(world), LOCAL_RANK=str(rank))
    os.environ.update(env or {})
    torch.set_num_threads(1)
    import hipress_b200 as hp
    hp.init(backend=backend)
    try:
        res = fn(rank, world, *args)
        torch.save(res, os.path.join(outdir, f"r{rank}.pt"))
    finally:
        hp.shutdown()


def spawn(fn, world, *args, backend="gloo", env=None):
    """Run fn(rank, world, *args) in `world` processes; returns their results."""
    port = free_port()
    with tempfile.TemporaryDirectory() as d:
        mp.spawn(_entry, args=(world, port, fn, d, backend, args, env), nprocs=world, join=True)
        return [torch.load(os.path.join(d, f"r{r}.pt"), weights_only=False) for r in range(world)]
