"""Process bootstrap: one process per GPU over ``torch.distributed`` (NCCL on a GPU
box, gloo on CPU), Horovod-style module functions ``init / rank / size /
local_rank / shutdown``.  A lone process with no launcher environment runs as a
world of one without creating a process group."""
from __future__ import annotations

import datetime
import os
import zlib

import torch
import torch.distributed as dist

_state = {"init": False, "rank": 0, "size": 1, "local_rank": 0, "own_pg": False, "device": None}


def init(backend: str | None = None, timeout_s: float | None = None):
    """Join the job described by RANK / WORLD_SIZE / LOCAL_RANK / MASTER_ADDR /
    MASTER_PORT (as set by ``torch.distributed.run``).  ``timeout_s`` (default 600,
    or HIPRESS_PG_TIMEOUT_S) bounds every collective and message of the process
    group: a peer that never joins ends the call with an error."""
    if _state["init"]:
        return
    if timeout_s is None:
        timeout_s = float(os.environ.get("HIPRESS_PG_TIMEOUT_S", "600"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank_ = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    use_cuda = torch.cuda.is_available()
    if use_cuda:
        torch.cuda.set_device(local % torch.cuda.device_count())
        _state["device"] = torch.device("cuda", torch.cuda.current_device())
    else:
        _state["device"] = torch.device("cpu")
    if dist.is_initialized():
        world, rank_ = dist.get_world_size(), dist.get_rank()
    elif world > 1 or "MASTER_ADDR" in os.environ and "RANK" in os.environ:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29500")
        be = backend or ("nccl" if use_cuda else "gloo")
        kw = {}
        if be == "nccl":
            kw["device_id"] = _state["device"]
        dist.init_process_group(be, rank=rank_, world_size=world,
                                timeout=datetime.timedelta(seconds=timeout_s), **kw)
        _state["own_pg"] = True
    _state.update(init=True, rank=rank_, size=world, local_rank=local)


def shutdown():
    if _state["own_pg"] and dist.is_initialized():
        dist.destroy_process_group()
    _state.update(init=False, rank=0, size=1, local_rank=0, own_pg=False)
    _state.pop("hier", None)


def is_initialized() -> bool:
    return _state["init"]


def rank() -> int:
    return _state["rank"]


def size() -> int:
    return _state["size"]


def local_rank() -> int:
    return _state["local_rank"]


def local_size() -> int:
    """Ranks on this machine (LOCAL_WORLD_SIZE as set by ``torch.distributed.run``;
    every rank of the job on a single box)."""
    return int(os.environ.get("LOCAL_WORLD_SIZE", _state["size"]))


def group_size(group=None) -> int:
    return size() if group is None else dist.get_world_size(group)


def group_rank(group=None) -> int:
    return rank() if group is None else dist.get_rank(group)


def hierarchy():
    """How the job's ranks sit on machines.  Returns ``None`` for a job on one
    machine (or a world of one) and otherwise a dict with

    * ``node_of``: machine index of every rank, ``nodes``: number of machines,
    * ``local_size``: ranks per machine, or ``None`` when machines differ,
    * ``local_group`` / ``cross_group``: this rank's machine-local group and the
      group of the ranks with its local index on every machine (only for equal
      machine sizes above 1).

    Machines are told apart by host name; ``HIPRESS_NODE_ID`` (per rank) or
    ``HIPRESS_NODE_SIZE=K`` (consecutive ranks in groups of K) override it, so one
    machine can stand in for several.  Collective over the job: every rank
    must call it at the same point.  The result is cached."""
    if "hier" in _state:
        return _state["hier"]
    out = None
    if size() > 1:
        import socket
        ident = os.environ.get("HIPRESS_NODE_ID") or socket.gethostname()
        if os.environ.get("HIPRESS_NODE_SIZE"):   # consecutive ranks in groups of K pose as machines
            ident = f"node{rank() // max(1, int(os.environ['HIPRESS_NODE_SIZE']))}"
        ids = [None] * size()
        dist.all_gather_object(ids, ident)
        order = list(dict.fromkeys(ids))
        if len(order) > 1:
            node_of = [order.index(i) for i in ids]
            members = [[r for r, n in enumerate(node_of) if n == k] for k in range(len(order))]
            sizes = {len(m) for m in members}
            out = {"node_of": node_of, "nodes": len(order), "local_size": None,
                   "local_group": None, "cross_group": None}
            if len(sizes) == 1 and len(members[0]) > 1:
                per = len(members[0])
                me = rank()
                # every rank creates every group, in the same order
                locals_ = [dist.new_group(m) for m in members]
                crosses = [dist.new_group([m[j] for m in members]) for j in range(per)]
                out.update(local_size=per, local_group=locals_[node_of[me]],
                           cross_group=crosses[members[node_of[me]].index(me)])
            elif len(sizes) == 1:
                out["local_size"] = 1
    _state["hier"] = out
    return out


def device() -> torch.device:
    return _state["device"] or torch.device("cuda" if torch.cuda.is_available() else "cpu")


def barrier():
    if size() > 1:
        dist.barrier()


def broadcast_parameters(params, root_rank: int = 0):
    """Broadcast a ``state_dict`` or ``named_parameters`` from root to every rank."""
    if size() == 1:
        return
    items = params.items() if isinstance(params, dict) else params
    for _, p in items:
        if torch.is_tensor(p):
            dist.broadcast(p.data if hasattr(p, "data") else p, root_rank)


def broadcast_optimizer_state(optimizer, root_rank: int = 0):
    """Broadcast the tensors of an optimizer's state from root to every rank."""
    if size() == 1:
        return
    opt = getattr(optimizer, "optimizer", optimizer)
    obj = [opt.state_dict() if rank() == root_rank else None]
    dist.broadcast_object_list(obj, src=root_rank)
    if rank() != root_rank:
        opt.load_state_dict(obj[0])
        if hasattr(optimizer, "_relink"):
            optimizer._relink()


_syncers: dict = {}


def allreduce(tensor: torch.Tensor, average: bool = True, name: str | None = None,
              algorithm: str | None = None, topology: str = "ring", **algorithm_kwargs) -> torch.Tensor:
    """Horovod-style ``allreduce``: returns the sum (or average) of `tensor` over all
    ranks.  With ``algorithm`` set ("tbq", "onebit", ...) the tensor travels
    compressed through the CaSync schedule; ``name`` keys the error-feedback state
    that is kept between calls."""
    out = tensor.clone()
    if size() == 1 and algorithm is None:
        return out
    if algorithm is None:
        return allreduce_(out, average)
    from ..config import HipressConfig
    from .hooks import FlatSyncer
    key = (algorithm, topology, tuple(sorted(algorithm_kwargs.items())))
    if key not in _syncers:
        cfg = HipressConfig(algorithm=algorithm, topology=topology, comp_threshold=0)
        for k, v in algorithm_kwargs.items():
            setattr(cfg, k, v)
        _syncers[key] = FlatSyncer(cfg)
    flat = out.reshape(-1).float().contiguous()
    # a stable key (str hashes differ between processes and runs); the element count is
    # part of it, so unnamed tensors of different sizes never share error-feedback state
    _syncers[key].sync_(flat, key=zlib.crc32(f"{name or ''}#{flat.numel()}".encode()) % (1 << 20))
    if not average:
        flat.mul_(size())
    return flat.view_as(out).to(tensor.dtype)


def broadcast(tensor: torch.Tensor, root_rank: int = 0) -> torch.Tensor:
    """Horovod-style ``broadcast``: returns root's tensor on every rank."""
    out = tensor.clone()
    if size() > 1:
        dist.broadcast(out, root_rank)
    return out


def allgather(tensor: torch.Tensor) -> torch.Tensor:
    """Horovod-style ``allgather``: concatenation along dim 0 of every rank's tensor;
    the first dimension may differ between ranks, the others must agree."""
    if size() == 1:
        return tensor.clone()
    t = tensor.contiguous()
    rows = torch.tensor([t.shape[0] if t.dim() else 1], dtype=torch.int64, device=t.device)
    every = [torch.empty_like(rows) for _ in range(size())]
    dist.all_gather(every, rows)
    counts = [int(r.item()) for r in every]
    if len(set(counts)) == 1:
        parts = [torch.empty_like(t) for _ in range(size())]
        dist.all_gather(parts, t)
        return torch.cat([p.reshape(-1, *t.shape[1:]) if not t.dim() else p for p in parts], dim=0)
    most = max(counts)
    padded = torch.zeros((most, *t.shape[1:]), dtype=t.dtype, device=t.device)
    padded[:t.shape[0]] = t
    parts = [torch.empty_like(padded) for _ in range(size())]
    dist.all_gather(parts, padded)
    return torch.cat([p[:c] for p, c in zip(parts, counts)], dim=0)


def broadcast_object(obj, root_rank: int = 0):
    """Horovod-style ``broadcast_object``: root's picklable object on every rank."""
    if size() == 1:
        return obj
    box = [obj if rank() == root_rank else None]
    dist.broadcast_object_list(box, src=root_rank)
    return box[0]


def allgather_object(obj) -> list:
    """Horovod-style ``allgather_object``: every rank's picklable object, by rank."""
    if size() == 1:
        return [obj]
    out = [None] * size()
    dist.all_gather_object(out, obj)
    return out


def allreduce_(t: torch.Tensor, average: bool = True):
    """Plain (uncompressed) in-place all-reduce."""
    if size() > 1:
        dist.all_reduce(t)
        if average:
            t.div_(size())
    return t
