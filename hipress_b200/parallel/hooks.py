"""Gradient-hook flavours of the synchronisation API.

* :func:`ddp_comm_hook` plugs compressed synchronisation into
  ``torch.nn.parallel.DistributedDataParallel.register_comm_hook``: every DDP
  bucket (a flat fp32 tensor) is synchronised with the CaSync schedule and its
  compressor state is kept per bucket index.
* :class:`FlatSyncer` is the object behind it and can be used directly to
  synchronise any flat gradient tensor (for example from a raw
  ``register_post_accumulate_grad_hook``).

Reference parity: the reference offers only the Horovod optimizer wrapper
(README.md:184-186 of mark14wu/hipress); a DDP hook is the idiomatic PyTorch
equivalent of its per-gradient callbacks.
"""
import torch
import torch.distributed as dist

from ..config import HipressConfig
from ..ops.algorithms import get_algorithm
from ..ops.compressor import Compressor
from . import comm
from .host_schedule import HostSchedule, SegView
from .simulate import chunk_elems


class FlatSyncer:
    def __init__(self, config=None, group=None):
        self.cfg = config or HipressConfig()
        self.group = group
        from ..ops.custom import custom_compressor
        self.comp = custom_compressor(self.cfg.algorithm) or \
            Compressor(get_algorithm(self.cfg.algorithm, **self.cfg.algorithm_kwargs()))
        self.sched = None
        self.state = {}
        self.step = 0

    def _state(self, key, n, device):
        st = self.state.get(key)
        if st is None or st[2] != n:
            N = comm.group_size(self.group)
            sp = self.comp.spec
            s = {k: torch.zeros(n, dtype=torch.float32, device=device) for k in sp.state_names()}
            server = {}
            if self.cfg.topology == "ps" and self.cfg.server_residual and \
                    (sp.sparse or "residual" in sp.state_names()):
                server = {"residual": torch.zeros(chunk_elems(n, N), dtype=torch.float32, device=device)}
            st = (s, server, n)
            self.state[key] = st
        return st

    def sync_(self, flat: torch.Tensor, key=0) -> torch.Tensor:
        """Averages `flat` (fp32, contiguous) across ranks in place, compressed
        when it has at least comp_threshold elements."""
        if self.sched is None:
            self.sched = HostSchedule(self.comp, self.cfg.topology, self.group)
        n = flat.numel()
        if n < self.cfg.comp_threshold or flat.dtype != torch.float32:
            # average over the ranks of THIS syncer's group (a sub-group, a DDP
            # process_group), not over the whole job
            N = comm.group_size(self.group)
            if N > 1:
                dist.all_reduce(flat, group=self.group)
                flat.div_(N)
            return flat
        s, server, _ = self._state(key, n, flat.device)
        self.sched.sync([SegView(flat.view(-1), s, server, int(key) * 64)], step=self.step)
        return flat


def ddp_comm_hook(state: FlatSyncer, bucket: dist.GradBucket) -> torch.futures.Future[torch.Tensor]:
    """``model.register_comm_hook(FlatSyncer(cfg), ddp_comm_hook)``"""
    buf = bucket.buffer()
    idx = bucket.index()
    if idx == 0:
        state.step += 1
    state.sync_(buf, key=idx)
    fut = torch.futures.Future()
    fut.set_result(buf)
    return fut
