"""Gradient-hook flavours of the synchronisation API.

* :func:`ddp_comm_hook` plugs compressed synchronisation into
  ``torch.nn.parallel.DistributedDataParallel.register_comm_hook``: every DDP
  bucket (a flat fp32 tensor) is synchronised with the CaSync schedule and its
  compressor state is kept per bucket index.
* :class:`FlatSyncer` is the object behind it and can be used directly to
  synchronise any flat gradient tensor (for example from a raw
  ``register_post_accumulate_grad_hook``); it also serves
  ``hp.allreduce(..., algorithm=)``.  On GPUs both run the fused kernels.

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
    """Synchronises flat fp32 gradient tensors, keyed by the caller (a DDP bucket
    index, a name).  On CUDA every key gets a region of symmetric memory on first use
    and is synchronised by ONE fused launch (encode + peer stores + decode-aggregate,
    the same kernels the DistributedOptimizer uses); on CPU ranks, for registered
    custom algorithms and with ``backend="host"`` the schedule runs from decoupled
    primitives around messages.  Every rank must present the same keys in the same
    order the first time (the regions are allocated collectively)."""

    def __init__(self, config=None, group=None):
        self.cfg = config or HipressConfig()
        self.group = group
        from ..ops.custom import custom_compressor
        self._custom = custom_compressor(self.cfg.algorithm)
        self.comp = self._custom or \
            Compressor(get_algorithm(self.cfg.algorithm, **self.cfg.algorithm_kwargs()))
        self.sched = None
        self.state = {}
        self.step = 0
        self._fused = {}        # key -> (impl, arena, status)
        self.stream = None      # communication stream of the DDP hook
        self.launch_count = 0

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

    def _use_fused(self, flat) -> bool:
        return flat.is_cuda and self._custom is None and self.cfg.backend in ("auto", "fused")

    def _fused_impl(self, key, n, device):
        ent = self._fused.get(key)
        if ent is not None and ent[0].sizes[0] == n:
            return ent
        if ent is not None:
            ent[1].close()
        from .fused import FusedDenseBucket
        from .fused_sparse import FusedSparseBucket
        from .symm import SymmetricArena
        N, R = comm.group_size(self.group), comm.group_rank(self.group)
        sp, cfg = self.comp.spec, self.cfg
        status = torch.zeros(4, dtype=torch.int32, device=device)
        if sp.sparse:
            impl = FusedSparseBucket(sp, [n], N, R, timeout_s=cfg.timeout_s, topology=cfg.topology)
        else:
            impl = FusedDenseBucket(sp, cfg.topology, [n], N, R, ctas=cfg.ctas, timeout_s=cfg.timeout_s)
        arena = SymmetricArena(impl.region_bytes() + 8192, self.group)
        region = arena.carve(impl.region_bytes())
        impl.bind(region, status, device) if sp.sparse else impl.bind(region, status)
        ent = (impl, arena, status)
        self._fused[key] = ent
        return ent

    def _sync_fused(self, flat, key, stream=None):
        n = flat.numel()
        s, server, _ = self._state(key, n, flat.device)
        impl, _, _ = self._fused_impl(key, n, flat.device)
        sp = self.comp.spec
        g = flat.data_ptr()
        if sp.sparse:
            acc = s["accum_v"] if "accum_v" in s else s["residual"]
            u = s.get("momentum_u")
            sr = server.get("residual")
            if sr is None and self.cfg.topology == "ps":   # the owner always needs an accumulator
                sr = server.setdefault("_scratch", torch.zeros(
                    chunk_elems(n, comm.group_size(self.group)), dtype=torch.float32, device=flat.device))
                if stream is not None:
                    with torch.cuda.stream(stream):
                        sr.zero_()
                else:
                    sr.zero_()
            impl.launch_ptrs([g], [acc.data_ptr()], None if u is None else [u.data_ptr()], [g],
                             [None if sr is None else sr.data_ptr()], stream=stream)
        else:
            r = s.get("residual")
            sr = server.get("residual")
            impl.launch_ptrs([g], [None if r is None else r.data_ptr()], [g],
                             [None if sr is None else sr.data_ptr()], step=self.step,
                             tensor_ids=[int(key) * 64], stream=stream)
        self.launch_count += 1

    def sync_(self, flat: torch.Tensor, key=0, stream=None) -> torch.Tensor:
        """Averages `flat` (fp32, contiguous) across the ranks of the group in place,
        compressed when it has at least comp_threshold elements.  ``stream``: launch
        there instead of on the current stream (the caller orders the streams)."""
        n = flat.numel()
        if n < self.cfg.comp_threshold or flat.dtype != torch.float32:
            # average over the ranks of THIS syncer's group (a sub-group, a DDP
            # process_group), not over the whole job
            N = comm.group_size(self.group)
            ctx = torch.cuda.stream(stream) if stream is not None else _null()
            with ctx:
                if N > 1:
                    dist.all_reduce(flat, group=self.group)
                    flat.div_(N)
            return flat
        if self._use_fused(flat):
            self._sync_fused(flat.view(-1), key, stream)
            return flat
        if self.sched is None:
            self.sched = HostSchedule(self.comp, self.cfg.topology, self.group)
        s, server, _ = self._state(key, n, flat.device)
        ctx = torch.cuda.stream(stream) if stream is not None else _null()
        with ctx:
            self.sched.sync([SegView(flat.view(-1), s, server, int(key) * 64)], step=self.step)
        return flat

    def check(self):
        """Blocking check of the fused kernels' status words and guard words."""
        from .fused import HipressTimeoutError, decode_status
        for impl, arena, status in self._fused.values():
            arena.check_guards()
            words = [w & 0xFFFFFFFF for w in status.cpu().tolist()]
            if any(words):
                status.zero_()
                raise HipressTimeoutError(decode_status(next(w for w in words if w)))

    def close(self, collective: bool = True):
        for _, arena, _ in self._fused.values():
            arena.close(collective=collective)
        self._fused = {}


def _null():
    import contextlib
    return contextlib.nullcontext()


def ddp_comm_hook(state: FlatSyncer, bucket: dist.GradBucket) -> torch.futures.Future[torch.Tensor]:
    """``model.register_comm_hook(FlatSyncer(cfg), ddp_comm_hook)``

    On CUDA the bucket is synchronised on the syncer's own high-priority stream, behind
    an event recorded where DDP finished filling the bucket, so it overlaps the rest of
    backward; the returned future completes with that stream's work."""
    buf = bucket.buffer()
    idx = bucket.index()
    if idx == 0:
        state.step += 1
    if not buf.is_cuda:
        state.sync_(buf, key=idx)
        fut = torch.futures.Future()
        fut.set_result(buf)
        return fut
    if state.stream is None:
        state.stream = torch.cuda.Stream(priority=-1)
    ready = torch.cuda.Event()
    ready.record()
    state.stream.wait_event(ready)
    state.sync_(buf, key=idx, stream=state.stream)
    fut = torch.futures.Future(devices=[buf.device])
    with torch.cuda.stream(state.stream):
        fut.set_result(buf)     # marks completion with the communication stream's work
    return fut
