"""CaSync runtime: turns the parameters of a model into buckets, launches each
bucket's synchronisation as soon as its gradients exist (from autograd hooks, on a
communication stream that overlaps the rest of backward) and hands averaged
gradients to the optimizer.

Per gradient the plan decides compressed or not (SeCoPa plan file or a size
threshold) and the number of partitions K.  Compressed gradients go through

* ``fused``  : one persistent sm_100a kernel per bucket (encode + peer-to-peer
               transfer + decode-aggregate, csrc/cuda/fused_dense.cu); sparse
               algorithms use the fused sparse kernels when present, else ``host``;
* ``host``   : the same schedule from separate encode / decode calls around
               ``torch.distributed`` messages (CPU/gloo ranks and the unfused GPU
               baseline);
* ``allreduce``: no compression, plain all-reduce (the uncompressed baseline).

A job that spans several machines (the reference's usual deployment: one GPU per
machine over Ethernet, README.md:29-45) is handled in two ways.  With one rank per
machine the ``host`` schedule carries the compressed payloads over the network
transport.  With several ranks per machine the engine works hierarchically: the
fused kernels (or the host schedule on CPU ranks) average a bucket inside the
machine, every local rank then takes one 1/L shard of each tensor through a
compressed exchange with the ranks of the same local index on the other
machines, and an all-gather inside the machine hands every rank the full result.
Peer-mapped memory never leaves a machine.

Uncompressed gradients always use a bucketed plain all-reduce, as in the
reference ("PS-Lite and NCCL are used", README.md:153 of mark14wu/hipress).
Every rank launches buckets in the same fixed order; the order of parameter names
is checked across ranks once at start-up, so no per-step negotiation is needed
(the reference inherits Horovod's background coordinator for that).
"""
from __future__ import annotations

import logging
from dataclasses import dataclass, field

import torch
import torch.distributed as dist

from ..config import HipressConfig
from ..ops.algorithms import get_algorithm
from ..ops.compressor import TILE, Compressor
from ..secopa.planner import read_plan
from . import comm
from .host_schedule import HostSchedule, SegView
from .simulate import chunk_elems
from ..utils.timeline import Timeline, nvtx_range

log = logging.getLogger("hipress")
MAX_SEGS = 40


@dataclass
class Entry:
    name: str
    param: torch.nn.Parameter
    numel: int
    compress: bool
    partitions: int
    index: int
    state: dict = field(default_factory=dict)         # name -> flat fp32 [numel]
    server_state: list = field(default_factory=list)  # per partition: dict of owner-side state


@dataclass
class Segment:
    entry: Entry
    lo: int
    hi: int
    part: int

    @property
    def n(self):
        return self.hi - self.lo

    @property
    def seg_id(self):
        return self.entry.index * 64 + self.part


@dataclass
class Bucket:
    index: int
    fused: bool
    entries: list = field(default_factory=list)
    segs: list = field(default_factory=list)
    pending: int = 0
    launched: bool = False
    impl: object = None
    flat: torch.Tensor | None = None
    work: object = None
    stream: object = None
    # hierarchical mode: per segment (lo, hi, state, owner state) of this rank's shard,
    # and the staging buffers of the all-gather inside the machine
    outer: list = field(default_factory=list)
    ag_in: torch.Tensor | None = None
    ag_out: list = field(default_factory=list)


def _flat(t: torch.Tensor) -> torch.Tensor:
    """Memory-order 1-D view of a dense tensor (any memory format)."""
    if t.is_contiguous():
        return t.view(-1)
    return t.as_strided((t.numel(),), (1,))


def split_partitions(n: int, k: int):
    """k contiguous parts with tile-aligned boundaries (fewer when n is small)."""
    k = max(1, min(k, (n + TILE - 1) // TILE))
    per = ((n + k - 1) // k + TILE - 1) // TILE * TILE
    out, lo = [], 0
    while lo < n:
        out.append((lo, min(n, lo + per)))
        lo += per
    return out


class GradSyncEngine:
    def __init__(self, named_parameters, config: HipressConfig | None = None, group=None,
                 backward_passes_per_step: int = 1):
        self.cfg = cfg = config or HipressConfig()
        self.passes = max(1, int(backward_passes_per_step))
        if not comm.is_initialized():
            comm.init()
        self.world_group = group          # plain buckets and consistency checks span the whole job
        self.outer = None                 # hierarchical mode: the exchange between machines
        force_host = False
        if group is None and cfg.hierarchical != "off" and comm.size() > 1 and \
                cfg.algorithm not in ("none", None, ""):
            h = comm.hierarchy()
            if h is not None and h["local_group"] is not None:
                group = h["local_group"]
                self.outer = {"group": h["cross_group"], "nodes": h["nodes"], "local": h["local_size"]}
            elif h is not None and cfg.backend in ("auto", "fused"):
                if cfg.hierarchical == "on" and h["local_size"] != 1:
                    raise ValueError("hierarchical synchronisation needs the same number of ranks "
                                     "on every machine")
                log.info("ranks sit on %d machines: compressed payloads travel over the host "
                         "transport", h["nodes"])
                force_host = True         # peer-mapped memory does not cross machines
        self.N, self.R, self.group = comm.group_size(group), comm.group_rank(group), group
        self.world, self.world_rank = comm.group_size(self.world_group), comm.group_rank(self.world_group)
        named = [(n, p) for n, p in named_parameters if p.requires_grad]
        if not named:
            raise ValueError("no trainable parameters")
        seen_names, seen_params = set(), set()
        for n, p in named:
            if n in seen_names:
                raise ValueError(f"parameter name {n!r} appears twice: names key plans, state and "
                                 "checkpoints and must be unique")
            if id(p) in seen_params:
                raise ValueError(f"parameter {n!r} was passed twice (a shared tensor is listed once)")
            seen_names.add(n)
            seen_params.add(id(p))
        self.device = named[0][1].device
        self.on_cuda = self.device.type == "cuda"
        self.compress = cfg.algorithm not in ("none", None, "")
        from ..ops.custom import custom_compressor
        custom = custom_compressor(cfg.algorithm) if self.compress else None
        self.comp = custom or (Compressor(get_algorithm(cfg.algorithm, **cfg.algorithm_kwargs()))
                               if self.compress else None)
        backend = cfg.backend
        if force_host or custom is not None:
            # user-registered algorithms run from decoupled primitives: there is no
            # fused kernel for an encode/decode pair the runtime has never seen
            if custom is not None and backend == "fused":
                raise ValueError(f"{cfg.algorithm} is a registered algorithm: it has no fused backend")
            backend = "host"
        if backend == "auto":
            backend = "fused" if self.on_cuda else "host"
        if backend == "fused" and not self.on_cuda:
            raise ValueError("the fused backend needs CUDA tensors")
        if not self.compress:
            backend = "allreduce"
        self.backend = backend
        self.step_no = 0
        self.entries = self._make_entries(named)
        self._check_order()
        self.buckets = self._make_buckets()
        self._alloc_state()
        self.comm_stream = torch.cuda.Stream(priority=-1) if self.on_cuda else None
        self.arena = None
        self._setup_backend()
        self._next = 0
        self._hooks = []
        self._by_param = {}
        for b in self.buckets:
            for e in b.entries:
                self._by_param[e.param] = b
        if cfg.overlap:
            for e in self.entries:
                self._hooks.append(e.param.register_post_accumulate_grad_hook(self._on_grad))
        self._begin()
        # called as on_bucket_done(bucket) with the bucket's averaged gradients
        # next in order on the current stream (DistributedOptimizer's overlapped step)
        self.on_bucket_done = None
        self.launch_count = 0
        self.bytes_sent = 0
        self.timeline = Timeline()
        self._events = [torch.cuda.Event() for _ in self.buckets] if self.on_cuda else []

    # ------------------------------------------------------------------ plan
    def _make_entries(self, named):
        cfg = self.cfg
        plan = None
        self.plan_source = "comp_threshold"     # what decided: reported by stats()
        if cfg.plan in ("auto", "auto:bucketed"):
            plan = self._auto_plan(named, bucketed=cfg.plan.endswith("bucketed"))
            if plan is not None:
                self.plan_source = f"{cfg.plan} ({self._plan_profile_name})"
        elif cfg.plan:
            plan = read_plan(cfg.plan)
            self.plan_source = str(cfg.plan)
        entries = []
        for i, (name, p) in enumerate(named):
            n = p.numel()
            if not self.compress:
                c, k = False, 1
            elif plan is not None and name in plan:
                size, c, k = plan[name]
                if size != n:
                    raise ValueError(f"plan row {name}: size {size} != parameter size {n}")
            else:
                if plan is not None:
                    log.warning("gradient %s is not in the plan; using the size threshold", name)
                c, k = n >= cfg.comp_threshold, 1
            entries.append(Entry(name, p, n, bool(c), max(1, int(k)), i))
        return entries

    def _auto_plan(self, named, bucketed=False):
        """plan="auto": run the SeCoPa planner in process with a measured cost
        profile for this world size (the shipped one, or cfg.plan_profile).  Without
        a matching profile the size threshold decides.  plan="auto:bucketed" decides
        jointly for the bucket sizes of this engine instead of gradient by gradient."""
        from pathlib import Path
        from ..secopa.planner import CostProfile, Planner
        cfg = self.cfg
        path = Path(cfg.plan_profile) if cfg.plan_profile else \
            Path(__file__).resolve().parents[1] / "secopa" / "profiles" / \
            f"b200_{cfg.algorithm}_n{self.N}.json"
        if not path.exists():
            log.info("no cost profile %s: falling back to comp_threshold", path)
            return None
        prof = CostProfile.from_json(path.read_text())
        self._plan_profile_name = path.name
        if prof.nodes != self.N:
            log.warning("cost profile %s is for %d ranks, not %d: falling back to comp_threshold",
                        path, prof.nodes, self.N)
            return None
        topo = "PS" if cfg.topology == "ps" else "RING"
        grads = [(n, p.numel()) for n, p in named]
        if bucketed:
            rows = Planner(prof).plan_bucketed(grads, topo, cfg.bucket_bytes, cfg.plain_bucket_bytes)
        else:
            rows = Planner(prof).plan(grads, topo)
        return {name: (size, c == "y", k) for name, size, c, k in rows}

    def _check_order(self):
        """All ranks must register the same parameters in the same order."""
        if self.world == 1:
            return
        mine = [(e.name, e.numel, e.compress, e.partitions) for e in self.entries]
        every = [None] * self.world
        dist.all_gather_object(every, mine, group=self.world_group)
        for q, other in enumerate(every):
            if other != mine:
                raise RuntimeError(f"rank {self.world_rank} and rank {q} disagree on the gradient "
                                   "list or plan")

    def _make_buckets(self):
        """Bucket planning is done by the native planner (csrc/cpu/planner.cpp):
        fused buckets of tile-aligned segments for compressed gradients, plain
        buckets for the rest, in completion (= launch) order."""
        import numpy as np
        from .._native import lib as _lib
        cfg, n = self.cfg, len(self.entries)
        fused_ok = self.backend != "allreduce"
        numel = np.array([e.numel for e in self.entries], dtype=np.uint64)
        comp = np.array([1 if (e.compress and fused_ok) else 0 for e in self.entries], dtype=np.int32)
        parts = np.array([e.partitions for e in self.entries], dtype=np.int32)
        cap = int(sum(max(1, int(p)) for p in parts)) + n + MAX_SEGS
        bucket_of = np.zeros(n, dtype=np.int32)
        bucket_fused = np.zeros(n, dtype=np.int32)
        sb, se, sp = (np.zeros(cap, dtype=np.int32) for _ in range(3))
        slo, shi = np.zeros(cap, dtype=np.uint64), np.zeros(cap, dtype=np.uint64)
        nseg = np.zeros(1, dtype=np.int32)
        nb = _lib.cpu().hp_plan_buckets(
            n, numel.ctypes.data, comp.ctypes.data, parts.ctypes.data, cfg.bucket_bytes,
            cfg.plain_bucket_bytes, bucket_of.ctypes.data, bucket_fused.ctypes.data, cap,
            sb.ctypes.data, se.ctypes.data, sp.ctypes.data, slo.ctypes.data, shi.ctypes.data,
            nseg.ctypes.data)
        if nb < 0:
            _lib.check(nb, "bucket planner")
        buckets = [Bucket(i, bool(bucket_fused[i])) for i in range(nb)]
        for i in reversed(range(n)):  # entries of a bucket in the order backward produces them
            buckets[int(bucket_of[i])].entries.append(self.entries[i])
        for j in range(int(nseg[0])):
            buckets[int(sb[j])].segs.append(
                Segment(self.entries[int(se[j])], int(slo[j]), int(shi[j]), int(sp[j])))
        return buckets

    def _alloc_state(self):
        if not self.compress:
            return
        sp = self.comp.spec
        for b in self.buckets:
            if not b.fused:
                continue
            for e in b.entries:
                e.state = {k: torch.zeros(e.numel, dtype=torch.float32, device=self.device)
                           for k in sp.state_names()}
            for s in b.segs:
                sst = {}
                if self.cfg.topology == "ps" and self.cfg.server_residual and \
                        (sp.sparse or "residual" in sp.state_names()):
                    sst = {"residual": torch.zeros(chunk_elems(s.n, self.N), dtype=torch.float32,
                                                   device=self.device)}
                s.entry.server_state.append(sst)

    # --------------------------------------------------------------- backends
    def _setup_backend(self):
        cfg = self.cfg
        fused_buckets = [b for b in self.buckets if b.fused]
        self._host = None
        use_fused_kernels = self.backend == "fused" and self.compress and not self.comp.spec.sparse
        if self.backend == "fused" and self.compress and self.comp.spec.sparse:
            use_fused_kernels = self._setup_fused_sparse(fused_buckets)
        if use_fused_kernels and not self.comp.spec.sparse:
            from .fused import FusedDenseBucket
            from .symm import SymmetricArena
            self._make_partition_stream()
            impls = []
            for i, b in enumerate(fused_buckets):
                # buckets that complete while backward still runs go to the SM
                # partition; the last one has nothing left to overlap with
                on_part = cfg.partition_sms > 0 and i < len(fused_buckets) - 1
                b.stream = self.part_stream if on_part else self.comm_stream
                impls.append(FusedDenseBucket(
                    self.comp.spec, cfg.topology, [s.n for s in b.segs], self.N, self.R,
                    ctas=cfg.partition_ctas if on_part else cfg.ctas, timeout_s=cfg.timeout_s))
            total = sum(i.region_bytes() + 512 for i in impls) + 4096
            self.arena = SymmetricArena(total, self.group)
            self.status = torch.zeros(4, dtype=torch.int32, device=self.device)
            for b, impl in zip(fused_buckets, impls):
                impl.bind(self.arena.carve(impl.region_bytes()), self.status)
                b.impl = impl
            self._status_host = torch.zeros(4, dtype=torch.int32).pin_memory()
            self._status_event = None
        elif fused_buckets and not use_fused_kernels:
            self._host = HostSchedule(self.comp, cfg.topology, self.group)
        for b in self.buckets:
            if not b.fused and self.world > 1:
                b.flat = torch.zeros(sum(e.numel for e in b.entries), dtype=torch.float32,
                                     device=self.device)
        if self.outer is not None:
            self._setup_outer(fused_buckets)

    def _make_partition_stream(self):
        """Stream bound to a green context of cfg.partition_sms SMs; falls back to
        the ordinary communication stream when the driver refuses."""
        self.part_stream, self._green = self.comm_stream, None
        if self.cfg.partition_sms <= 0:
            return
        import ctypes as C
        from .._native import lib as _lib
        st, sms, g = C.c_void_p(), C.c_int(), C.c_void_p()
        rc = _lib.cuda().hp_cuda_partition_stream_create(
            self.device.index if self.device.index is not None else torch.cuda.current_device(),
            self.cfg.partition_sms, -1, C.byref(st), C.byref(sms), C.byref(g))
        if rc != 0 or not st.value:
            log.warning("SM partition unavailable; fused kernels share the whole GPU")
            return
        self._green = (st.value, g.value)
        self.partition_sms = sms.value
        self.part_stream = torch.cuda.ExternalStream(st.value, device=self.device)

    def _setup_fused_sparse(self, fused_buckets) -> bool:
        try:
            from .fused_sparse import FusedSparseBucket  # noqa: F401
        except ImportError:
            return False
        from .fused_sparse import setup_engine_buckets
        return setup_engine_buckets(self, fused_buckets)

    # ------------------------------------------------------------------ hooks
    def _begin(self):
        for b in self.buckets:
            b.pending = len(b.entries) * self.passes
            b.launched = False
        self._next = 0

    def _on_grad(self, param):
        b = self._by_param[param]
        b.pending -= 1
        if b.pending == 0:
            self._launch_ready()

    def _launch_ready(self):
        """Launch buckets strictly in index order (every rank issues the same
        sequence), as far as their gradients are complete."""
        while self._next < len(self.buckets) and self.buckets[self._next].pending <= 0:
            self._launch(self.buckets[self._next])
            self._next += 1

    def _grad(self, e: Entry) -> torch.Tensor:
        p = e.param
        if p.grad is None:
            p.grad = torch.zeros_like(p, memory_format=torch.preserve_format)
        g = p.grad
        if g.is_sparse:
            raise TypeError(f"gradient of {e.name} is a sparse tensor; use dense gradients "
                            "(e.g. nn.Embedding(sparse=False))")
        if g.dtype != torch.float32:
            raise TypeError(f"gradient of {e.name} is {g.dtype}; fp32 gradients are required")
        if not (g.is_contiguous() or g.is_contiguous(memory_format=torch.channels_last)):
            p.grad = g = g.contiguous()
        return g

    def _launch(self, b: Bucket):
        b.launched = True
        if self.on_cuda and b.fused and b.impl is not None:
            # fused kernels take the raw stream: no stream context switch on the
            # autograd thread, which is busy launching backward
            st = b.stream or self.comm_stream
            ev = self._events[b.index]
            ev.record()
            st.wait_event(ev)
            tok = self.timeline.begin(f"bucket{b.index}", st) if self.timeline.enabled else None
            self._launch_fused(b)
            if self.outer is not None:
                with torch.cuda.stream(st):
                    self._between_machines(b)
            if tok is not None:
                self.timeline.end(tok, st, step=self.step_no, fused=True,
                                  elems=sum(e.numel for e in b.entries))
            if self.on_bucket_done is not None:
                with torch.cuda.stream(st):
                    self.on_bucket_done(b)
            return
        if self.on_cuda:
            st = b.stream or self.comm_stream
            ev = torch.cuda.Event()
            ev.record(torch.cuda.current_stream())
            st.wait_event(ev)
            ctx = torch.cuda.stream(st)
        else:
            import contextlib
            ctx = contextlib.nullcontext()
        with ctx, nvtx_range(f"hipress.bucket{b.index}.{'fused' if b.fused else 'plain'}"):
            tok = self.timeline.begin(f"bucket{b.index}", torch.cuda.current_stream()) \
                if self.timeline.enabled else None
            if b.fused:
                self._launch_fused(b)
                if self.outer is not None:
                    self._between_machines(b)
            else:
                self._launch_plain(b)
            if tok is not None:
                self.timeline.end(tok, torch.cuda.current_stream(), step=self.step_no,
                                  fused=b.fused, elems=sum(e.numel for e in b.entries))
            if b.fused and self.on_bucket_done is not None:
                self.on_bucket_done(b)

    def _launch_fused(self, b: Bucket):
        grads = {id(e): self._grad(e) for e in b.entries}
        if b.impl is not None and self.comp.spec.sparse:
            g_ptrs, a_ptrs, u_ptrs, sr_ptrs = [], [], [], []
            for s in b.segs:
                e = s.entry
                g_ptrs.append(grads[id(e)].data_ptr() + 4 * s.lo)
                acc = e.state["accum_v"] if "accum_v" in e.state else e.state["residual"]
                a_ptrs.append(acc.data_ptr() + 4 * s.lo)
                u = e.state.get("momentum_u")
                u_ptrs.append(None if u is None else u.data_ptr() + 4 * s.lo)
                sst = e.server_state[s.part] if e.server_state else {}
                if sst.get("_scratch"):  # on the launch stream, ordered before the kernels
                    with torch.cuda.stream(b.stream or self.comm_stream):
                        sst["residual"].zero_()
                sr_ptrs.append(sst["residual"].data_ptr() if "residual" in sst else None)
            b.impl.launch_ptrs(g_ptrs, a_ptrs, u_ptrs, g_ptrs, sr_ptrs,
                               stream=b.stream or self.comm_stream)
            self.launch_count += 1
        elif b.impl is not None:
            g_ptrs, r_ptrs, sr_ptrs, ids = [], [], [], []
            rname = "residual"
            for s in b.segs:
                e = s.entry
                base = grads[id(e)].data_ptr()
                g_ptrs.append(base + 4 * s.lo)
                r = e.state.get(rname)
                r_ptrs.append(None if r is None else r.data_ptr() + 4 * s.lo)
                sst = e.server_state[s.part] if e.server_state else {}
                sr = sst.get("residual")
                sr_ptrs.append(None if sr is None else sr.data_ptr())
                ids.append(s.seg_id)
            b.impl.launch_ptrs(g_ptrs, r_ptrs, g_ptrs, sr_ptrs, step=self.step_no, tensor_ids=ids,
                               stream=b.stream or self.comm_stream)
            self.launch_count += 1
        else:
            views = []
            for s in b.segs:
                e = s.entry
                fg = _flat(grads[id(e)])
                views.append(SegView(fg[s.lo:s.hi], {k: v[s.lo:s.hi] for k, v in e.state.items()},
                                     e.server_state[s.part] if e.server_state else {}, s.seg_id))
            self._host.sync(views, step=self.step_no)

    # ------------------------------------------------- between machines
    def _setup_outer(self, fused_buckets):
        """State of the exchange between machines: this rank's 1/L shard of every
        segment has its own error-feedback state (and owner-side state for PS)."""
        from .simulate import chunk_range
        o = self.outer
        spec = self.comp.spec
        if spec.sparse:
            # the momentum correction already ran inside the machine; between
            # machines the shard only needs a plain error-feedback accumulator
            o["comp"] = Compressor(get_algorithm("graddrop", ratio=spec.ratio))
        else:
            o["comp"] = self.comp
        o["sched"] = HostSchedule(o["comp"], self.cfg.topology, o["group"])
        M = o["nodes"]
        for b in fused_buckets:
            b.outer = []
            for s in b.segs:
                lo, hi = chunk_range(s.n, self.N, self.R)
                m = max(hi - lo, 0)
                st = o["comp"].new_state(m, self.device) if m else {}
                sst = {}
                if m and self.cfg.topology == "ps" and self.cfg.server_residual and \
                        (o["comp"].spec.sparse or "residual" in o["comp"].spec.state_names()):
                    sst = {"residual": torch.zeros(chunk_elems(m, M), dtype=torch.float32,
                                                   device=self.device)}
                b.outer.append((lo, hi, st, sst))
            per = sum(chunk_elems(s.n, self.N) for s in b.segs)
            b.ag_in = torch.zeros(per, dtype=torch.float32, device=self.device)
            b.ag_out = [torch.zeros(per, dtype=torch.float32, device=self.device) for _ in range(self.N)]

    def _between_machines(self, b: Bucket):
        """Second and third stage of a bucket in hierarchical mode: compressed
        exchange of this rank's shards with the other machines, then an all-gather
        of the shards inside the machine.  Runs on the current stream, behind the
        bucket's synchronisation inside the machine."""
        from .simulate import chunk_range
        o = self.outer
        flats = [_flat(self._grad(s.entry))[s.lo:s.hi] for s in b.segs]
        views = [SegView(f[lo:hi], st, sst, s.seg_id)
                 for f, s, (lo, hi, st, sst) in zip(flats, b.segs, b.outer) if hi > lo]
        if views:
            o["sched"].sync(views, step=self.step_no, salt=1 << 16)
        off = 0
        for f, s, (lo, hi, _, _) in zip(flats, b.segs, b.outer):
            if hi > lo:
                b.ag_in[off:off + hi - lo].copy_(f[lo:hi])
            off += chunk_elems(s.n, self.N)
        dist.all_gather(b.ag_out, b.ag_in, group=self.group)
        for q in range(self.N):
            if q == self.R:
                continue
            off = 0
            for f, s in zip(flats, b.segs):
                lo, hi = chunk_range(s.n, self.N, q)
                if hi > lo:
                    f[lo:hi].copy_(b.ag_out[q][off:off + hi - lo])
                off += chunk_elems(s.n, self.N)

    def _launch_plain(self, b: Bucket):
        if self.world == 1:
            return
        grads = [self._grad(e) for e in b.entries]
        torch.cat([g.reshape(-1) for g in grads], out=b.flat)
        b.work = dist.all_reduce(b.flat, group=self.world_group, async_op=True)

    def _finish_plain(self, b: Bucket):
        if self.world == 1 or b.work is None:
            return
        b.work.wait()
        b.work = None
        b.flat.div_(self.world)
        off = 0
        for e in b.entries:
            e.param.grad.copy_(b.flat[off:off + e.numel].view_as(e.param.grad))
            off += e.numel

    # ------------------------------------------------------------- step ends
    def synchronize(self):
        """Launch whatever has not been launched, then make the current stream
        wait for every bucket.  Gradients are averaged in place afterwards."""
        for b in self.buckets[self._next:]:
            self._launch(b)
        self._next = len(self.buckets)
        if self.on_cuda:
            part = getattr(self, "part_stream", None)
            if part is not None and part is not self.comm_stream:
                self.comm_stream.wait_stream(part)
            with torch.cuda.stream(self.comm_stream):
                for b in self.buckets:
                    if not b.fused:
                        self._finish_plain(b)
                        if self.on_bucket_done is not None:
                            self.on_bucket_done(b)
                if self.arena is not None:
                    self._poll_status()
            torch.cuda.current_stream().wait_stream(self.comm_stream)
            if self.arena is not None and self.cfg.strict_status:
                # the host waits for this step's kernels and raises before the
                # optimizer can apply a gradient that a late peer left incomplete
                self._status_event.synchronize()
                self._raise_on_status([w & 0xFFFFFFFF for w in self._status_host.tolist()])
        else:
            for b in self.buckets:
                if not b.fused:
                    self._finish_plain(b)
                    if self.on_bucket_done is not None:
                        self.on_bucket_done(b)
        self.step_no += 1
        self._begin()

    def _raise_on_status(self, words):
        from .fused import HipressTimeoutError, decode_status
        if any(words):
            self.status.zero_()
            self._status_host.zero_()
            raise HipressTimeoutError(f"rank {self.R}: " + decode_status(next(w for w in words if w)))

    def _poll_status(self):
        """Asynchronous read of the kernels' status words: a wait that expired in one
        step is raised at the next synchronize, by check(), or -- with
        ``strict_status`` -- by the same synchronize before the optimizer runs.  A CTA
        whose wait expired writes neither error-feedback state nor gradient
        (csrc/cuda/fused_dense.cu), so the late report costs one step whose affected
        tensors carry the local instead of the averaged gradient, never corrupt
        state; checkpoints call check() first."""
        if self._status_event is not None and self._status_event.query():
            self._raise_on_status([w & 0xFFFFFFFF for w in self._status_host.tolist()])
        self._status_host.copy_(self.status, non_blocking=True)
        self._status_event = torch.cuda.Event()
        self._status_event.record(self.comm_stream)

    def check(self):
        """Blocking check of the device status words and of the guard words
        behind every bucket's region of the symmetric arena."""
        if self.arena is None:
            return
        self.arena.check_guards()
        torch.cuda.synchronize()
        self._raise_on_status([w & 0xFFFFFFFF for w in self.status.cpu().tolist()])

    # ------------------------------------------------------------ checkpoint
    def state_dict(self) -> dict:
        """Per-rank compressor state keyed by parameter name."""
        out = {}
        for e in self.entries:
            if not e.state and not any(e.server_state):
                continue
            d = {k: v.detach().cpu().clone() for k, v in e.state.items()}
            for i, sst in enumerate(e.server_state):
                for k, v in sst.items():
                    if torch.is_tensor(v) and not sst.get("_scratch"):
                        d[f"server_{k}.{i}"] = v.detach().cpu().clone()
            d["step"] = self.step_no
            out[e.name] = d
        sd = {"world_size": self.N, "rank": self.R, "algorithm": self.cfg.algorithm,
              "topology": self.cfg.topology, "step": self.step_no, "tensors": out}
        if self.outer is not None:
            sd["machines"] = self.outer["nodes"]
            sd["between_machines"] = {
                f"{s.entry.name}.{s.part}": {
                    **{k: v.detach().cpu().clone() for k, v in st.items()},
                    **{f"server_{k}": v.detach().cpu().clone() for k, v in sst.items()}}
                for b in self.buckets if b.fused for s, (_, _, st, sst) in zip(b.segs, b.outer)}
        return sd

    def load_state_dict(self, sd: dict):
        self.step_no = int(sd.get("step", 0))
        if sd.get("world_size") != self.N or sd.get("algorithm") != self.cfg.algorithm:
            log.warning("compressor state was saved for world size %s / %s; residuals dropped",
                        sd.get("world_size"), sd.get("algorithm"))
            return
        for e in self.entries:
            d = sd["tensors"].get(e.name)
            if d is None:
                continue
            for k, v in e.state.items():
                if k in d and d[k].numel() == v.numel():
                    v.copy_(d[k])
            for i, sst in enumerate(e.server_state):
                for k, v in sst.items():
                    if not torch.is_tensor(v):
                        continue
                    key = f"server_{k}.{i}"
                    if key in d and d[key].numel() == v.numel():
                        v.copy_(d[key])
        saved = sd.get("between_machines")
        if self.outer is not None and saved and sd.get("machines") == self.outer["nodes"]:
            for b in self.buckets:
                if not b.fused:
                    continue
                for s, (_, _, st, sst) in zip(b.segs, b.outer):
                    d = saved.get(f"{s.entry.name}.{s.part}", {})
                    for k, v in st.items():
                        if k in d and d[k].numel() == v.numel():
                            v.copy_(d[k])
                    for k, v in sst.items():
                        if f"server_{k}" in d and d[f"server_{k}"].numel() == v.numel():
                            v.copy_(d[f"server_{k}"])

    def stats(self) -> dict:
        comp_elems = sum(e.numel for e in self.entries if e.compress and self.backend != "allreduce")
        tot = sum(e.numel for e in self.entries)
        return {"buckets": len(self.buckets), "fused_buckets": sum(b.fused for b in self.buckets),
                "compressed_elems": comp_elems, "total_elems": tot, "backend": self.backend,
                "kernel_launches": self.launch_count, "plan": self.plan_source,
                "compressed_gradients": sum(1 for e in self.entries if e.compress and
                                            self.backend != "allreduce")}

    def close(self, collective: bool = True):
        """``collective=False``: the process group this engine was built on is gone
        (elastic recovery); release the symmetric memory without any barrier."""
        self.timeline.dump(self.R)
        for h in self._hooks:
            h.remove()
        self._hooks = []
        if self.arena is not None:
            self.arena.close(collective=collective)
            self.arena = None
        if getattr(self, "_green", None):
            from .._native import lib as _lib
            torch.cuda.synchronize()
            self.part_stream = self.comm_stream
            _lib.cuda().hp_cuda_partition_stream_destroy(*self._green)
            self._green = None
