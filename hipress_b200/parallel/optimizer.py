"""Horovod-style ``DistributedOptimizer``: wraps any ``torch.optim`` optimizer so
that ``step()`` first waits for the compressed synchronisation of all gradients.

Reference parity: the reference front ends wrap the optimizer with Horovod's
``DistributedOptimizer`` / ``DistributedTrainer`` plus an algorithm selector
(``--algorithm tbq`` README.md:186, ``--comp-alg`` README.md:160 of
mark14wu/hipress)."""
from __future__ import annotations

import torch

from ..config import HipressConfig
from .engine import GradSyncEngine


class DistributedOptimizer:
    def __init__(self, optimizer: torch.optim.Optimizer, named_parameters=None,
                 config: HipressConfig | None = None, *, backward_passes_per_step: int = 1,
                 group=None, **overrides):
        """``overrides`` are :class:`HipressConfig` fields, e.g. ``algorithm="tbq"``,
        ``topology="ring"``, ``comp_threshold=262144``, ``plan="SeCoPaPlan.txt"``."""
        self.optimizer = optimizer
        cfg = config or HipressConfig.from_env()
        for k, v in overrides.items():
            if not hasattr(cfg, k):
                raise TypeError(f"unknown option {k}")
            setattr(cfg, k, v)
        if named_parameters is None:
            named_parameters = [(f"param.{gi}.{pi}", p)
                                for gi, g in enumerate(optimizer.param_groups)
                                for pi, p in enumerate(g["params"])]
        self.config = cfg
        self.engine = GradSyncEngine(list(named_parameters), cfg, group=group,
                                     backward_passes_per_step=backward_passes_per_step)
        self._synchronized = False
        self._bucket_opts = None
        if cfg.overlap_optimizer:
            self._make_bucket_optimizers()

    # ------------------------------------------------ overlapped parameter update
    def _make_bucket_optimizers(self):
        """One optimizer per synchronisation bucket, of the wrapped optimizer's class,
        stepped on the communication stream right behind the bucket's kernel, so the
        update of the layers that finish backward first hides behind the rest of
        backward.  The per-bucket optimizers share the wrapped optimizer's ``state``
        mapping (its ``state_dict`` stays complete) and re-read its hyper-parameters
        at every step (learning-rate schedulers keep working).  Anything that needs
        all gradients before the update (clipping, a closure) needs the option off."""
        src_group = {}
        for g in self.optimizer.param_groups:
            for p in g["params"]:
                src_group[p] = g
        cls = type(self.optimizer)
        self._bucket_opts = {}
        for b in self.engine.buckets:
            groups = {}
            for e in b.entries:
                g = src_group.get(e.param)
                if g is None:
                    raise ValueError(f"{e.name} is synchronised but not owned by the optimizer")
                groups.setdefault(id(g), (g, []))[1].append(e.param)
            pgs = [{**{k: v for k, v in g.items() if k != "params"}, "params": ps}
                   for g, ps in groups.values()]
            bo = cls(pgs)
            bo.state = self.optimizer.state
            self._bucket_opts[b.index] = (bo, [g for g, _ in groups.values()])
        self.engine.on_bucket_done = self._step_bucket

    def _step_bucket(self, bucket):
        bo, sources = self._bucket_opts[bucket.index]
        for pg, src in zip(bo.param_groups, sources):
            for k, v in src.items():
                if k != "params":
                    pg[k] = v
        bo.step()

    # Horovod API
    def synchronize(self):
        self.engine.synchronize()
        self._synchronized = True

    def skip_synchronize(self):
        """Horovod's context manager for ``synchronize(); clip; with
        skip_synchronize(): step()``.  ``step()`` already skips a second
        synchronisation after an explicit ``synchronize()``, so this only marks the
        gradients as synchronised for the duration of the block."""
        import contextlib

        @contextlib.contextmanager
        def ctx():
            before, self._synchronized = self._synchronized, True
            try:
                yield
            finally:
                self._synchronized = before if self._synchronized else False
        return ctx()

    def step(self, closure=None):
        if not self._synchronized:
            self.engine.synchronize()
        self._synchronized = False
        if self._bucket_opts is not None:
            if closure is not None:
                raise ValueError("overlap_optimizer does not support a closure")
            return None  # every bucket was stepped behind its synchronisation
        return self.optimizer.step(closure)

    def zero_grad(self, set_to_none: bool = True):
        self.optimizer.zero_grad(set_to_none=set_to_none)

    @property
    def param_groups(self):
        return self.optimizer.param_groups

    def state_dict(self):
        return {"optimizer": self.optimizer.state_dict(), "compressor_state": self.engine.state_dict()}

    def load_state_dict(self, sd):
        if "optimizer" in sd:
            self.optimizer.load_state_dict(sd["optimizer"])
            if sd.get("compressor_state"):
                self.engine.load_state_dict(sd["compressor_state"])
        else:
            self.optimizer.load_state_dict(sd)
        self._relink()

    def _relink(self):
        """Loading a state dict replaces the wrapped optimizer's state mapping: the
        per-bucket optimizers of the overlapped step must share the new one."""
        if self._bucket_opts is not None:
            for bo, _ in self._bucket_opts.values():
                bo.state = self.optimizer.state

    def close(self, collective: bool = True):
        self.engine.close(collective=collective)

    def __getattr__(self, name):
        return getattr(self.__dict__["optimizer"], name)
