"""Run-time configuration: one dataclass fed by command-line flags with the same
spellings the reference launchers use (``--topo``, ``--comp-alg``,
``--comp-threshold``, ``--comprplan`` for the MXNet script, README.md:160-169;
``--algorithm`` for the PyTorch script, README.md:186) and by ``HIPRESS_*``
environment variables."""
from __future__ import annotations

import argparse
import os
import typing
from dataclasses import dataclass, field, fields


@dataclass
class HipressConfig:
    algorithm: str = "tbq"            # onebit | tbq | terngrad | dgc | graddrop | none
    topology: str = "ring"            # ring | ps
    comp_threshold: int = 262144      # gradients with fewer elements are not compressed
    plan: str | None = None           # SeCoPa plan file (overrides comp_threshold), "auto" or "auto:bucketed"
    plan_profile: str | None = None   # cost profile for plan="auto" (default: shipped B200 profile)
    threshold: float = 0.01           # tbq
    bitwidth: int | None = None       # terngrad
    ratio: float = 0.001              # dgc / graddrop
    momentum: float = 0.9             # dgc momentum correction
    seed: int = 0
    backend: str = "auto"             # auto | fused | host | allreduce
    bucket_bytes: int = 256 << 20     # gradient bytes per fused launch
    plain_bucket_bytes: int = 32 << 20
    ctas: int = 444                   # CTAs of a fused kernel (3 per SM on a 148-SM B200)
    partition_sms: int = 0            # SMs reserved (green context) for fused kernels that overlap backward; 0 = off
    partition_ctas: int = 48          # CTAs of a fused kernel on the SM partition
    timeout_s: float = 10.0           # bound of every device-side wait
    strict_status: bool = False       # synchronize() waits for the step's kernels and raises on an expired wait before the optimizer runs
    server_residual: bool = True      # PS: error feedback on the re-encode at the owner
    hierarchical: str = "auto"        # job on several machines: auto | on | off (see GradSyncEngine)
    overlap: bool = True              # launch buckets from gradient hooks during backward
    overlap_optimizer: bool = False   # update a bucket's parameters right behind its synchronisation
    log_level: str = field(default_factory=lambda: os.environ.get("HIPRESS_LOG_LEVEL", "INFO"))

    def algorithm_kwargs(self) -> dict:
        return dict(threshold=self.threshold, bitwidth=self.bitwidth, ratio=self.ratio,
                    momentum=self.momentum, seed=self.seed)

    @staticmethod
    def from_env(**overrides) -> "HipressConfig":
        cfg = HipressConfig()
        hints = typing.get_type_hints(HipressConfig)
        for f in fields(HipressConfig):
            v = os.environ.get("HIPRESS_" + f.name.upper())
            if v is None:
                continue
            # convert by the declared type (``int | None`` fields default to None, so
            # the current value says nothing about them)
            kinds = [t for t in typing.get_args(hints[f.name]) if t is not type(None)] or [hints[f.name]]
            kind = kinds[0]
            if kind is not str and v.strip().lower() in ("", "none") and type(None) in typing.get_args(hints[f.name]):
                setattr(cfg, f.name, None)
            elif kind is bool:
                setattr(cfg, f.name, v.lower() in ("1", "true", "yes", "on"))
            elif kind is int:
                setattr(cfg, f.name, int(v))
            elif kind is float:
                setattr(cfg, f.name, float(v))
            else:
                setattr(cfg, f.name, v)
        for k, v in overrides.items():
            if v is not None:
                setattr(cfg, k, v)
        return cfg


def add_hipress_args(ap: argparse.ArgumentParser) -> argparse.ArgumentParser:
    g = ap.add_argument_group("hipress")
    g.add_argument("--topo", "--topology", dest="topo", default="Ring",
                   help="CaSync topology: PS or Ring")
    g.add_argument("--comp-alg", "--comp_alg", "--algorithm", dest="comp_alg", default="tbq",
                   help="onebit | tbq | terngrad | dgc | graddrop | none")
    g.add_argument("--comp-threshold", dest="comp_threshold", type=int, default=262144,
                   help="compress gradients with at least this many elements")
    g.add_argument("--comprplan", default=None, help="SeCoPa plan file (name,size,y|n,K rows)")
    g.add_argument("--threshold", type=float, default=0.01, help="tbq threshold")
    g.add_argument("--bitwidth", type=int, default=None, help="terngrad bits per element")
    g.add_argument("--ratio", type=float, default=0.001, help="dgc / graddrop send ratio")
    g.add_argument("--sync-backend", default="auto", choices=["auto", "fused", "host", "allreduce"])
    g.add_argument("--overlap-optimizer", action="store_true",
                   help="update each bucket's parameters right behind its synchronisation")
    return ap


def config_from_args(a) -> HipressConfig:
    return HipressConfig.from_env(
        algorithm=a.comp_alg.lower(), topology=a.topo.lower(), comp_threshold=a.comp_threshold,
        plan=a.comprplan, threshold=a.threshold, bitwidth=a.bitwidth, ratio=a.ratio,
        backend=a.sync_backend, overlap_optimizer=getattr(a, "overlap_optimizer", False) or None)
