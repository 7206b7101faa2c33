"""Logging and per-step metrics.

``setup_logging`` configures the ``hipress`` logger (level from HIPRESS_LOG_LEVEL,
INFO by default; only rank 0 prints below WARNING).  ``MetricsWriter`` appends one
JSON object per training step: step, throughput, milliseconds, bytes that crossed
NVLink, compression ratio, residual norm, plan decisions.
"""
from __future__ import annotations

import json
import logging
import os
import time

import torch

from ..parallel import comm


def setup_logging(level: str | None = None) -> logging.Logger:
    lg = logging.getLogger("hipress")
    if not lg.handlers:
        h = logging.StreamHandler()
        h.setFormatter(logging.Formatter(f"[hipress r{comm.rank()}] %(levelname)s %(message)s"))
        lg.addHandler(h)
    name = (level or os.environ.get("HIPRESS_LOG_LEVEL", "INFO")).upper()
    lvl = getattr(logging, name, logging.INFO)
    if comm.rank() != 0:
        lvl = max(lvl, logging.WARNING)
    lg.setLevel(lvl)
    return lg


class MetricsWriter:
    def __init__(self, path: str | None, every: int = 1):
        self.path, self.every = path, every
        self.f = open(path, "a") if path and comm.rank() == 0 else None
        self.t0 = time.time()

    def step(self, step: int, **fields):
        if self.f is None or step % self.every:
            return
        rec = {"step": step, "t": round(time.time() - self.t0, 3)}
        rec.update(fields)
        self.f.write(json.dumps(rec) + "\n")
        self.f.flush()

    def close(self):
        if self.f:
            self.f.close()
            self.f = None


def engine_metrics(engine) -> dict:
    """Compression statistics of a GradSyncEngine for the metrics stream."""
    comp = raw = 0
    for b in engine.buckets:
        for e in b.entries:
            raw += 4 * e.numel
            if b.fused and engine.comp is not None:
                comp += engine.comp.payload_bytes(e.numel)
            else:
                comp += 4 * e.numel
    held = [v for e in engine.entries for k, v in e.state.items() if k in ("residual", "accum_v")]
    # one reduction and one read of the device, whatever the number of tensors
    norm = float(torch.linalg.vector_norm(torch.stack(torch._foreach_norm(held)))) if held else 0.0
    return {"gradient_bytes": raw, "payload_bytes": comp,
            "compression_ratio": round(raw / max(comp, 1), 2), "residual_norm": norm,
            "buckets": len(engine.buckets), "backend": engine.backend}
