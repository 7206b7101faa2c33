"""Timeline tracing: NVTX ranges around bucket launches and a Chrome-trace file
(``HIPRESS_TIMELINE=<path>``, the counterpart of Horovod's HOROVOD_TIMELINE) with
one event per bucket launch, timed on the device with CUDA events."""
from __future__ import annotations

import json
import os
from contextlib import contextmanager

import torch


@contextmanager
def nvtx_range(name: str):
    on = torch.cuda.is_available()
    if on:
        torch.cuda.nvtx.range_push(name)
    try:
        yield
    finally:
        if on:
            torch.cuda.nvtx.range_pop()


class Timeline:
    """Collects (name, start event, end event) triples and writes a Chrome trace."""

    def __init__(self, path: str | None = None):
        self.path = path or os.environ.get("HIPRESS_TIMELINE")
        self.enabled = bool(self.path) and torch.cuda.is_available()
        self.events = []
        self.origin = None

    def begin(self, name: str, stream=None):
        if not self.enabled:
            return None
        s = torch.cuda.Event(enable_timing=True)
        s.record(stream)
        if self.origin is None:
            self.origin = s
        return (name, s)

    def end(self, token, stream=None, **args):
        if token is None:
            return
        e = torch.cuda.Event(enable_timing=True)
        e.record(stream)
        self.events.append((token[0], token[1], e, args))

    def dump(self, rank: int = 0):
        if not self.enabled or not self.events:
            return None
        torch.cuda.synchronize()
        out = []
        for name, s, e, args in self.events:
            out.append({"name": name, "ph": "X", "pid": rank, "tid": 0,
                        "ts": self.origin.elapsed_time(s) * 1e3, "dur": s.elapsed_time(e) * 1e3,
                        "args": args})
        path = self.path if rank == 0 else f"{self.path}.{rank}"
        with open(path, "w") as f:
            json.dump({"traceEvents": out}, f)
        self.events = []
        return path
