"""Device timing helpers: CUDA events on the launching stream, warm-up, an L2 flush
between timed iterations, and the measured roofline denominators."""
from __future__ import annotations

import json
import os
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parents[2]
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0,
                  "source": "fallback"}
NVLINK_GBS_PER_DIR = 770.0  # measured peer-copy bandwidth per direction on B200 NVLink 5 (nominal 900)


def measured_peaks() -> dict:
    p = Path(os.environ.get("HIPRESS_PEAKS", ROOT / "MEASURED_PEAKS.json"))
    if p.exists():
        d = json.loads(p.read_text())
        d["source"] = "measured"
        return d
    return dict(FALLBACK_PEAKS)


class L2Flusher:
    """Writes a buffer larger than the 126 MB L2 so the next timed run starts cold,
    then reads a second one so the cache is left holding clean lines (otherwise
    the timed kernel also pays for writing the flush buffer's dirty lines back)."""

    def __init__(self, device="cuda", mbytes=256):
        self.buf = torch.zeros(mbytes * 1024 * 1024 // 4, dtype=torch.float32, device=device)
        self.rd = torch.zeros(mbytes * 1024 * 1024 // 4, dtype=torch.float32, device=device)
        self.sink = torch.zeros((), dtype=torch.float32, device=device)

    def __call__(self):
        self.buf.add_(1.0)
        self.sink = self.rd.sum()


def time_cuda(fn, *, warmup=3, iters=10, flush: L2Flusher | None = None, setup=None):
    """Median / min milliseconds of fn() over `iters` runs timed with CUDA events."""
    for _ in range(warmup):
        if setup:
            setup()
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(iters):
        if setup:
            setup()
        if flush:
            flush()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        ts.append(a.elapsed_time(b))
    ts.sort()
    return {"median_ms": ts[len(ts) // 2], "min_ms": ts[0], "max_ms": ts[-1]}
