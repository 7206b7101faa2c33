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


def time_cuda(fn, *, warmup=3, iters=10, flush: L2Flusher | None = None, setup=None,
              hide_launch: bool = True, align=None):
    """Median / min milliseconds of fn() over `iters` runs timed with CUDA events.

    ``hide_launch`` (default): the first event and fn()'s launches are queued while
    earlier work (the L2 flush, or a short spin kernel) still occupies the stream, so
    the interval between the events is device time only -- what a training step
    sees, where a bucket's launch is queued behind backward kernels.  With
    ``hide_launch=False`` the stream is idle when fn() is called and the host's
    launch path (tens of microseconds from Python) is part of the figure.
    ``align`` (multi-GPU runs): a callable that queues a tiny collective right before
    the first event, so every rank's timed region starts at the same moment on the
    device instead of whenever its host got there."""
    for _ in range(warmup):
        if setup:
            setup()
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(iters):
        if setup:
            setup()
        torch.cuda.synchronize()
        if flush:
            flush()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        if not hide_launch:
            torch.cuda.synchronize()
        else:
            torch.cuda._sleep(400_000)      # ~0.2 ms of spinning: time to queue what follows
        if align is not None:
            align()
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        ts.append(a.elapsed_time(b))
    ts.sort()
    return {"median_ms": ts[len(ts) // 2], "min_ms": ts[0], "max_ms": ts[-1]}
