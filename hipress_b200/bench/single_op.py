"""Runs one stand-alone compression op a few times (the case to hand to a profiler).

    python -m hipress_b200.bench.single_op --alg dgc --op encode --mbytes 256 --iters 3
"""
import argparse
import json

import torch

from ..ops import Compressor
from .timing import L2Flusher, measured_peaks, time_cuda
from .sweep import algorithmic_bytes


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--alg", default="dgc")
    ap.add_argument("--op", default="encode", choices=["encode", "decode"])
    ap.add_argument("--mbytes", type=int, default=256)
    ap.add_argument("--iters", type=int, default=3)
    a = ap.parse_args(argv)
    c = Compressor(a.alg)
    n = a.mbytes * 1024 * 1024 // 4
    g = torch.randn(n, device="cuda", generator=torch.Generator("cuda").manual_seed(0))
    st = c.new_state(n, "cuda")
    pay = torch.empty(c.payload_bytes(n), dtype=torch.uint8, device="cuda")
    ws = c.new_workspace("cuda", n)
    out = torch.empty(n, device="cuda")
    c.encode(g, st, out=pay, workspace=ws)
    fn = (lambda: c.encode(g, st, out=pay, workspace=ws)) if a.op == "encode" else \
        (lambda: c.decode(pay, out))
    t = time_cuda(fn, warmup=1, iters=a.iters, flush=L2Flusher())
    b = algorithmic_bytes(c, n, a.op)
    gbs = b / (t["median_ms"] * 1e-3) / 1e9
    print(json.dumps({"alg": a.alg, "op": a.op, "mbytes": a.mbytes, "ms": round(t["median_ms"], 5),
                      "gbs": round(gbs, 1), "frac_hbm": round(gbs / measured_peaks()["hbm_gbs"], 4)}))


if __name__ == "__main__":
    main()
