"""Does the partition count K of a SeCoPa plan row change the time of one compressed
synchronisation on this fabric?

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \\
        -m hipress_b200.bench.partitions --elems 102760448 --out partitions_n8.json

The reference planner picks K per gradient to pipeline the partitions' encode, send
and decode steps against one another (the K loops of src/SeCoPa/SeCoPa.py:52,65,80,95
of mark14wu/hipress).  Here a plan row with K partitions becomes K tile-aligned
segments of ONE persistent launch, whose 4096-element tiles already flow through
encode, peer store and decode independently of one another; this bench times the
same tensor (default: VGG-19's first fully connected layer, 102,760,448 elements)
with K = 1, 2, 4, 8 through the DistributedOptimizer, device-timed, max over ranks.
"""
from __future__ import annotations

import argparse
import json
import tempfile

import torch
import torch.distributed as dist

from .. import DistributedOptimizer, HipressConfig
from ..parallel import comm
from .timing import L2Flusher, time_cuda


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--elems", type=int, default=102760448)
    ap.add_argument("--algorithm", default="tbq")
    ap.add_argument("--topo", default="ring")
    ap.add_argument("--ks", default="1,2,4,8")
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--out", default=None)
    a = ap.parse_args(argv)
    comm.init()
    N, R = comm.size(), comm.rank()
    dev = comm.device()
    flush = L2Flusher(dev)
    tick = torch.zeros(1, device=dev)
    align = (lambda: dist.all_reduce(tick)) if N > 1 else None
    g = torch.randn(a.elems, device=dev, generator=torch.Generator(dev).manual_seed(R)) * 0.02
    rows = []
    for k in [int(x) for x in a.ks.split(",")]:
        p = torch.nn.Parameter(torch.zeros(a.elems, device=dev))
        with tempfile.NamedTemporaryFile("w", suffix=".txt", delete=False) as f:
            f.write(f"w,{a.elems},y,{k}\n")
            plan = f.name
        cfg = HipressConfig(algorithm=a.algorithm, topology=a.topo, plan=plan, bucket_bytes=1 << 31)
        opt = DistributedOptimizer(torch.optim.SGD([p], lr=0.0), [("w", p)], cfg)
        eng = opt.engine
        p.grad = torch.empty_like(g)

        def sync():
            opt.synchronize()
            opt._synchronized = False

        t = time_cuda(sync, iters=a.iters, flush=flush, setup=lambda: p.grad.copy_(g), align=align)
        ms = torch.tensor([t["median_ms"]], device=dev, dtype=torch.float64)
        if N > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        eng.check()
        row = {"K": k, "segments": sum(len(b.segs) for b in eng.buckets if b.fused),
               "launches_per_sync": sum(1 for b in eng.buckets if b.fused), "ms": round(ms.item(), 5),
               "elems": a.elems, "algorithm": a.algorithm, "topology": a.topo, "n_gpus": N}
        rows.append(row)
        if R == 0:
            print(json.dumps(row), flush=True)
        opt.close()
        del opt, p
    if R == 0 and a.out:
        with open(a.out, "w") as f:
            json.dump(rows, f, indent=1)
    comm.shutdown()


if __name__ == "__main__":
    main()
