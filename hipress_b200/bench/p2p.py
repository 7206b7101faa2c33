"""Peer-to-peer store bandwidth between the GPUs of one box, the way the fused
kernels move payloads: plain 128-bit stores from a kernel into a peer's memory
mapped through CUDA IPC (no copy engine, no NCCL).

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 \\
        -m hipress_b200.bench.p2p --min-kb 64 --max-mb 256 --out p2p.json

Every rank stores into its successor's arena at the same time (a ring of
unidirectional streams), so with N ranks every GPU sends and receives at once.
Times are CUDA events on the launching stream, max over ranks; the fitted line
``ms = slope * bytes + intercept`` is the ``ring_send`` term of a SeCoPa profile
(`--profile-out` writes it in the planner's units, per fp32 element).
"""
from __future__ import annotations

import argparse
import json

import torch
import torch.distributed as dist

from .._native import lib as _lib
from ..parallel import comm
from ..parallel.symm import SymmetricArena
from .timing import NVLINK_GBS_PER_DIR, time_cuda


def sweep(min_bytes: int, max_bytes: int, iters: int = 10, ctas: int = 0):
    N, R = comm.size(), comm.rank()
    if N < 2:
        raise SystemExit("the peer-to-peer microbench needs at least 2 ranks")
    L = _lib.cuda()
    arena = SymmetricArena(max_bytes + 4096)
    dst = arena.carve(max_bytes)[(R + 1) % N]
    src = torch.randn(max_bytes // 4, device="cuda")
    stream = _lib.stream_ptr()
    rows = []
    b = min_bytes
    while b <= max_bytes:
        nbytes = b // 16 * 16

        def store():
            _lib.check(L.hp_cuda_peer_store(src.data_ptr(), dst, nbytes, ctas, stream), "peer store")

        dist.barrier()
        t = time_cuda(store, iters=iters)
        ms = torch.tensor([t["median_ms"]], device="cuda")
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        rows.append({"bytes": nbytes, "ms": round(ms.item(), 5),
                     "gbs": round(nbytes / ms.item() / 1e6, 1), "n_gpus": N})
        b *= 4
    torch.cuda.synchronize()
    dist.barrier()
    arena.check_guards()
    arena.close()
    return rows


def main(argv=None):
    ap = argparse.ArgumentParser(description="in-kernel peer store bandwidth between GPUs")
    ap.add_argument("--min-kb", type=int, default=64)
    ap.add_argument("--max-mb", type=int, default=256)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--ctas", type=int, default=0, help="CTAs of the store kernel (0: 4 per SM)")
    ap.add_argument("--out", default=None)
    ap.add_argument("--profile-out", default=None, help="write the fitted send term (per element)")
    a = ap.parse_args(argv)
    comm.init()
    rows = sweep(a.min_kb << 10, a.max_mb << 20, a.iters, a.ctas)
    if comm.rank() == 0:
        for r in rows:
            print(json.dumps(r))
        peak = max(r["gbs"] for r in rows)
        print(json.dumps({"peak_gbs": peak, "of_measured_peer_copy": round(peak / NVLINK_GBS_PER_DIR, 3)}))
        if a.out:
            with open(a.out, "w") as f:
                json.dump(rows, f, indent=1)
        if a.profile_out:
            from ..secopa.profiler import fit_linear
            fit = fit_linear([r["bytes"] / 4.0 for r in rows], [r["ms"] for r in rows])
            with open(a.profile_out, "w") as f:
                json.dump({"ring_send": {"slope": fit.slope, "intercept": fit.intercept, "floor": fit.floor},
                           "n_gpus": rows[0]["n_gpus"]}, f, indent=1)
    comm.shutdown()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
