"""Multi-GPU compress-sync sweep (one process per GPU, launch with
``python -m torch.distributed.run --nproc-per-node N -m hipress_b200.bench.sweep_multi``).

For fp32 gradients of 4 KB - 1 GB (powers of 4, N(0,1), seed 0 + rank) and each of
onebit, TBQ, TernGrad, DGC 0.1 %, GradDrop 0.1 % through Ring and PS it times

* ``fused``     the fused kernels (every algorithm through ring and PS),
* ``unfused``   the same schedule from separate encode / decode kernels around NCCL
                point-to-point and all-gather calls (the reference's structure),
* ``allreduce`` the uncompressed NCCL all-reduce of the same gradient,

on the device (CUDA events, max over ranks, L2 flushed between runs) and reports
the fused path's fraction of its roofline: the slower of (HBM bytes the rank must
move / measured copy bandwidth) and (payload bytes the rank must send over NVLink /
770 GB/s measured peer-copy bandwidth)."""
from __future__ import annotations

import argparse
import json

import torch
import torch.distributed as dist

from ..ops import Compressor
from ..parallel import comm
from ..parallel.fused import FusedDenseBucket
from ..parallel.fused_sparse import FusedSparseBucket
from ..parallel.host_schedule import HostSchedule, SegView
from ..parallel.simulate import chunk_elems
from ..parallel.symm import SymmetricArena
from .timing import NVLINK_GBS_PER_DIR, L2Flusher, measured_peaks, time_cuda

ALGS = [("onebit", {}), ("tbq", {}), ("terngrad", {"bitwidth": 2}), ("dgc", {}), ("graddrop", {})]


def _max_over_ranks(ms: float) -> float:
    t = torch.tensor([ms], device="cuda", dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return t.item()


def roofline_ms(comp: Compressor, n: int, N: int, topo: str, peaks) -> dict:
    sp = comp.spec
    if sp.sparse:
        state = 20.0 if sp.name == "dgc" else 12.0
        hbm = (state + 4.0) * n + 8.0 * n / N        # update + zero-fill/scatter + owner accumulator
    else:
        ef = 8.0 if "residual" in sp.state_names() else 0.0
        hbm = (4.0 + ef + 4.0) * n                    # encode pass + decoded write
        if topo == "ps" and ef:
            hbm += 8.0 * n / N                        # server residual of the owned chunk
    pay = comp.payload_bytes(chunk_elems(n, N))
    if not sp.sparse:
        pay *= 2          # the fused dense kernels ship codes in {data, epoch} slots
    link = pay * (N - 1) * (1 if topo == "ring" else 2)   # bytes this rank stores into peers
    t_hbm = hbm / (peaks["hbm_gbs"] * 1e9) * 1e3
    t_link = link / (NVLINK_GBS_PER_DIR * 1e9) * 1e3
    return {"hbm_ms": t_hbm, "link_ms": t_link, "roof_ms": max(t_hbm, t_link)}


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--min-kb", type=int, default=4)
    ap.add_argument("--max-mb", type=int, default=1024)
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--ctas", type=int, default=444)
    ap.add_argument("--algs", default="onebit,tbq,terngrad,dgc,graddrop")
    ap.add_argument("--skip-unfused", action="store_true")
    ap.add_argument("--trace", action="store_true",
                    help="dense kernels: one more launch per row with the device-side phase trace "
                         "(when the last CTA left each hop, and how long CTAs polled for input)")
    ap.add_argument("--out", default=None)
    a = ap.parse_args(argv)
    comm.init()
    N, R = comm.size(), comm.rank()
    dev = comm.device()
    peaks = measured_peaks()
    flush = L2Flusher(dev)
    sizes, s = [], a.min_kb * 1024
    while s <= a.max_mb * 1024 * 1024:
        sizes.append(s)
        s *= 4
    rows = []
    status = torch.zeros(4, dtype=torch.int32, device=dev)
    tick = torch.zeros(1, device=dev)
    align = (lambda: dist.all_reduce(tick)) if N > 1 else None
    for nbytes in sizes:
        n = nbytes // 4
        gen = torch.Generator(dev).manual_seed(R)
        g = torch.randn(n, device=dev, generator=gen)
        work = torch.empty_like(g)
        if N > 1:
            t = time_cuda(lambda: dist.all_reduce(work), iters=a.iters, flush=flush,
                          setup=lambda: work.copy_(g), align=align)
            ar_ms = _max_over_ranks(t["median_ms"])
        else:
            ar_ms = 0.0
        for name, kw in ALGS:
            if name not in a.algs.split(","):
                continue
            comp = Compressor(name, **kw)
            for topo in ("ring", "ps"):
                row = {"alg": name, "topo": topo, "bytes": nbytes, "n_gpus": N,
                       "allreduce_ms": round(ar_ms, 5)}
                st = comp.new_state(n, dev)
                sr = torch.zeros(chunk_elems(n, N), device=dev)
                arena = None
                fused = None
                if not comp.spec.sparse:
                    fused = FusedDenseBucket(comp.spec, topo, [n], N, R, ctas=a.ctas)
                else:
                    fused = FusedSparseBucket(comp.spec, [n], N, R, topology=topo)
                if fused is not None:
                    arena = SymmetricArena(fused.region_bytes() + 8192)
                    if comp.spec.sparse:
                        fused.bind(arena.carve(fused.region_bytes()), status, dev)
                        acc = st["accum_v"] if "accum_v" in st else st["residual"]
                        u = st.get("momentum_u")
                        fn = lambda: fused.launch_ptrs(  # noqa: E731
                            [work.data_ptr()], [acc.data_ptr()], [u.data_ptr()] if u is not None else None,
                            [work.data_ptr()], [sr.data_ptr()])
                    else:
                        fused.bind(arena.carve(fused.region_bytes()), status)
                        r = st.get("residual")
                        fn = lambda: fused.launch_ptrs(  # noqa: E731
                            [work.data_ptr()], [None if r is None else r.data_ptr()], [work.data_ptr()],
                            [sr.data_ptr() if r is not None else None])
                    dist.barrier() if N > 1 else None
                    t = time_cuda(fn, iters=a.iters, flush=flush, setup=lambda: work.copy_(g), align=align)
                    row["fused_ms"] = round(_max_over_ranks(t["median_ms"]) if N > 1 else t["median_ms"], 5)
                    roof = roofline_ms(comp, n, N, topo, peaks)
                    row.update({k: round(v, 5) for k, v in roof.items()})
                    row["roofline_frac"] = round(roof["roof_ms"] / row["fused_ms"], 4)
                    if a.trace and not comp.spec.sparse:
                        fused.enable_trace()
                        work.copy_(g)
                        torch.cuda.synchronize()
                        dist.barrier() if N > 1 else None
                        fn()
                        torch.cuda.synchronize()
                        row["trace_rank0"] = [{"phase": p["phase"], "end_ms": round(p["end_ms"], 4),
                                               "mean_poll_ms": round(p["mean_poll_ms"], 4)}
                                              for p in fused.last_trace_phases()[0]]
                        fused.enable_trace(False)
                    if a.trace and comp.spec.sparse:
                        torch.cuda.synchronize()
                        row["phase_end_ms_rank0"] = [round(x, 4) for x in fused.last_phase_times()]
                    if int(status.abs().sum()) != 0:
                        row["status"] = [w & 0xFFFFFFFF for w in status.tolist()]
                        status.zero_()
                if not a.skip_unfused and (N > 1 or fused is None):
                    hs = HostSchedule(comp, topo)
                    st2 = comp.new_state(n, dev)
                    sst = {"residual": sr} if (comp.spec.sparse or "residual" in st2) else {}
                    seg = [SegView(work, st2, sst, 0)]
                    t = time_cuda(lambda: hs.sync(seg), iters=max(2, a.iters // 2), warmup=1, flush=flush,
                                  setup=lambda: work.copy_(g), align=align)
                    row["unfused_ms"] = round(_max_over_ranks(t["median_ms"]) if N > 1 else t["median_ms"], 5)
                if "fused_ms" in row:
                    if N > 1:
                        row["speedup_vs_allreduce"] = round(ar_ms / row["fused_ms"], 3)
                    if "unfused_ms" in row:
                        row["speedup_vs_unfused"] = round(row["unfused_ms"] / row["fused_ms"], 3)
                rows.append(row)
                if R == 0:
                    print(json.dumps(row), flush=True)
                if arena is not None:
                    torch.cuda.synchronize()
                    arena.close()
                del fused, st
        del g, work
    if R == 0 and a.out:
        with open(a.out, "w") as f:
            json.dump(rows, f, indent=1)
    comm.shutdown()


if __name__ == "__main__":
    main()
