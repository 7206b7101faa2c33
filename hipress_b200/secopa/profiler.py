"""On-box cost profiler for the planner.

The reference states that its coefficients were "measured in our local cluster
and fit with the least square method" and ships no profiling tool
(src/SeCoPa/README.md:14-15 of mark14wu/hipress).  This module is that tool for
a B200 box: it times, over a sweep of gradient sizes,

* the stand-alone encode and decode kernels of the chosen algorithm,
* the fused ring / PS synchronisation (real ranks when launched under
  ``torch.distributed.run``, otherwise the ranks emulated on one GPU),
* the uncompressed all-reduce (NCCL) it competes with,

fits ``cost(x) = slope*x + intercept`` (milliseconds, x in fp32 elements) by least
squares with the smallest measured time as the floor, and writes a
:class:`~hipress_b200.secopa.planner.CostProfile` as JSON for ``--profile``.

    python -m hipress_b200.secopa.profiler --algorithm tbq --nnodes 8 --output b200_tbq_n8.json
"""
from __future__ import annotations

import argparse
import json

import torch

from .planner import CostProfile, LinearCost, TableCost


TILE = 4096   # elements per tile of the wire format: a rank's chunk should hold at least one
MARGIN = 0.1  # run-to-run spread of the sub-0.1 ms timings the fits' floors come from


def fit_linear(xs, ys) -> LinearCost:
    """Least-squares line through (x, y) with the minimum y as floor."""
    n = len(xs)
    if n == 0:
        return LinearCost()
    if n == 1:
        return LinearCost(0.0, ys[0], ys[0])
    mx, my = sum(xs) / n, sum(ys) / n
    sxx = sum((x - mx) ** 2 for x in xs)
    slope = sum((x - mx) * (y - my) for x, y in zip(xs, ys)) / sxx if sxx else 0.0
    slope = max(slope, 0.0)
    return LinearCost(slope, my - slope * mx, min(ys))


def _sizes(min_elems, max_elems):
    s, out = min_elems, []
    while s <= max_elems:
        out.append(s)
        s *= 4
    return out


def profile(algorithm="tbq", nnodes=8, min_elems=1 << 14, max_elems=1 << 26, iters=5, ctas=32,
            verbose=False) -> CostProfile:
    import torch.distributed as dist
    from ..bench.timing import L2Flusher, time_cuda
    from ..ops import Compressor
    from ..parallel import comm
    from ..parallel.fused import FusedDenseBucket

    comp = Compressor(algorithm)
    flush = L2Flusher()
    sizes = _sizes(min_elems, max_elems)
    real = comm.is_initialized() and comm.size() > 1
    if real:
        nnodes = comm.size()
    pts = {k: ([], []) for k in ("encode", "decode", "ring", "ps", "allreduce")}

    def add(key, n, t):
        pts[key][0].append(float(n))
        pts[key][1].append(t["median_ms"])
        if verbose and comm.rank() == 0:
            print(json.dumps({"term": key, "elems": n, "ms": round(t["median_ms"], 5)}), flush=True)

    for n in sizes:
        g = torch.randn(n, device="cuda")
        st = comp.new_state(n, "cuda")
        pay = torch.empty(comp.payload_bytes(n), dtype=torch.uint8, device="cuda")
        ws = comp.new_workspace("cuda", n)
        out = torch.empty(n, device="cuda")
        add("encode", n, time_cuda(lambda: comp.encode(g, st, out=pay, workspace=ws), iters=iters, flush=flush))
        add("decode", n, time_cuda(lambda: comp.decode(pay, out), iters=iters, flush=flush))
        if real:
            add("allreduce", n, time_cuda(lambda: dist.all_reduce(g), iters=iters, flush=flush))
        if comp.spec.sparse:
            continue
        ef = "residual" in comp.spec.state_names()
        if not real and n * 4 * nnodes * 3 <= 16e9:
            for topo in ("ring", "ps"):
                b = FusedDenseBucket(comp.spec, topo, [n], nnodes, 0, ctas=ctas, emulate=True)
                b.bind_local("cuda")
                G = torch.randn(nnodes, n, device="cuda")
                R = torch.zeros(nnodes, n, device="cuda") if ef else None
                t = time_cuda(lambda: b.launch([G], [R] if ef else None, [G]), iters=iters, flush=flush)
                # one GPU ran all ranks back to back: a rank's share is 1/N of it
                t = {k: v / nnodes for k, v in t.items()}
                add(topo, n, t)
                del b, G, R
    fits = {k: ((fit_linear if k in ("encode", "decode") else fit_table)(*v) if v[0] else None)
            for k, v in pts.items()}
    send = LinearCost(4.0 / 770e9 * 1e3, 0.003, 0.003)  # 770 GB/s measured peer copy, ~3 us latency
    return CostProfile(nodes=nnodes, encode=fits["encode"], decode=fits["decode"], ring_send=send,
                       gather=send, broadcast=send, comp_ratio=comp.payload_bytes(1 << 20) / (4 << 20),
                       fused_ring=fits["ring"], fused_ps=fits["ps"], allreduce=fits["allreduce"],
                       margin=MARGIN, min_compress_elems=nnodes * TILE,
                       source=f"measured on {torch.cuda.get_device_name()} ({'real' if real else 'emulated'} ranks)")


def fit_table(xs, ys) -> TableCost:
    """The measured points themselves (one time per size: the smallest seen)."""
    best = {}
    for x, y in zip(xs, ys):
        best[x] = min(y, best.get(x, y))
    return TableCost(tuple(sorted(best.items())))


def profile_from_sweep(path, algorithm="tbq", ops_path=None, fit="table", p2p_path=None) -> CostProfile:
    """Fit a profile from the rows a multi-GPU run of
    ``hipress_b200.bench.sweep_multi`` wrote (fused ring / PS and NCCL all-reduce
    times per size, measured on real ranks).  ``ops_path``: rows of
    ``hipress_b200.bench.sweep --what ops`` (stand-alone encode / decode times) for
    the encode and decode terms; without it the TBQ kernel coefficients stand in."""
    from ..ops import Compressor
    rows = [r for r in json.load(open(path)) if r["alg"] == algorithm]
    if not rows:
        raise ValueError(f"no rows for {algorithm} in {path}")
    n = rows[0]["n_gpus"]

    def term(key, topo=None):
        pts = [(r["bytes"] / 4.0, r[key]) for r in rows
               if key in r and r[key] and (topo is None or r["topo"] == topo)]
        pts = sorted(set(pts))
        fn = fit_table if fit == "table" else fit_linear
        return fn([p[0] for p in pts], [p[1] for p in pts]) if pts else None

    send = LinearCost(4.0 / 770e9 * 1e3, 0.003, 0.003)
    send_note = ""
    if p2p_path:   # rows of hipress_b200.bench.p2p: stores issued by a kernel into a peer's memory
        pr = json.load(open(p2p_path))
        send = fit_linear([r["bytes"] / 4.0 for r in pr], [r["ms"] for r in pr])
        send_note = ", send term from the in-kernel peer-store bench"
    enc = LinearCost(1.65e-9, 0.0208, 0.0196)   # stand-alone TBQ kernels, one B200 (profile())
    dec = LinearCost(1.26e-9, 0.0178, 0.0183)
    note = ""
    if ops_path:
        ops = [r for r in json.load(open(ops_path)) if r["alg"] == algorithm]
        for op in ("encode", "decode"):
            pts = sorted({(r["bytes"] / 4.0, r["ms"]) for r in ops if r["op"] == op})
            if pts:
                f = fit_linear([x for x, _ in pts], [y for _, y in pts])
                enc, dec = (f, dec) if op == "encode" else (enc, f)
        note = ", encode/decode from the kernel sweep"
    ratio = Compressor(algorithm).payload_bytes(1 << 20) / float(4 << 20)
    return CostProfile(nodes=n, encode=enc, decode=dec, ring_send=send, gather=send, broadcast=send,
                       comp_ratio=ratio, fused_ring=term("fused_ms", "ring"),
                       fused_ps=term("fused_ms", "ps"), allreduce=term("allreduce_ms"), margin=MARGIN,
                       min_compress_elems=n * TILE,
                       source=f"fitted from {n}-GPU sweep rows ({algorithm}){note}{send_note}")


def main(argv=None):
    ap = argparse.ArgumentParser(description="measure B200 cost coefficients for SeCoPa")
    ap.add_argument("--from-sweep", default=None,
                    help="fit from a sweep_multi JSON instead of measuring now")
    ap.add_argument("--from-ops-sweep", default=None,
                    help="with --from-sweep: kernel sweep JSON for the encode / decode terms")
    ap.add_argument("--from-p2p", default=None,
                    help="with --from-sweep: rows of hipress_b200.bench.p2p for the send term "
                         "(default: the 770 GB/s peer-copy figure)")
    ap.add_argument("--fit", default="table", choices=["table", "linear"],
                    help="with --from-sweep: keep the measured points (interpolated) or fit one line")
    ap.add_argument("--algorithm", default="tbq")
    ap.add_argument("--nnodes", type=int, default=8)
    ap.add_argument("--min-elems", type=int, default=1 << 14)
    ap.add_argument("--max-elems", type=int, default=1 << 26)
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--output", default="secopa_profile.json")
    ap.add_argument("--verbose", action="store_true")
    a = ap.parse_args(argv)
    if a.from_sweep:
        prof = profile_from_sweep(a.from_sweep, a.algorithm, a.from_ops_sweep, a.fit, a.from_p2p)
        with open(a.output, "w") as f:
            f.write(prof.to_json())
        print(a.output)
        return
    from ..parallel import comm
    comm.init()
    prof = profile(a.algorithm, a.nnodes, a.min_elems, a.max_elems, a.iters, verbose=a.verbose)
    if comm.rank() == 0:
        with open(a.output, "w") as f:
            f.write(prof.to_json())
        print(a.output)
    comm.shutdown()


if __name__ == "__main__":
    main()
