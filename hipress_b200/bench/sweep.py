"""Kernel sweep on one GPU: stand-alone encode / decode of the five algorithms and
the fused ring / PS kernels with N emulated ranks, fp32 gradients of 4 KB - 1 GB
(powers of 4), values N(0,1) seed 0.  Reports milliseconds, achieved GB/s over the
algorithmic HBM bytes and the fraction of the measured copy bandwidth.

    python -m hipress_b200.bench.sweep --what ops --out sweep_ops.json
    python -m hipress_b200.bench.sweep --what fused --ranks 8 --max-mb 256
    python -m hipress_b200.bench.sweep --what generated --mbytes 256   # CompLL output vs hand kernels
"""
from __future__ import annotations

import argparse
import json

import torch

from ..ops import Compressor
from ..parallel.fused import FusedDenseBucket
from .timing import L2Flusher, measured_peaks, time_cuda

ALGS = [("onebit", {}), ("tbq", {}), ("terngrad", {"bitwidth": 2}), ("dgc", {}), ("graddrop", {})]


def algorithmic_bytes(c: Compressor, n: int, op: str) -> float:
    """HBM bytes the op has to move at minimum."""
    sp = c.spec
    pay = c.payload_bytes(n)
    if op == "decode":
        return pay + 4.0 * n
    if sp.sparse:
        state = 20.0 if sp.name == "dgc" else 12.0  # read g,(u),v write (u),v
        return state * n + pay
    ef = 8.0 if "residual" in sp.state_names() else 0.0
    return (4.0 + ef) * n + pay


def sweep_ops(sizes, iters, out):
    peaks = measured_peaks()
    flush = L2Flusher()
    for name, kw in ALGS:
        c = Compressor(name, **kw)
        for nbytes in sizes:
            n = nbytes // 4
            g = torch.randn(n, device="cuda", generator=torch.Generator("cuda").manual_seed(0))
            st = c.new_state(n, "cuda")
            pay = torch.empty(c.payload_bytes(n), dtype=torch.uint8, device="cuda")
            ws = c.new_workspace("cuda", n)
            res = torch.empty(n, device="cuda")
            enc = time_cuda(lambda: c.encode(g, st, out=pay, workspace=ws), iters=iters, flush=flush)
            dec = time_cuda(lambda: c.decode(pay, res), iters=iters, flush=flush)
            for op, t in (("encode", enc), ("decode", dec)):
                b = algorithmic_bytes(c, n, op)
                gbs = b / (t["median_ms"] * 1e-3) / 1e9
                row = {"alg": name, "op": op, "bytes": nbytes, "ms": round(t["median_ms"], 5),
                       "min_ms": round(t["min_ms"], 5), "alg_gb": round(b / 1e9, 6),
                       "gbs": round(gbs, 1), "frac_hbm": round(gbs / peaks["hbm_gbs"], 4),
                       "peak_source": peaks["source"]}
                out.append(row)
                print(json.dumps(row), flush=True)
            del g, st, pay, res


def sweep_fused(sizes, iters, ranks, ctas, out):
    peaks = measured_peaks()
    flush = L2Flusher()
    for topo in ("ring", "ps"):
        for name, kw in ALGS[:3]:
            c = Compressor(name, **kw)
            ef = "residual" in c.spec.state_names()
            for nbytes in sizes:
                n = nbytes // 4
                if n * 4 * ranks * 3 > 24e9:
                    continue
                b = FusedDenseBucket(c.spec, topo, [n], ranks, 0, ctas=ctas, emulate=True)
                b.bind_local("cuda")
                G = torch.randn(ranks, n, device="cuda",
                                generator=torch.Generator("cuda").manual_seed(0))
                Rr = torch.zeros(ranks, n, device="cuda") if ef else None
                O = torch.empty(ranks, n, device="cuda")
                t = time_cuda(lambda: b.launch([G], [Rr] if ef else None, [O]), iters=iters,
                              flush=flush)
                b.check_status()
                # all emulated ranks share one GPU's HBM: bytes = ranks * per-rank bytes
                per_rank = (4.0 + (8.0 if ef else 0.0) + 4.0) * n
                gbs = per_rank * ranks / (t["median_ms"] * 1e-3) / 1e9
                row = {"kernel": f"{topo}_{name}", "ranks_emulated": ranks, "bytes": nbytes,
                       "ms": round(t["median_ms"], 5), "gbs_all_ranks": round(gbs, 1),
                       "frac_hbm": round(gbs / peaks["hbm_gbs"], 4), "ctas_per_rank": b.ctas,
                       "peak_source": peaks["source"]}
                out.append(row)
                print(json.dumps(row), flush=True)
                del b, G, Rr, O


def run_single(alg, topo, mbytes, ctas, iters, out, flush_l2=True, in_place=False):
    """One rank, one tensor, one fused launch per iteration (the case to hand to
    a profiler): encode + local hand-off + decode of `mbytes` of fp32 gradient."""
    peaks = measured_peaks()
    flush = L2Flusher() if flush_l2 else None
    c = Compressor(alg)
    n = mbytes * 1024 * 1024 // 4
    if c.spec.sparse:
        from ..parallel.fused_sparse import FusedSparseBucket
        b = FusedSparseBucket(c.spec, [n], 1, 0, topology=topo).bind_local("cuda")
        g = torch.randn(n, device="cuda", generator=torch.Generator("cuda").manual_seed(0))
        st = c.new_state(n, "cuda")
        acc = st["accum_v"] if "accum_v" in st else st["residual"]
        u = st.get("momentum_u")
        o = g if in_place else torch.empty(n, device="cuda")   # the engine synchronises in place
        sr = torch.zeros(b.chunk_elems(0), device="cuda")
        t = time_cuda(lambda: b.launch_ptrs([g.data_ptr()], [acc.data_ptr()],
                                            [u.data_ptr()] if u is not None else None,
                                            [o.data_ptr()], [sr.data_ptr()]), iters=iters, flush=flush)
        b.check_status()
        nbytes = ((20.0 if alg == "dgc" else 12.0) + 4.0 + (8.0 if topo == "ps" else 0.0)) * n
        gbs = nbytes / (t["median_ms"] * 1e-3) / 1e9
        row = {"kernel": f"{topo}_{alg}_1rank", "mbytes": mbytes, "ms": round(t["median_ms"], 5),
               "gbs": round(gbs, 1), "frac_hbm": round(gbs / peaks["hbm_gbs"], 4),
               "peak_source": peaks["source"],
               "phase_end_ms": [round(x, 4) for x in b.last_phase_times()],
               "marks_ms": [round(x, 4) for x in b.last_marks]}
        out.append(row)
        print(json.dumps(row), flush=True)
        return
    ef = "residual" in c.spec.state_names()
    b = FusedDenseBucket(c.spec, topo, [n], 1, 0, ctas=ctas).bind_local("cuda")
    g = torch.randn(n, device="cuda", generator=torch.Generator("cuda").manual_seed(0))
    r = torch.zeros(n, device="cuda") if ef else None
    o = torch.empty(n, device="cuda")
    t = time_cuda(lambda: b.launch([g], [r] if ef else None, [o]), iters=iters, flush=flush)
    b.check_status()
    nbytes = (8.0 + (8.0 if ef else 0.0)) * n
    gbs = nbytes / (t["median_ms"] * 1e-3) / 1e9
    row = {"kernel": f"{topo}_{alg}_1rank", "mbytes": mbytes, "ctas": b.ctas,
           "ms": round(t["median_ms"], 5), "gbs": round(gbs, 1),
           "frac_hbm": round(gbs / peaks["hbm_gbs"], 4), "peak_source": peaks["source"]}
    out.append(row)
    print(json.dumps(row), flush=True)


def sweep_generated(mbytes, iters, out):
    """Every dense operator generated from the shipped DSL sources (one fused launch
    per function) against its hand-written twin, on `mbytes` of fp32 gradient."""
    from ..compll import load_op
    peaks = measured_peaks()
    flush = L2Flusher()
    n = mbytes * 1024 * 1024 // 4
    g = torch.randn(n, device="cuda", generator=torch.Generator("cuda").manual_seed(0)) * 0.02
    res = torch.empty(n, device="cuda")
    cases = [("Tbq", "tbq", {}, 4 + (n + 3) // 4, lambda f, r, c: f(g, r, c, 0.01)),
             ("Onebit", "onebit", {}, 4 + (n + 7) // 8, lambda f, r, c: f(g, r, c)),
             ("TernGrad", "terngrad", {"bitwidth": 2}, 10 + (n + 3) // 4, lambda f, r, c: f(g, c, 2, seed=1))]
    for stem, alg, kw, nbytes, call in cases:
        hand = Compressor(alg, **kw)
        st = hand.new_state(n, "cuda")
        pay = torch.empty(hand.payload_bytes(n), dtype=torch.uint8, device="cuda")
        comp = torch.zeros(nbytes, dtype=torch.uint8, device="cuda")
        r = torch.zeros(n, device="cuda")
        enc, dec, acc = load_op(f"{stem}Encode"), load_op(f"{stem}Decode"), load_op(f"{stem}DecodeAccumulate")
        ops = [("encode", lambda: call(enc, r, comp), lambda: hand.encode(g, st, out=pay)),
               ("decode", lambda: dec(comp, res), lambda: hand.decode(pay, res)),
               ("decode_accumulate", lambda: acc(comp, res, 0.5),
                lambda: hand.decode(pay, res, scale=0.5, accumulate=True))]
        for op, gen_fn, hand_fn in ops:
            tg = time_cuda(gen_fn, iters=iters, flush=flush)
            th = time_cuda(hand_fn, iters=iters, flush=flush)
            row = {"operator": f"{stem}{op.title().replace('_', '')}", "mbytes": mbytes,
                   "generated_ms": round(tg["median_ms"], 5), "hand_ms": round(th["median_ms"], 5),
                   "generated_over_hand": round(tg["median_ms"] / th["median_ms"], 3),
                   "peak_source": peaks["source"]}
            out.append(row)
            print(json.dumps(row), flush=True)
    # DGC encode: the generated function is one kernel for both state updates plus the
    # run-time library's exact top-k; the hand-written path folds the updates into the
    # selection's histogram pass
    ratio, m = 0.001, 0.9
    k = int(n * ratio) + 16      # the function rounds ratio * n up in fp32; the buffer may be larger
    hand = Compressor("dgc", ratio=ratio)
    st = hand.new_state(n, "cuda")
    pay = torch.empty(hand.payload_bytes(n), dtype=torch.uint8, device="cuda")
    comp = torch.zeros(16 + 2 * ((4 * k + 15) // 16 * 16), dtype=torch.uint8, device="cuda")
    u, v = torch.zeros(n, device="cuda"), torch.zeros(n, device="cuda")
    enc = load_op("DgcEncode")
    tg = time_cuda(lambda: enc(g, u, v, comp, ratio, m), iters=iters, flush=flush)
    ws = hand.new_workspace("cuda", n)
    th = time_cuda(lambda: hand.encode(g, st, out=pay, workspace=ws), iters=iters, flush=flush)
    row = {"operator": "DgcEncode", "mbytes": mbytes, "generated_ms": round(tg["median_ms"], 5),
           "hand_ms": round(th["median_ms"], 5),
           "generated_over_hand": round(tg["median_ms"] / th["median_ms"], 3), "peak_source": peaks["source"]}
    out.append(row)
    print(json.dumps(row), flush=True)


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--what", choices=["ops", "fused", "single", "generated", "all"], default="all")
    ap.add_argument("--alg", default="tbq")
    ap.add_argument("--topo", default="ring")
    ap.add_argument("--mbytes", type=int, default=256)
    ap.add_argument("--min-kb", type=int, default=4)
    ap.add_argument("--max-mb", type=int, default=1024)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--ranks", type=int, default=8)
    ap.add_argument("--ctas", type=int, default=32, help="CTAs per emulated rank")
    ap.add_argument("--out", default=None)
    ap.add_argument("--in-place", action="store_true",
                    help="--what single, sparse: the result overwrites the gradient, as in training")
    ap.add_argument("--no-flush", action="store_true",
                    help="--what single: leave L2 (data and code) warm between timed runs")
    a = ap.parse_args(argv)
    sizes = []
    s = a.min_kb * 1024
    while s <= a.max_mb * 1024 * 1024:
        sizes.append(s)
        s *= 4
    out = []
    if a.what == "single":
        run_single(a.alg, a.topo, a.mbytes, a.ctas, a.iters, out, flush_l2=not a.no_flush, in_place=a.in_place)
    if a.what == "generated":
        sweep_generated(a.mbytes, a.iters, out)
    if a.what in ("ops", "all"):
        sweep_ops(sizes, a.iters, out)
    if a.what in ("fused", "all"):
        sweep_fused(sizes, a.iters, a.ranks, a.ctas, out)
    if a.out:
        with open(a.out, "w") as f:
            json.dump(out, f, indent=1)


if __name__ == "__main__":
    main()
