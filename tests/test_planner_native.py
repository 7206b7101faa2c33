"""The native bucket planner (csrc/cpu/planner.cpp) through the engine."""
import torch

import hipress_b200 as hp


def _engine(sizes, **cfg):
    params = [(f"p{i}", torch.nn.Parameter(torch.zeros(s))) for i, s in enumerate(sizes)]
    opt = hp.DistributedOptimizer(torch.optim.SGD([p for _, p in params], lr=1.0), params, **cfg)
    return opt.engine


def test_buckets_follow_completion_order_and_size_limits():
    # registration order p0..p5; backward produces p5 first
    sizes = [100, 5000, 300000, 50, 400000, 20]
    eng = _engine(sizes, algorithm="tbq", comp_threshold=1000, bucket_bytes=1 << 21)
    fused = [b for b in eng.buckets if b.fused]
    plain = [b for b in eng.buckets if not b.fused]
    assert [[e.name for e in b.entries] for b in fused] == [["p4"], ["p2", "p1"]]
    assert [[e.name for e in b.entries] for b in plain] == [["p5", "p3", "p0"]]
    # launch order = order of completion: a bucket is complete with its lowest index
    order = [min(e.index for e in b.entries) for b in eng.buckets]
    assert order == sorted(order, reverse=True)
    assert [b.index for b in eng.buckets] == list(range(len(eng.buckets)))


def test_partitions_are_tile_aligned_and_capped():
    eng = _engine([1_000_000], algorithm="tbq", comp_threshold=1000)
    assert [(s.lo, s.hi) for s in eng.buckets[0].segs] == [(0, 1_000_000)]
    import tempfile, os
    with tempfile.TemporaryDirectory() as d:
        plan = os.path.join(d, "plan.txt")
        open(plan, "w").write("p0,1000000,y,7\n")
        eng = _engine([1_000_000], algorithm="tbq", plan=plan)
        segs = [(s.lo, s.hi) for s in eng.buckets[0].segs]
        assert len(segs) == 7 and segs[0][0] == 0 and segs[-1][1] == 1_000_000
        assert all(lo % 4096 == 0 for lo, _ in segs)
        assert all(a[1] == b[0] for a, b in zip(segs, segs[1:]))
        # more partitions than a launch can hold: merged into fewer, larger ones
        open(plan, "w").write("p0,1000000,y,200\n")
        eng = _engine([1_000_000], algorithm="tbq", plan=plan)
        assert 1 <= len(eng.buckets[0].segs) <= 40


def test_uncompressed_run_has_only_plain_buckets():
    eng = _engine([5000, 10], algorithm="none")
    assert all(not b.fused for b in eng.buckets) and eng.backend == "allreduce"
