"""The native bucket planner (csrc/cpu/planner.cpp) through the engine."""
import pytest
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


def test_measured_profile_compresses_only_what_pays_off_on_nvswitch(vgg19_gradient_list):
    """With coefficients fitted on the 8 x B200 box the planner keeps small
    gradients on the plain all-reduce and compresses the large FC layers."""
    from pathlib import Path
    from hipress_b200.secopa import CostProfile, Planner, read_gradient_list
    root = Path(__file__).resolve().parents[1]
    prof = CostProfile.from_json((root / "hipress_b200/secopa/profiles/b200_tbq_n8.json").read_text())
    assert prof.nodes == 8 and prof.fused_ring is not None and prof.allreduce is not None
    rows = Planner(prof).plan(read_gradient_list(vgg19_gradient_list), "RING")
    by = {r[0]: r for r in rows}
    assert by["vgg0_dense0_weight"][2] == "y" and by["vgg0_dense1_weight"][2] == "y"
    assert by["vgg0_conv0_weight"][2] == "n" and by["vgg0_dense2_bias"][2] == "n"


def test_gradient_accumulation_and_unused_parameters():
    used = torch.nn.Parameter(torch.zeros(5000))
    unused = torch.nn.Parameter(torch.zeros(3000))
    small = torch.nn.Parameter(torch.zeros(10))
    params = [("used", used), ("unused", unused), ("small", small)]
    opt = hp.DistributedOptimizer(torch.optim.SGD([p for _, p in params], lr=1.0), params,
                                  algorithm="tbq", comp_threshold=1000, threshold=0.01,
                                  backward_passes_per_step=2)
    for micro in range(2):                  # two micro-batches, one synchronisation
        (used.sum() * 0.02 + small.sum()).backward()
        if micro == 0:
            assert not any(b.launched for b in opt.engine.buckets)
    opt.step()
    # accumulated gradient 0.04 per element -> one +threshold level sent, rest kept
    assert torch.allclose(used.detach(), torch.full((5000,), -0.01))
    assert torch.allclose(small.detach(), torch.full((10,), -2.0))
    assert torch.all(unused.detach() == 0) and unused.grad is not None
    res = opt.engine.entries[0].state["residual"]
    assert torch.allclose(res, torch.full((5000,), 0.03))


def test_plan_auto_uses_a_measured_profile(tmp_path):
    from hipress_b200.secopa import CostProfile, LinearCost
    prof = CostProfile(nodes=1, encode=LinearCost(), decode=LinearCost(), ring_send=LinearCost(),
                       gather=LinearCost(), broadcast=LinearCost(),
                       fused_ring=LinearCost(3e-9, 0.1, 0.05), allreduce=LinearCost(1e-8, 0.08, 0.05))
    path = tmp_path / "prof.json"
    path.write_text(prof.to_json())
    # crossover at (0.1 - 0.08) / (1e-8 - 3e-9) ~ 2.86 M elements
    eng = _engine([4_000_000, 1_000_000, 100], algorithm="tbq", plan="auto", plan_profile=str(path),
                  comp_threshold=1)
    assert [e.compress for e in eng.entries] == [True, False, False]
    # no profile for this world size: the threshold decides
    eng = _engine([4_000_000, 1_000_000, 100], algorithm="tbq", plan="auto", comp_threshold=500_000)
    assert [e.compress for e in eng.entries] == [True, True, False]


def test_horovod_clipping_pattern_with_skip_synchronize():
    p = torch.nn.Parameter(torch.zeros(4))
    opt = hp.DistributedOptimizer(torch.optim.SGD([p], lr=1.0), [("w", p)], algorithm="none")
    p.grad = torch.full((4,), 3.0)
    opt.synchronize()
    torch.nn.utils.clip_grad_norm_([p], 1.0)
    with opt.skip_synchronize():
        opt.step()
    assert torch.allclose(p.detach(), torch.full((4,), -0.5)) and not opt._synchronized
    opt.close()


def test_overlapped_optimizer_keeps_sharing_state_after_a_checkpoint_load():
    def make(overlap):
        torch.manual_seed(0)
        model = torch.nn.Sequential(torch.nn.Linear(32, 64), torch.nn.Linear(64, 8))
        inner = torch.optim.SGD(model.parameters(), lr=0.1, momentum=0.9)
        opt = hp.DistributedOptimizer(inner, list(model.named_parameters()), algorithm="tbq",
                                      comp_threshold=1000, threshold=1e-4, bucket_bytes=4096,
                                      overlap_optimizer=overlap)
        return model, opt

    def run(model, opt, steps, seed):
        g = torch.Generator().manual_seed(seed)
        for _ in range(steps):
            opt.zero_grad()
            model(torch.randn(8, 32, generator=g)).square().mean().backward()
            opt.step()

    ref_m, ref_o = make(False)
    run(ref_m, ref_o, 4, 1)
    m1, o1 = make(True)
    run(m1, o1, 2, 1)
    sd = {"model": {k: v.clone() for k, v in m1.state_dict().items()}, "opt": o1.state_dict()}
    m2, o2 = make(True)                      # a fresh job resumes from the checkpoint
    m2.load_state_dict(sd["model"])
    o2.load_state_dict(sd["opt"])
    g = torch.Generator().manual_seed(1)
    for _ in range(2):
        torch.randn(8, 32, generator=g)      # skip the batches the first job consumed
    for _ in range(2):
        o2.zero_grad()
        m2(torch.randn(8, 32, generator=g)).square().mean().backward()
        o2.step()
    for a, b in zip(ref_m.parameters(), m2.parameters()):
        assert torch.allclose(a, b, atol=1e-7)
    assert len(o2.optimizer.state_dict()["state"]) == 4
    for o in (ref_o, o1, o2):
        o.close()


def test_bad_parameter_lists_and_sparse_gradients_are_refused():
    a, b = torch.nn.Parameter(torch.zeros(10)), torch.nn.Parameter(torch.zeros(10))
    with pytest.raises(ValueError, match="twice"):
        hp.GradSyncEngine([("w", a), ("w", b)], hp.HipressConfig(algorithm="tbq"))
    with pytest.raises(ValueError, match="twice"):
        hp.GradSyncEngine([("w", a), ("v", a)], hp.HipressConfig(algorithm="tbq"))
    emb = torch.nn.Embedding(50, 40, sparse=True)
    opt = hp.DistributedOptimizer(torch.optim.SGD(emb.parameters(), lr=0.1), list(emb.named_parameters()),
                                  algorithm="tbq", comp_threshold=100)
    with pytest.raises(TypeError, match="sparse"):   # raised from the hook that launches the bucket
        emb(torch.tensor([1, 2])).sum().backward()
        opt.step()
    opt.close()
