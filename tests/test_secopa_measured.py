"""SeCoPa with measured profiles: cost tables, the decision margin, the minimum
compressed size, the joint (bucketed) plan and the shipped B200 profiles."""
import subprocess
import sys
from pathlib import Path

import pytest

from hipress_b200.secopa import CostProfile, LinearCost, Planner, TableCost
from hipress_b200.secopa.profiler import fit_linear, fit_table, profile_from_sweep

ROOT = Path(__file__).resolve().parents[1]
PROFILES = ROOT / "hipress_b200" / "secopa" / "profiles"


def _zero():
    return LinearCost()


def _profile(**kw):
    return CostProfile(nodes=8, encode=_zero(), decode=_zero(), ring_send=_zero(), gather=_zero(),
                       broadcast=_zero(), **kw)


def test_table_cost_interpolates_and_extrapolates():
    t = TableCost(((4000, 0.08), (1000, 0.05), (2000, 0.06)))     # any order in
    assert t.points[0] == (1000.0, 0.05)
    assert t(10) == 0.05                                            # latency floor
    assert t(1500) == pytest.approx(0.055)
    assert t(4000) == pytest.approx(0.08)
    assert t(8000) == pytest.approx(0.08 + 0.01 * 4)                # last slope continues
    falling = TableCost(((1000, 0.05), (2000, 0.04)))
    assert falling(4000) == pytest.approx(0.04)                     # never extrapolates downwards
    with pytest.raises(ValueError):
        TableCost(())


def test_profiles_with_tables_round_trip_through_json():
    prof = _profile(fused_ring=TableCost(((1000, 0.05), (1e6, 0.06))),
                    allreduce=LinearCost(1e-8, 0.07, 0.05), margin=0.1, min_compress_elems=32768)
    back = CostProfile.from_json(prof.to_json())
    assert isinstance(back.fused_ring, TableCost) and back.fused_ring.points == prof.fused_ring.points
    assert isinstance(back.allreduce, LinearCost) and back.margin == 0.1
    assert back.min_compress_elems == 32768


def test_margin_and_minimum_size_keep_marginal_gradients_uncompressed():
    fused = TableCost(((1000, 0.048), (1e6, 0.06), (1e8, 0.4)))
    plain = TableCost(((1000, 0.054), (1e6, 0.058), (1e8, 1.0)))
    strict = Planner(_profile(fused_ring=fused, allreduce=plain))
    assert strict.decide(1000, "RING")[0] == "y"        # 0.048 < 0.054: noise decides
    careful = Planner(_profile(fused_ring=fused, allreduce=plain, margin=0.15))
    assert careful.decide(1000, "RING")[0] == "n"
    assert careful.decide(10**8, "RING") == ("y", 1)
    small = Planner(_profile(fused_ring=fused, allreduce=plain, min_compress_elems=32768))
    assert small.decide(1000, "RING")[0] == "n" and small.decide(10**8, "RING")[0] == "y"


def test_bucketed_plan_amortises_the_launch_latency():
    """200 gradients of 1M elements: one by one each loses to the all-reduce (0.2 ms
    launch floor of the fused path), together they share one launch and win."""
    fused = TableCost(((1e5, 0.2), (1e6, 0.2), (2e8, 1.0)))
    plain = TableCost(((1e5, 0.05), (1e6, 0.06), (2e8, 3.0)))
    prof = _profile(fused_ps=fused, fused_ring=fused, allreduce=plain, margin=0.1, min_compress_elems=32768)
    grads = [(f"w{i}", 1_000_000) for i in range(200)] + [(f"b{i}", 1000) for i in range(200)]
    p = Planner(prof)
    assert all(r[2] == "n" for r in p.plan(grads, "PS"))
    rows = p.plan_bucketed(grads, "PS")
    assert [r[2] for r in rows[:200]] == ["y"] * 200
    assert [r[2] for r in rows[200:]] == ["n"] * 200       # under the minimum size
    # nothing to gain: everything stays plain
    slow = _profile(fused_ps=TableCost(((1e5, 5.0), (2e8, 9.0))), allreduce=plain)
    assert all(r[2] == "n" for r in Planner(slow).plan_bucketed(grads, "PS"))
    with pytest.raises(ValueError):
        Planner(_profile()).plan_bucketed(grads, "PS")


def test_fit_helpers():
    line = fit_linear([1.0, 2.0, 3.0], [3.0, 5.0, 7.0])
    assert line.slope == pytest.approx(2.0) and line.intercept == pytest.approx(1.0) and line.floor == 3.0
    table = fit_table([2.0, 1.0, 2.0], [5.0, 3.0, 4.5])
    assert table.points == ((1.0, 3.0), (2.0, 4.5))


@pytest.mark.parametrize("alg", ["onebit", "tbq", "terngrad", "dgc", "graddrop"])
@pytest.mark.parametrize("n", [2, 4, 8])
def test_shipped_profiles_give_sane_vgg19_plans(alg, n, vgg19_gradient_list):
    from hipress_b200.secopa import read_gradient_list
    prof = CostProfile.from_json((PROFILES / f"b200_{alg}_n{n}.json").read_text())
    assert prof.nodes == n and prof.allreduce is not None and prof.min_compress_elems == n * 4096
    grads = read_gradient_list(vgg19_gradient_list)
    for topo in ("RING", "PS"):
        rows = Planner(prof).plan(grads, topo)
        by = {r[0]: r for r in rows}
        assert by["vgg0_dense2_bias"][2] == "n" and by["vgg0_conv0_bias"][2] == "n"
        compressed = [r[1] for r in rows if r[2] == "y"]
        plain = [r[1] for r in rows if r[2] == "n"]
        # a size threshold in effect: nothing compressed is smaller than something left plain
        if compressed and plain:
            assert min(compressed) >= max(s for s in plain if s < min(compressed))
    # the quantisers pay off on the 392 MB FC layer at either size, over the ring
    if alg in ("onebit", "tbq", "terngrad"):
        assert {r[0]: r for r in Planner(prof).plan(grads, "RING")}["vgg0_dense0_weight"][2] == "y"


def test_profile_from_sweep_rows(tmp_path):
    import json
    rows = []
    for b, ar, fr, fp in [(4096, 0.05, 0.06, 0.07), (1 << 20, 0.06, 0.07, 0.08), (1 << 28, 0.8, 0.25, 0.3)]:
        rows.append({"alg": "tbq", "topo": "ring", "bytes": b, "n_gpus": 4, "allreduce_ms": ar, "fused_ms": fr})
        rows.append({"alg": "tbq", "topo": "ps", "bytes": b, "n_gpus": 4, "allreduce_ms": ar, "fused_ms": fp})
    ops = [{"alg": "tbq", "op": op, "bytes": b, "ms": 0.02 + b * 1e-10} for op in ("encode", "decode")
           for b in (4096, 1 << 20, 1 << 28)]
    (tmp_path / "multi.json").write_text(json.dumps(rows))
    (tmp_path / "ops.json").write_text(json.dumps(ops))
    prof = profile_from_sweep(tmp_path / "multi.json", "tbq", tmp_path / "ops.json")
    assert prof.nodes == 4 and prof.min_compress_elems == 4 * 4096 and prof.margin > 0
    assert prof.fused_ring(1 << 26) == pytest.approx(0.25) and prof.fused_ps(1 << 26) == pytest.approx(0.3)
    assert prof.encode.slope == pytest.approx(4e-10, rel=1e-3)
    assert prof.comp_ratio == pytest.approx(1 / 16, rel=0.01)
    line = profile_from_sweep(tmp_path / "multi.json", "tbq", fit="linear")
    assert isinstance(line.fused_ring, LinearCost)
    with pytest.raises(ValueError):
        profile_from_sweep(tmp_path / "multi.json", "dgc")


def test_cli_bucketed_flag(tmp_path, vgg19_gradient_list):
    out = tmp_path / "plan.txt"
    subprocess.run([sys.executable, "-m", "hipress_b200.secopa", "--input", str(vgg19_gradient_list),
                    "--output", str(out), "--topology", "RING", "--nnodes", "8", "--bucketed",
                    "--profile", str(PROFILES / "b200_tbq_n8.json")], check=True, cwd=ROOT)
    rows = [r.split(",") for r in out.read_text().splitlines()]
    assert len(rows) == 38
    assert all(r[2] == ("y" if int(r[1]) >= 8 * 4096 else "n") for r in rows)


def test_engine_plan_auto_bucketed(tmp_path):
    import torch
    import hipress_b200 as hp
    prof = _profile(fused_ring=TableCost(((1e3, 0.2), (1e8, 1.0))), allreduce=TableCost(((1e3, 0.05), (1e8, 3.0))),
                    min_compress_elems=4096)
    prof.nodes = 1
    path = tmp_path / "prof.json"
    path.write_text(prof.to_json())
    ps = [torch.nn.Parameter(torch.zeros(n)) for n in (8_000_000, 8_000_000, 5000, 100)]
    named = [(f"p{i}", p) for i, p in enumerate(ps)]
    opt = hp.DistributedOptimizer(torch.optim.SGD(ps, lr=1.0), named, algorithm="tbq",
                                  plan="auto:bucketed", plan_profile=str(path))
    assert [e.compress for e in opt.engine.entries] == [True, True, True, False]
    opt.close()
    opt = hp.DistributedOptimizer(torch.optim.SGD(ps, lr=1.0), named, algorithm="tbq",
                                  plan="auto", plan_profile=str(path))
    # one by one, a 5000-element gradient never repays the fused launch
    assert [e.compress for e in opt.engine.entries][2:] == [False, False]
    opt.close()


def test_cli_takes_the_gradient_list_from_the_model_zoo(tmp_path):
    out = tmp_path / "plan.txt"
    subprocess.run([sys.executable, "-m", "hipress_b200.secopa", "--model", "vgg19", "--output", str(out),
                    "--topology", "PS", "--nnodes", "4"], check=True, cwd=ROOT)
    rows = [r.split(",") for r in out.read_text().splitlines()]
    assert len(rows) == 38 and rows[32][:2] == ["vgg0_dense0_weight", "102760448"] and rows[32][2] == "y"
