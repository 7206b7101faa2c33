"""The command-line contracts that need no GPU: the reference arm of bench.py, the
build entry point, and the SeCoPa CLI against the golden plans."""
import json
import os
import subprocess
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]


def test_reference_arm_reports_unavailable():
    out = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--impl", "reference", "--gpus", "1",
                          "--steps", "2", "--warmup", "1"], capture_output=True, text=True, timeout=120)
    assert out.returncode == 0
    line = json.loads(out.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and "unavailable" in line and "\n" not in line["unavailable"]


def test_reference_arm_prints_one_line_per_job_under_torchrun():
    """For N > 1 the arm is launched like the product arm, one process per GPU: only
    rank 0 answers."""
    out = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
                          "--master-addr", "127.0.0.1", "--master-port", "29587", str(ROOT / "bench.py"),
                          "--impl", "reference", "--gpus", "2", "--steps", "2", "--warmup", "1"],
                         capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stderr[-2000:]
    lines = [l for l in out.stdout.splitlines() if l.startswith("{")]
    assert len(lines) == 1 and json.loads(lines[0])["impl"] == "reference"


def test_graft_entry_has_build_and_smoke():
    sys.path.insert(0, str(ROOT))
    import __graft_entry__ as g
    assert callable(g.build) and callable(g.smoke)
    g.build()  # compiles nothing when up to date, imports the package, loads both libraries
    from hipress_b200._native import lib
    assert lib.cuda().hp_cuda_error_string(-1)


@pytest.mark.parametrize("topology,nnodes", [("PS", 4), ("PS", 8), ("PS", 16), ("RING", 4), ("RING", 8),
                                             ("RING", 16)])
def test_secopa_cli_reproduces_the_reference_plans(tmp_path, vgg19_gradient_list, topology, nnodes):
    gold = json.loads((ROOT / "tests" / "data" / "secopa_golden_plans.json").read_text())
    out = tmp_path / "plan.txt"
    rc = subprocess.run([sys.executable, "-m", "hipress_b200.secopa", "--input",
                         str(vgg19_gradient_list), "--output", str(out),
                         "--topology", topology, "--nnodes", str(nnodes)], cwd=ROOT, timeout=120)
    assert rc.returncode == 0
    rows = out.read_text().splitlines()
    assert len(rows) == 38
    got = [r.split(",")[2] + r.split(",")[3] for r in rows]
    assert got == gold[f"{topology}_{nnodes}"]
    assert rows[32].startswith("vgg0_dense0_weight,102760448,y,")


def test_secopa_rejects_unmeasured_cluster_sizes_but_profiles_cover_any_n(tmp_path):
    from hipress_b200.secopa import CostProfile, LinearCost, Planner, reference_profile
    with pytest.raises(ValueError):
        reference_profile(2)
    prof = CostProfile(nodes=2, encode=LinearCost(1e-8, 0.01, 0.01), decode=LinearCost(1e-8, 0.01, 0.01),
                       ring_send=LinearCost(5e-9, 0.003, 0.003), gather=LinearCost(5e-9, 0.003, 0.003),
                       broadcast=LinearCost(5e-9, 0.003, 0.003),
                       fused_ring=LinearCost(3e-9, 0.03, 0.03), allreduce=LinearCost(8e-9, 0.05, 0.05))
    p = Planner(CostProfile.from_json(prof.to_json()))
    assert p.decide(100_000_000, "RING")[0] == "y"
    assert p.decide(100, "RING")[0] == "y"  # 0.03 ms fused floor beats the 0.05 ms all-reduce floor
    prof2 = CostProfile.from_json(prof.to_json())
    prof2.fused_ring = LinearCost(3e-9, 0.2, 0.2)
    assert Planner(prof2).decide(100, "RING")[0] == "n"
