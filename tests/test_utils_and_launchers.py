"""Checkpoint round trip, metrics, host-side failure detection (gloo ranks, no GPU),
launcher command construction, SeCoPa plan consumption by the engine."""
import json
import os
import time

import pytest
import torch

from _mp import spawn

SHAPES = [(64, 100), (64,), (5000,)]


def _ckpt_worker(rank, world, d):
    import hipress_b200 as hp
    from hipress_b200.utils import load_checkpoint, save_checkpoint
    torch.manual_seed(0)
    model = torch.nn.Sequential(torch.nn.Linear(100, 64), torch.nn.Linear(64, 80))
    opt = hp.DistributedOptimizer(torch.optim.SGD(model.parameters(), lr=0.1, momentum=0.9),
                                  model.named_parameters(), algorithm="tbq", comp_threshold=1000,
                                  threshold=0.001)
    g = torch.Generator().manual_seed(rank)
    for _ in range(3):
        model(torch.randn(8, 100, generator=g)).pow(2).mean().backward()
        opt.step()
        opt.zero_grad()
    save_checkpoint(d, model, opt, epoch=2, step=3)
    before = opt.engine.state_dict()
    w_before = model[0].weight.detach().clone()
    # a fresh job resumes
    model2 = torch.nn.Sequential(torch.nn.Linear(100, 64), torch.nn.Linear(64, 80))
    opt2 = hp.DistributedOptimizer(torch.optim.SGD(model2.parameters(), lr=0.1, momentum=0.9),
                                   model2.named_parameters(), algorithm="tbq", comp_threshold=1000,
                                   threshold=0.001)
    info = load_checkpoint(d, model2, opt2)
    after = opt2.engine.state_dict()
    same = all(torch.equal(before["tensors"][k]["residual"], after["tensors"][k]["residual"])
               for k in before["tensors"])
    nz = any(float(v["residual"].abs().sum()) > 0 for v in before["tensors"].values())
    return {"info": info, "same": same, "nonzero": nz,
            "weights": torch.equal(w_before, model2[0].weight.detach()),
            "momentum": len(opt2.optimizer.state_dict()["state"]) > 0,
            "step": opt2.engine.step_no}


def test_checkpoint_roundtrip_with_compressor_state(tmp_path):
    res = spawn(_ckpt_worker, 2, str(tmp_path))
    for r in res:
        assert r["info"]["epoch"] == 2 and r["info"]["step"] == 3
        assert r["same"] and r["nonzero"] and r["weights"] and r["momentum"] and r["step"] == 3
    assert sorted(os.listdir(tmp_path)) == ["model.pt", "rank0.pt", "rank1.pt"]


def _health_worker(rank, world, mode):
    from hipress_b200.utils.health import HealthMonitor, PeerFailure, default_store
    import torch.distributed as dist
    mon = HealthMonitor(default_store(), rank, world, interval_s=0.05, timeout_s=0.6)
    dist.barrier()
    time.sleep(0.3)
    mon.check()  # everybody alive
    dist.barrier()
    out = "ok"
    if rank == world - 1:
        if mode == "leave":
            mon.leave()          # orderly exit between steps
        else:
            mon.pause()          # host thread stops beating (a hung rank)
        time.sleep(2.0)
    else:
        t0 = time.time()
        while time.time() - t0 < 3.0:
            try:
                mon.check()
            except PeerFailure as e:
                out = (e.ranks, "left" if "left" in str(e) else "silent", round(time.time() - t0, 1))
                break
            time.sleep(0.05)
    mon.close()
    return out


@pytest.mark.parametrize("mode", ["leave", "silent"])
def test_peer_failure_is_detected_on_the_host(mode):
    res = spawn(_health_worker, 3, mode)
    for r in res[:2]:
        assert r != "ok", "failure was not detected"
        ranks, kind, dt = r
        assert ranks == [2] and kind == ("left" if mode == "leave" else "silent") and dt < 2.5


def test_launcher_builds_a_local_torchrun_command(capsys):
    from hipress_b200.train import data_parallel_train as L
    rc = L.main(["--numprocess", "4", "--servers", "localhost:4", "--model", "vgg19", "--topo", "Ring",
                 "--comp-alg", "tbq", "--comp-threshold", "262144", "--horovodrun", "--interface",
                 "eth0", "--dry-run"])
    out = capsys.readouterr().out
    assert rc == 0 and "--nproc-per-node=4" in out and "--comp-alg tbq" in out and "--topo Ring" in out
    # the reference's own example: one GPU on each of two machines, reached over ssh
    rc = L.main(["--numprocess", "2", "--servers", "node1:1,node2:1", "--interface", "eth0",
                 "--comp-alg", "onebit", "--topo", "PS", "--dry-run"])
    lines = capsys.readouterr().out.strip().splitlines()
    assert rc == 0 and len(lines) == 2
    for k, (line, host) in enumerate(zip(lines, ("node1", "node2"))):
        assert line.startswith(f"ssh -p 22222 -o StrictHostKeyChecking=no {host} ")
        assert f"--nnodes=2 --node-rank={k} --nproc-per-node=1 --master-addr node1" in line
        assert "NCCL_SOCKET_IFNAME=eth0" in line and "--comp-alg onebit" in line
    for bad in (["--numprocess", "3", "--servers", "node1:1,node2:2"],
                ["--numprocess", "4", "--servers", "node1:1,node2:1"],
                ["--numprocess", "2", "--servers", "node1:1,node1:1"]):
        with pytest.raises(SystemExit):
            L.main(bad + ["--dry-run"])


def test_engine_consumes_a_secopa_plan(tmp_path):
    import hipress_b200 as hp
    params = [("a", torch.nn.Parameter(torch.zeros(30000))), ("b", torch.nn.Parameter(torch.zeros(30000))),
              ("c", torch.nn.Parameter(torch.zeros(10)))]
    plan = tmp_path / "plan.txt"
    plan.write_text("a,30000,y,3\nb,30000,n,4\nc,10,n,4\n")
    opt = hp.DistributedOptimizer(torch.optim.SGD([p for _, p in params], lr=1.0), params,
                                  algorithm="tbq", plan=str(plan), comp_threshold=1)
    eng = opt.engine
    by = {e.name: e for e in eng.entries}
    assert by["a"].compress and not by["b"].compress and not by["c"].compress
    fused = [b for b in eng.buckets if b.fused]
    assert len(fused) == 1 and [(s.lo, s.hi) for s in fused[0].segs] == [(0, 12288), (12288, 24576), (24576, 30000)]
    for _, p in params:
        p.grad = torch.full_like(p, 0.5)
    opt.step()
    assert torch.allclose(params[0][1].detach(), torch.full((30000,), -0.01))  # one tbq level
    assert torch.allclose(params[1][1].detach(), torch.full((30000,), -0.5))
    bad = tmp_path / "bad.txt"
    bad.write_text("a,7,y,1\n")
    with pytest.raises(ValueError):
        hp.DistributedOptimizer(torch.optim.SGD([p for _, p in params], lr=1.0), params,
                                algorithm="tbq", plan=str(bad))


def test_metrics_writer_and_engine_metrics(tmp_path):
    import hipress_b200 as hp
    from hipress_b200.utils import MetricsWriter, engine_metrics
    p = torch.nn.Parameter(torch.zeros(8192))
    opt = hp.DistributedOptimizer(torch.optim.SGD([p], lr=1.0), [("w", p)], algorithm="onebit",
                                  comp_threshold=1)
    p.grad = torch.randn(8192)
    opt.step()
    m = engine_metrics(opt.engine)
    assert m["compression_ratio"] > 25 and m["residual_norm"] > 0
    mw = MetricsWriter(str(tmp_path / "m.jsonl"))
    mw.step(1, loss=1.5, **m)
    mw.close()
    rec = json.loads((tmp_path / "m.jsonl").read_text().splitlines()[0])
    assert rec["step"] == 1 and rec["loss"] == 1.5 and rec["backend"] == "host"


def test_training_script_runs_end_to_end_on_cpu(tmp_path):
    from hipress_b200.train import pytorch_imagenet as T
    import hipress_b200 as hp
    rc = T.main(["--model", "bert_tiny", "--batch-size", "2", "--seq-len", "16", "--num-iterations", "3",
                 "--fp32", "--algorithm", "onebit", "--comp-threshold", "1000",
                 "--checkpoint-dir", str(tmp_path / "ck"), "--metrics", str(tmp_path / "m.jsonl")])
    assert rc == 0
    assert (tmp_path / "ck" / "model.pt").exists() and (tmp_path / "ck" / "rank0.pt").exists()
    rec = json.loads((tmp_path / "m.jsonl").read_text().splitlines()[-1])
    assert rec["loss"] == rec["loss"] and rec["compression_ratio"] > 1
    rc = T.main(["--model", "bert_tiny", "--batch-size", "2", "--seq-len", "16", "--num-iterations", "1",
                 "--epochs", "2", "--fp32", "--algorithm", "onebit", "--comp-threshold", "1000",
                 "--checkpoint-dir", str(tmp_path / "ck"), "--resume"])
    assert rc == 0


def _elastic_worker(rank, world, port2):
    """Three ranks train; rank 2 leaves between steps; ranks 0 and 1 detect it on the
    host, re-form a group of two and keep training with a rebuilt optimizer."""
    import hipress_b200 as hp
    import torch.distributed as dist
    from hipress_b200.parallel.elastic import reform_process_group, survivors_rendezvous
    from hipress_b200.utils.health import HealthMonitor, PeerFailure, default_store

    def make(pv):
        p = torch.nn.Parameter(pv.clone())
        opt = hp.DistributedOptimizer(torch.optim.SGD([p], lr=1.0), [("w", p)], algorithm="none")
        return p, opt

    store = default_store()
    mon = HealthMonitor(store, rank, world, interval_s=0.05, timeout_s=0.6)
    p, opt = make(torch.zeros(4))
    p.grad = torch.full((4,), float(rank + 1))
    opt.step()                                   # average of 1,2,3 = 2
    first = p.detach().clone()
    dist.barrier()
    if rank == 2:
        mon.leave()                              # orderly exit between steps
        time.sleep(1.5)
        return {"first": first, "left": True}
    dead = None
    t0 = time.time()
    while time.time() - t0 < 5:
        try:
            mon.check()
        except PeerFailure as e:
            dead = e.ranks
            break
        time.sleep(0.05)
    assert dead == [2]
    mon.close()
    new_rank, new_world = survivors_rendezvous(store, rank, world, dead, generation=1)
    reform_process_group(new_rank, new_world, port=port2, backend="gloo")
    assert hp.size() == 2 and hp.rank() == new_rank
    p2, opt2 = make(p.detach())                  # rebuilt for the new world size
    p2.grad = torch.full((4,), float(rank + 1))
    opt2.step()                                  # average of 1,2 = 1.5
    return {"first": first, "second": p2.detach().clone(), "new": (new_rank, new_world)}


def test_survivors_reform_a_smaller_group_and_continue():
    from _mp import free_port
    res = spawn(_elastic_worker, 3, free_port())
    assert res[2]["left"]
    for r in (0, 1):
        assert torch.allclose(res[r]["first"], torch.full((4,), -2.0))
        assert torch.allclose(res[r]["second"], torch.full((4,), -3.5))
        assert res[r]["new"] == (r, 2)


def _api_worker(rank, world):
    import hipress_b200 as hp
    t = torch.arange(6, dtype=torch.float32) + rank
    s = hp.allreduce(t, average=False)
    a = hp.allreduce(t)
    g = hp.allgather(torch.full((2, 3), float(rank)))
    b = hp.broadcast(torch.full((3,), float(rank)), root_rank=1)
    big = torch.full((5000,), 0.02 * (rank + 1))
    c1 = hp.allreduce(big, name="g", algorithm="tbq", threshold=0.01)
    c2 = hp.allreduce(big, name="g", algorithm="tbq", threshold=0.01)
    ragged = hp.allgather(torch.full((rank + 1, 2), float(rank)))     # 1 row from rank 0, 2 from rank 1
    objs = hp.allgather_object({"rank": rank})
    root = hp.broadcast_object({"from": rank}, root_rank=1)
    return {"s": s, "a": a, "g": g, "b": b, "c": (c1, c2), "ragged": ragged, "objs": objs, "root": root,
            "local_size": hp.local_size(), "alias": hp.DistributedTrainer is hp.DistributedOptimizer}


def test_horovod_style_function_api():
    res = spawn(_api_worker, 2)
    for r in res:
        assert torch.equal(r["s"], 2 * torch.arange(6, dtype=torch.float32) + 1)
        assert torch.equal(r["a"], torch.arange(6, dtype=torch.float32) + 0.5)
        assert r["g"].shape == (4, 3) and r["g"][:2].eq(0).all() and r["g"][2:].eq(1).all()
        assert r["b"].eq(1).all() and r["alias"]
        assert r["ragged"].shape == (3, 2) and r["ragged"][:, 0].tolist() == [0.0, 1.0, 1.0]
        assert r["objs"] == [{"rank": 0}, {"rank": 1}] and r["root"] == {"from": 1}
        assert r["local_size"] == 2
        # compressed: one +threshold level per rank and call (ring: partial sums are
        # re-quantised per hop), the rest stays in the error-feedback state
        c1, c2 = r["c"]
        assert torch.allclose(c1, torch.full((5000,), 0.005)) and torch.allclose(c2, c1)
    assert torch.equal(res[0]["c"][0], res[1]["c"][0])


@pytest.mark.parametrize("name,kw", [
    ("bert_base", dict(vocab_size=500, hidden=32, layers=2, heads=4, ffn=64, max_pos=32)),
    ("lstm", dict(vocab_size=300, emb=32, hidden=32)),
    ("transformer", dict(vocab_size=300, d_model=32, heads=4, layers=1, ffn=64, max_len=32)),
])
def test_sequence_model_zoo_trains_through_the_harness(name, kw):
    import hipress_b200 as hp
    from hipress_b200.train.harness import build_job
    cfg = hp.HipressConfig(algorithm="tbq", topology="ring", comp_threshold=1000, threshold=1e-4)
    job = build_job(name, cfg, batch=2, seq_len=8, dtype=torch.float32, model_kwargs=kw,
                    device=torch.device("cpu"))
    losses = [job.step(*job.to_device(*job.host_batch(i))).item() for i in range(3)]
    assert all(l == l and l > 0 for l in losses)
    assert job.optimizer.engine.stats()["compressed_elems"] > 0


def test_full_size_models_have_the_published_parameter_counts():
    from hipress_b200.models import get_model
    with torch.device("meta"):
        counts = {n: sum(p.numel() for p in get_model(n).parameters())
                  for n in ("vgg19", "resnet50", "bert_large", "bert_base", "lstm", "transformer")}
    assert counts["vgg19"] == 143_667_240 and counts["resnet50"] == 25_557_032
    assert 334e6 < counts["bert_large"] < 337e6 and 109e6 < counts["bert_base"] < 111e6
    assert 130e6 < counts["lstm"] < 140e6 and 55e6 < counts["transformer"] < 65e6


def test_training_script_reads_an_image_folder(tmp_path):
    """--train-dir: ImageNet-style directory -> sharded loader -> training steps."""
    from PIL import Image
    import numpy as np
    from hipress_b200.train import pytorch_imagenet as T
    rng = np.random.default_rng(0)
    for cls in ("cat", "dog"):
        d = tmp_path / "train" / cls
        d.mkdir(parents=True)
        for i in range(3):
            Image.fromarray(rng.integers(0, 255, (40, 48, 3), dtype=np.uint8)).save(d / f"{i}.png")
    rc = T.main(["--model", "resnet50", "--num-classes", "2", "--batch-size", "2", "--image-size", "32",
                 "--train-dir", str(tmp_path / "train"), "--val-dir", str(tmp_path / "train"),
                 "--workers", "0", "--num-iterations", "2", "--warmup-iters", "2", "--lr-decay-epochs", "1",
                 "--fp32", "--algorithm", "tbq", "--comp-threshold", "100000",
                 "--metrics", str(tmp_path / "m.jsonl")])
    assert rc == 0
    recs = [json.loads(r) for r in (tmp_path / "m.jsonl").read_text().splitlines()]
    train = [r for r in recs if "loss" in r]
    assert train and train[-1]["step"] == 2 and train[-1]["loss"] == train[-1]["loss"]
    val = [r for r in recs if "val_top1" in r]
    assert val and val[-1]["val_images"] == 6 and 0.0 <= val[-1]["val_top1"] <= 1.0


def _elastic_training_worker(rank, world, port2, outdir):
    from hipress_b200.train import pytorch_imagenet as T
    rc = T.main(["--model", "bert_tiny", "--batch-size", "2", "--seq-len", "16", "--num-iterations", "6",
                 "--fp32", "--algorithm", "tbq", "--comp-threshold", "1000", "--threshold", "0.0001",
                 "--heartbeat-timeout", "1.0", "--elastic", "--elastic-port", str(port2),
                 "--inject-leave", "2:3", "--metrics", f"{outdir}/m{rank}.jsonl"])
    return rc


def test_training_script_continues_after_a_rank_leaves(tmp_path):
    """Three ranks train; rank 2 leaves before step 3 (injected on the host); the
    other two notice between steps, re-form a job of two and finish the epoch."""
    from _mp import free_port
    res = spawn(_elastic_training_worker, 3, free_port(), str(tmp_path))
    assert res == [0, 0, 0]
    recs = [json.loads(r) for r in (tmp_path / "m0.jsonl").read_text().splitlines()]
    assert recs[-1]["step"] == 6 and recs[-1]["ranks"] == 2
    assert recs[-1]["loss"] == recs[-1]["loss"]


def _split_view_worker(rank, world):
    """Four ranks; ranks 2 and 3 leave at the same step.  Rank 0 only noticed rank 2,
    rank 1 only rank 3: the rendezvous must still give both the same membership."""
    from hipress_b200.parallel.elastic import survivors_rendezvous
    from hipress_b200.utils.health import default_store
    store = default_store()
    if rank >= 2:
        return {"left": True}
    seen = [2] if rank == 0 else [3]
    time.sleep(0.2 * rank)          # and they do not arrive together
    return {"new": survivors_rendezvous(store, rank, world, seen, generation=1, timeout_s=10.0)}


def test_survivors_agree_when_they_saw_different_failures():
    res = spawn(_split_view_worker, 4)
    assert res[0]["new"] == (0, 2) and res[1]["new"] == (1, 2)


def test_environment_overrides_convert_by_declared_type(monkeypatch):
    """Fields that default to None (bitwidth, plan) take their type from the
    declaration, not from the current value."""
    import hipress_b200 as hp
    monkeypatch.setenv("HIPRESS_BITWIDTH", "2")
    monkeypatch.setenv("HIPRESS_PLAN", "auto")
    monkeypatch.setenv("HIPRESS_OVERLAP", "0")
    monkeypatch.setenv("HIPRESS_RATIO", "0.01")
    monkeypatch.setenv("HIPRESS_STRICT_STATUS", "true")
    cfg = hp.HipressConfig.from_env()
    assert cfg.bitwidth == 2 and isinstance(cfg.bitwidth, int)
    assert cfg.plan == "auto" and cfg.overlap is False and cfg.ratio == 0.01 and cfg.strict_status is True
    spec = hp.get_algorithm("terngrad", **cfg.algorithm_kwargs())
    assert spec.bits == 2
    monkeypatch.setenv("HIPRESS_BITWIDTH", "none")
    assert hp.HipressConfig.from_env().bitwidth is None


def _subgroup_worker(rank, world):
    """FlatSyncer on a 2-of-4 sub-group: small (uncompressed) tensors are averaged
    over the sub-group only."""
    import torch.distributed as dist
    import hipress_b200 as hp
    from hipress_b200.parallel.hooks import FlatSyncer
    groups = [dist.new_group([0, 1]), dist.new_group([2, 3])]
    g = groups[rank // 2]
    fs = FlatSyncer(hp.HipressConfig(algorithm="tbq", comp_threshold=1000), group=g)
    small = torch.full((10,), float(rank))
    fs.sync_(small, key=0)
    a = hp.allreduce(torch.full((2000,), 0.02), algorithm="tbq", threshold=0.01)
    b = hp.allreduce(torch.full((3000,), 0.02), algorithm="tbq", threshold=0.01)   # unnamed, other size
    return {"small": small, "a": a, "b": b}


def test_flat_syncer_respects_its_group_and_unnamed_tensors_do_not_share_state():
    res = spawn(_subgroup_worker, 4)
    for r in range(4):
        assert torch.allclose(res[r]["small"], torch.full((10,), 0.5 if r < 2 else 2.5))
        assert res[r]["a"].shape == (2000,) and res[r]["b"].shape == (3000,)
