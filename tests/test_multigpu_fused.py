"""Fused ring / PS kernels across real GPUs (one process per GPU, peer memory
through CUDA IPC) against the lock-step simulation on the CPU oracle."""
import pytest
import torch

from _mp import spawn
from hipress_b200.ops import Compressor
from hipress_b200.parallel.simulate import chunk_elems, simulate_ps, simulate_ring

pytestmark = pytest.mark.multigpu

SIZES = [300001, 1 << 20, 5000, 70001]


def _grads(rank, step):
    g = torch.Generator().manual_seed(77 * step + rank)
    return [torch.randn(s, generator=g) * 0.02 for s in SIZES]


def _worker(rank, world, alg, topo, steps):
    import hipress_b200 as hp
    dev = hp.device()
    params = [torch.nn.Parameter(torch.zeros(s, device=dev)) for s in SIZES]
    names = [f"t{i}" for i in range(len(SIZES))]
    opt = hp.DistributedOptimizer(torch.optim.SGD(params, lr=1.0), list(zip(names, params)),
                                  algorithm=alg, topology=topo, comp_threshold=4096, ctas=16,
                                  timeout_s=5.0)
    assert opt.engine.backend == "fused"
    outs = []
    for step in range(steps):
        for p, g in zip(params, _grads(rank, step)):
            p.grad = g.to(dev)
        opt.synchronize()
        opt._synchronized = False
        torch.cuda.synchronize()
        outs.append([p.grad.cpu() for p in params])
    opt.engine.check()
    res = {"outs": outs, "launches": opt.engine.launch_count,
           "resid": [e.state["residual"].cpu() if "residual" in e.state else None
                     for e in opt.engine.entries]}
    opt.close()
    return res


def _world():
    return min(torch.cuda.device_count(), 8)


@pytest.mark.parametrize("alg,topo", [("tbq", "ring"), ("tbq", "ps"), ("onebit", "ring"),
                                      ("terngrad", "ps"), ("dgc", "ps"), ("graddrop", "ps"),
                                      ("dgc", "ring")])
def test_fused_multigpu_matches_simulation(alg, topo):
    world, steps = _world(), 2
    res = spawn(_worker, world, alg, topo, steps, backend="nccl")
    comp = Compressor(alg)
    ef = "residual" in comp.spec.state_names() or comp.spec.sparse
    states = [[comp.new_state(s, "cpu") for _ in range(world)] for s in SIZES]
    sst = [[({"residual": torch.zeros(chunk_elems(s, world))} if ef else {}) for _ in range(world)]
           for s in SIZES]
    for step in range(steps):
        gs = [_grads(r, step) for r in range(world)]
        for i, s in enumerate(SIZES):
            flat = [gs[r][i] for r in range(world)]
            if topo == "ring":
                ref = simulate_ring(comp, flat, states[i], step=step, tensor_id=i * 64)
            else:
                ref = simulate_ps(comp, flat, states[i], sst[i], step=step, tensor_id=i * 64)
            for r in range(world):
                got = res[r]["outs"][step][i]
                assert torch.allclose(got, ref[r], rtol=1e-5, atol=1e-8), (alg, topo, step, i, r)
                assert torch.equal(got, res[0]["outs"][step][i])
    assert res[0]["launches"] >= steps


def _ddp_vs_optimizer(rank, world, alg, topo):
    """The same one-tensor model trained through (a) DistributedDataParallel with the
    compression hook and (b) DistributedOptimizer: both run the fused kernels on the
    same layout (one tensor = one DDP bucket = one segment), so the parameters must
    agree bit for bit; the function API takes the fused path as well."""
    import hipress_b200 as hp
    from torch.nn.parallel import DistributedDataParallel as DDP
    from hipress_b200.parallel.hooks import FlatSyncer, ddp_comm_hook
    dev = hp.device()
    cfg = dict(algorithm=alg, topology=topo, comp_threshold=4096, threshold=1e-3, ratio=0.01, ctas=32,
               timeout_s=5.0)

    def data(step):
        g = torch.Generator().manual_seed(1000 * step + rank)
        return torch.randn(16, 512, generator=g).to(dev)

    def model():
        torch.manual_seed(0)
        return torch.nn.Linear(512, 1024, bias=False).to(dev)

    m1 = model()
    ddp = DDP(m1, device_ids=[dev.index])
    syncer = FlatSyncer(hp.HipressConfig(**cfg))
    ddp.register_comm_hook(syncer, ddp_comm_hook)
    o1 = torch.optim.SGD(m1.parameters(), lr=0.1)
    m2 = model()
    o2 = hp.DistributedOptimizer(torch.optim.SGD(m2.parameters(), lr=0.1), list(m2.named_parameters()), **cfg)
    assert o2.engine.backend == "fused"
    for step in range(3):
        x = data(step)
        o1.zero_grad()
        ddp(x).square().mean().backward()
        o1.step()
        o2.zero_grad()
        m2(x).square().mean().backward()
        o2.step()
    torch.cuda.synchronize()
    syncer.check()
    o2.engine.check()
    t = torch.full((20000,), 0.02 * (rank + 1), device=dev)
    fa = hp.allreduce(t, name="fa", algorithm="tbq", threshold=0.01)
    res = {"ddp": m1.weight.detach().cpu(), "opt": m2.weight.detach().cpu(), "launches": syncer.launch_count,
           "fa": fa.cpu()}
    syncer.close()
    o2.close()
    from hipress_b200.parallel import comm
    for s in comm._syncers.values():
        s.close()
    comm._syncers.clear()
    return res


@pytest.mark.parametrize("alg,topo", [("tbq", "ring"), ("onebit", "ps"), ("dgc", "ps")])
def test_ddp_hook_runs_the_fused_kernels_and_matches_the_optimizer(alg, topo):
    world = min(_world(), 4)
    res = spawn(_ddp_vs_optimizer, world, alg, topo, backend="nccl")
    for r in res:
        assert r["launches"] == 3, "one fused launch per DDP bucket and step"
        assert torch.equal(r["ddp"], r["opt"]), (alg, topo)
        assert torch.equal(r["ddp"], res[0]["ddp"])
        assert torch.equal(r["fa"], res[0]["fa"]) and float(r["fa"].abs().max()) > 0


def _elastic_gpu_worker(rank, world, port2, outdir, leave):
    from hipress_b200.train import pytorch_imagenet as T
    return T.main(["--model", "bert_tiny", "--batch-size", "2", "--seq-len", "16", "--num-iterations", "6",
                   "--fp32", "--algorithm", "tbq", "--comp-threshold", "1000", "--threshold", "0.0001",
                   "--heartbeat-timeout", "1.0", "--elastic", "--elastic-port", str(port2),
                   "--inject-leave", leave, "--metrics", f"{outdir}/m{rank}.jsonl"])


@pytest.mark.timeout(600)
@pytest.mark.parametrize("world", [2, 3])
def test_training_continues_on_gpus_after_a_rank_leaves(tmp_path, world):
    """Fused backend, real GPUs: the last rank leaves between two steps (announced on
    the host, nothing of it in flight); the survivors notice before their next launch,
    release the symmetric memory of the old membership without any collective (the
    group it was built on is gone), re-form -- down to a single rank when two become
    one -- and finish the epoch.  NVLS is off and the kernels use plain peer stores."""
    import json
    from _mp import free_port
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    env = {"NCCL_NVLS_ENABLE": "0", "HIPRESS_PG_TIMEOUT_S": "60"}
    res = spawn(_elastic_gpu_worker, world, free_port(), str(tmp_path), f"{world - 1}:3", backend="nccl", env=env)
    assert res == [0] * world
    recs = [json.loads(r) for r in (tmp_path / "m0.jsonl").read_text().splitlines()]
    assert recs[-1]["step"] == 6 and recs[-1]["ranks"] == world - 1
    assert recs[-1]["loss"] == recs[-1]["loss"]


def _hier_worker(rank, world, alg, topo, steps):
    """One box posing as two machines (HIPRESS_NODE_SIZE): fused kernels inside a
    machine, compressed exchange of shards between machines, all-gather inside."""
    import hipress_b200 as hp
    dev = hp.device()
    sizes = [300001, 5000]
    params = [torch.nn.Parameter(torch.zeros(s, device=dev)) for s in sizes]
    opt = hp.DistributedOptimizer(torch.optim.SGD(params, lr=1.0), [("big", params[0]), ("small", params[1])],
                                  algorithm=alg, topology=topo, comp_threshold=100000, ctas=16,
                                  timeout_s=5.0, threshold=0.002)
    eng = opt.engine
    outs = []
    for step in range(steps):
        g = torch.Generator().manual_seed(31 * step + rank)
        grads = [torch.randn(s, generator=g) * 0.02 for s in sizes]
        for p, x in zip(params, grads):
            p.grad = x.to(dev)
        opt.synchronize()
        opt._synchronized = False
        torch.cuda.synchronize()
        outs.append([p.grad.cpu() for p in params])
    eng.check()
    sd = opt.state_dict()["compressor_state"]
    res = {"outs": outs, "state": sd, "backend": eng.backend, "N": eng.N, "world": eng.world,
           "hier": eng.outer is not None and (eng.outer["nodes"], eng.outer["local"])}
    opt.close()
    return res


def test_one_box_split_in_two_machines_runs_hierarchically():
    from hipress_b200.parallel.simulate import chunk_range
    world = 8 if torch.cuda.device_count() >= 8 else 4
    if torch.cuda.device_count() < 4:
        pytest.skip("needs 4 GPUs")
    per, steps = world // 2, 4
    res = spawn(_hier_worker, world, "tbq", "ring", steps, backend="nccl",
                env={"HIPRESS_NODE_SIZE": str(per), "NCCL_NVLS_ENABLE": "0"})
    assert all(r["hier"] == (2, per) and r["N"] == per and r["world"] == world and r["backend"] == "fused"
               for r in res)
    for r in res[1:]:
        for s in range(steps):
            for a, b in zip(r["outs"][s], res[0]["outs"][s]):
                assert torch.equal(a, b), "replicas differ"
    sizes = [300001, 5000]
    def grads(rank, step):
        g = torch.Generator().manual_seed(31 * step + rank)
        return [torch.randn(s, generator=g) * 0.02 for s in sizes]
    for s in range(steps):                                  # uncompressed tensor: exact mean over the job
        want = sum(grads(r, s)[1] for r in range(world)) / world
        assert torch.allclose(res[0]["outs"][s][1], want, atol=1e-7)
    # conservation over both levels: delivered + residuals inside the machines + residuals of
    # the exchange between machines == exact mean
    n = sizes[0]
    delivered = sum(res[0]["outs"][s][0] for s in range(steps))
    exact = sum(sum(grads(r, s)[0] for r in range(world)) / world for s in range(steps))
    inner = sum(r["state"]["tensors"]["big"]["residual"] for r in res) / world
    outer = torch.zeros(n)
    for q, r in enumerate(res):
        lo, hi = chunk_range(n, per, q % per)
        outer[lo:hi] += r["state"]["between_machines"]["big.0"]["residual"] / 2
    assert torch.allclose(delivered + inner + outer, exact, atol=2e-6)
    assert not torch.allclose(delivered, exact, atol=1e-4)
