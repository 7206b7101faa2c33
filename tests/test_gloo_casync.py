"""Multi-process CPU tests (gloo, world_size 2 and 3): the CaSync host schedule
against the lock-step simulation, and the headline CPU configuration: TBQ
(threshold 0.01) + error feedback, CaSync-Ring, comp-threshold 1024, MLP
784->256->10 gradients ~ N(0, 1e-3), 10 steps against uncompressed all-reduce."""
import os
import socket
import tempfile

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from hipress_b200.ops import Compressor
from hipress_b200.parallel.simulate import chunk_elems, simulate_ps, simulate_ring

SHAPES = [(256, 784), (256,), (10, 256), (10,)]


def _spawn(fn, world, *args):
    from _mp import spawn
    return spawn(fn, world, *args, backend="gloo")


def _grads(rank, step):
    g = torch.Generator().manual_seed(1000 * step + rank)
    return [torch.randn(s, generator=g) * 1e-3 for s in SHAPES]


# ----------------------------------------------------------------------------
def _run_optimizer(rank, world, alg, topo, steps):
    import hipress_b200 as hp
    params = [torch.nn.Parameter(torch.zeros(s)) for s in SHAPES]
    names = ["fc1.weight", "fc1.bias", "fc2.weight", "fc2.bias"]
    opt = hp.DistributedOptimizer(torch.optim.SGD(params, lr=1.0), list(zip(names, params)),
                                  algorithm=alg, topology=topo, comp_threshold=1024,
                                  threshold=0.01, ratio=0.01)
    outs = []
    for step in range(steps):
        for p, g in zip(params, _grads(rank, step)):
            p.grad = g.clone()
        opt.synchronize()
        outs.append([p.grad.clone() for p in params])
        opt._synchronized = False
    state = opt.state_dict()["compressor_state"]
    return {"outs": outs, "state": state, "stats": opt.engine.stats()}


def _simulate(world, alg, topo, steps, **kw):
    comp = Compressor(alg, threshold=0.01, ratio=0.01)
    big = [i for i, s in enumerate(SHAPES) if torch.Size(s).numel() >= 1024]
    states = {i: [comp.new_state(torch.Size(SHAPES[i]).numel(), "cpu") for _ in range(world)] for i in big}
    sst = {i: [({"residual": torch.zeros(chunk_elems(torch.Size(SHAPES[i]).numel(), world))}
                if (comp.spec.sparse or "residual" in comp.spec.state_names()) else {})
               for _ in range(world)] for i in big}
    outs = []
    for step in range(steps):
        gs = [_grads(r, step) for r in range(world)]
        row = []
        for i, s in enumerate(SHAPES):
            if i in big:
                flat = [gs[r][i].reshape(-1).clone() for r in range(world)]
                if topo == "ring":
                    res = simulate_ring(comp, flat, states[i], step=step, tensor_id=i * 64)
                else:
                    res = simulate_ps(comp, flat, states[i], sst[i], step=step, tensor_id=i * 64)
                row.append(res[0].view(s))
            else:
                row.append(sum(gs[r][i] for r in range(world)) / world)
        outs.append(row)
    return outs, states


@pytest.mark.parametrize("alg,topo,world", [("tbq", "ring", 2), ("tbq", "ps", 3), ("onebit", "ring", 3),
                                            ("terngrad", "ps", 2), ("dgc", "ps", 2),
                                            ("graddrop", "ring", 2), ("dgc", "ring", 3)])
def test_host_schedule_matches_simulation(alg, topo, world):
    steps = 3
    res = _spawn(_run_optimizer, world, alg, topo, steps)
    ref, states = _simulate(world, alg, topo, steps)
    for r in range(world):
        for step in range(steps):
            for i in range(len(SHAPES)):
                got, want = res[r]["outs"][step][i], ref[step][i]
                assert torch.allclose(got, want, rtol=1e-6, atol=1e-9), (alg, topo, r, step, i)
        # every rank holds the same averaged gradient
        for step in range(steps):
            for i in range(len(SHAPES)):
                assert torch.equal(res[r]["outs"][step][i], res[0]["outs"][step][i])
    assert res[0]["stats"]["compressed_elems"] == 256 * 784 + 10 * 256


def test_config1_tbq_ring_tracks_uncompressed_allreduce():
    """10 steps: delivered + pending residual == exact average, and what was
    delivered is a sum of +-threshold levels divided by N."""
    world, steps = 2, 10
    res = _spawn(_run_optimizer, world, "tbq", "ring", steps)
    exact = [sum(_grads(r, s)[0] for r in range(world)) / world for s in range(steps)]
    delivered = sum(res[0]["outs"][s][0] for s in range(steps))
    pending = sum(res[r]["state"]["tensors"]["fc1.weight"]["residual"] for r in range(world)) / world
    total = sum(exact)
    assert torch.allclose(delivered.reshape(-1) + pending, total.reshape(-1), atol=1e-6)
    # small tensors are averaged exactly
    for s in range(steps):
        want = sum(_grads(r, s)[1] for r in range(world)) / world
        assert torch.allclose(res[0]["outs"][s][1], want, atol=1e-8)
    lv = (delivered / 0.005).round()
    assert torch.allclose(delivered, lv * 0.005, atol=1e-6)


def _run_uncompressed(rank, world, steps):
    import hipress_b200 as hp
    params = [torch.nn.Parameter(torch.zeros(s)) for s in SHAPES]
    opt = hp.DistributedOptimizer(torch.optim.SGD(params, lr=1.0), None, algorithm="none")
    outs = []
    for step in range(steps):
        for p, g in zip(params, _grads(rank, step)):
            p.grad = g.clone()
        opt.step()
        outs.append([p.detach().clone() for p in params])
    return outs


def test_uncompressed_path_is_exact_average():
    res = _spawn(_run_uncompressed, 2, 2)
    acc = [torch.zeros(s) for s in SHAPES]
    for step in range(2):
        for i in range(len(SHAPES)):
            acc[i] -= sum(_grads(r, step)[i] for r in range(2)) / 2
            assert torch.allclose(res[0][step][i], acc[i], atol=1e-7)
            assert torch.equal(res[0][step][i], res[1][step][i])


def _run_mismatch(rank, world):
    import hipress_b200 as hp
    shapes = SHAPES if rank == 0 else SHAPES[:-1]
    params = [torch.nn.Parameter(torch.zeros(s)) for s in shapes]
    try:
        hp.DistributedOptimizer(torch.optim.SGD(params, lr=1.0), None, algorithm="tbq")
        return "no error"
    except RuntimeError as e:
        return str(e)


def test_parameter_order_mismatch_is_detected():
    res = _spawn(_run_mismatch, 2)
    assert all("disagree" in r for r in res)


def _run_ddp_hook(rank, world):
    import hipress_b200 as hp
    from hipress_b200.parallel.hooks import FlatSyncer, ddp_comm_hook
    from torch.nn.parallel import DistributedDataParallel as DDP
    torch.manual_seed(0)
    model = torch.nn.Sequential(torch.nn.Linear(64, 256), torch.nn.ReLU(), torch.nn.Linear(256, 10))
    ddp = DDP(model)
    syncer = FlatSyncer(hp.HipressConfig(algorithm="tbq", topology="ring", comp_threshold=1024,
                                         threshold=0.001))
    ddp.register_comm_hook(syncer, ddp_comm_hook)
    g = torch.Generator().manual_seed(rank)
    for _ in range(2):
        ddp(torch.randn(16, 64, generator=g)).pow(2).mean().backward()
    grads = [p.grad.clone() for p in model.parameters()]
    res = sum(float(s[0]["residual"].abs().sum()) for s in syncer.state.values())
    return {"grads": grads, "resid": res}


def test_ddp_comm_hook_keeps_replicas_identical():
    res = _spawn(_run_ddp_hook, 2)
    for a, b in zip(res[0]["grads"], res[1]["grads"]):
        assert torch.equal(a, b)
    assert res[0]["resid"] > 0  # error feedback is active


# ----------------------------------------------------------------------------
def _run_overlapped_update(rank, world, overlap):
    import hipress_b200 as hp
    torch.manual_seed(0)
    model = torch.nn.Sequential(torch.nn.Linear(64, 96), torch.nn.ReLU(), torch.nn.Linear(96, 48),
                                torch.nn.ReLU(), torch.nn.Linear(48, 8))
    inner = torch.optim.SGD([{"params": model[0].parameters()},
                             {"params": list(model[2].parameters()) + list(model[4].parameters()),
                              "weight_decay": 1e-3}], lr=0.5, momentum=0.9)
    sched = torch.optim.lr_scheduler.StepLR(inner, step_size=2, gamma=0.5)
    opt = hp.DistributedOptimizer(inner, list(model.named_parameters()), algorithm="tbq",
                                  topology="ring", comp_threshold=1024, threshold=0.001,
                                  bucket_bytes=16 << 10, overlap_optimizer=overlap)
    g = torch.Generator().manual_seed(7 + rank)
    for step in range(5):
        x = torch.randn(16, 64, generator=g)
        opt.zero_grad()
        model(x).square().mean().backward()
        opt.step()
        sched.step()
    sd = opt.state_dict()["optimizer"]
    return {"params": [p.detach().clone() for p in model.parameters()],
            "momenta": [sd["state"][i]["momentum_buffer"].clone() for i in sorted(sd["state"])],
            "buckets": len(opt.engine.buckets)}


def test_overlapped_optimizer_step_matches_plain_step():
    """Stepping each bucket right behind its synchronisation gives the parameters,
    momenta and schedule of one step() after synchronize()."""
    plain = _spawn(_run_overlapped_update, 2, False)
    over = _spawn(_run_overlapped_update, 2, True)
    assert plain[0]["buckets"] > 1
    assert len(over[0]["momenta"]) == 6
    for a, b in zip(plain[0]["params"] + plain[0]["momenta"], over[0]["params"] + over[0]["momenta"]):
        assert torch.equal(a, b)
    for a, b in zip(over[0]["params"], over[1]["params"]):
        assert torch.equal(a, b)


# ----------------------------------------------------------------------------
def _run_two_machines(rank, world, alg, topo, per_machine, steps):
    """`world` gloo ranks posing as world/per_machine machines."""
    import os
    import hipress_b200 as hp
    if per_machine == 2 and world == 4:
        os.environ["HIPRESS_NODE_SIZE"] = "2"                 # the job-wide spelling
    else:
        os.environ["HIPRESS_NODE_ID"] = f"machine{rank // per_machine}"
    params = [torch.nn.Parameter(torch.zeros(s)) for s in SHAPES]
    names = ["fc1.weight", "fc1.bias", "fc2.weight", "fc2.bias"]
    opt = hp.DistributedOptimizer(torch.optim.SGD(params, lr=1.0), list(zip(names, params)),
                                  algorithm=alg, topology=topo, comp_threshold=1024,
                                  threshold=0.01, ratio=0.05)
    eng = opt.engine
    outs = []
    for step in range(steps):
        for p, g in zip(params, _grads(rank, step)):
            p.grad = g.clone()
        opt.synchronize()
        outs.append([p.grad.clone() for p in params])
        opt._synchronized = False
    sd = opt.state_dict()["compressor_state"]
    return {"outs": outs, "state": sd, "backend": eng.backend, "N": eng.N, "world": eng.world,
            "hier": eng.outer is not None and (eng.outer["nodes"], eng.outer["local"])}


@pytest.mark.parametrize("alg,topo", [("tbq", "ring"), ("onebit", "ps"), ("graddrop", "ps")])
def test_two_machines_of_two_ranks_synchronise_hierarchically(alg, topo):
    world, steps = 4, 6
    res = _spawn(_run_two_machines, world, alg, topo, 2, steps)
    assert all(r["hier"] == (2, 2) and r["N"] == 2 and r["world"] == 4 for r in res)
    for r in res[1:]:                                   # replicas stay identical
        for s in range(steps):
            for a, b in zip(r["outs"][s], res[0]["outs"][s]):
                assert torch.equal(a, b)
    for s in range(steps):                              # small tensors: exact mean over the job
        want = sum(_grads(r, s)[1] for r in range(world)) / world
        assert torch.allclose(res[0]["outs"][s][1], want, atol=1e-8)
    if alg == "tbq":
        # conservation: what was delivered plus what still waits in the residuals of
        # both levels is the exact mean (ring: no owner-side state)
        delivered = sum(res[0]["outs"][s][0] for s in range(steps)).reshape(-1)
        exact = sum(sum(_grads(r, s)[0] for r in range(world)) / world for s in range(steps)).reshape(-1)
        inner = sum(r["state"]["tensors"]["fc1.weight"]["residual"] for r in res) / world
        n = exact.numel()
        outer = torch.zeros(n)
        from hipress_b200.parallel.simulate import chunk_range
        for q, r in enumerate(res):
            lo, hi = chunk_range(n, 2, q % 2)
            outer[lo:hi] += r["state"]["between_machines"]["fc1.weight.0"]["residual"] / 2
        assert torch.allclose(delivered + inner + outer, exact, atol=1e-6)
        assert not torch.allclose(delivered, exact, atol=1e-4)      # it really was quantised


def test_one_rank_per_machine_uses_the_host_transport():
    res = _spawn(_run_two_machines, 2, "tbq", "ring", 1, 2)
    assert all(r["backend"] == "host" and not r["hier"] and r["N"] == 2 for r in res)
    plain = _spawn(_run_optimizer, 2, "tbq", "ring", 2)
    for s in range(2):
        for a, b in zip(res[0]["outs"][s], plain[0]["outs"][s]):
            assert torch.equal(a, b)


# ----------------------------------------------------------------------------
def _run_registered_algorithm(rank, world, topo, steps):
    """A DSL-generated TernGrad pair (4 bits) registered under a new name and used
    through the optimizer, with error feedback composed around it."""
    import hipress_b200 as hp
    from hipress_b200.compll import load_op
    enc, dec = load_op("TernGradEncode", "cpu"), load_op("TernGradDecode", "cpu")
    hp.register_algorithm("dsl_terngrad4", encode=enc, decode=dec, encode_args=(4,),
                          payload_bytes=lambda n: 10 + (n + 1) // 2, error_feedback=True)
    params = [torch.nn.Parameter(torch.zeros(s)) for s in SHAPES]
    names = ["fc1.weight", "fc1.bias", "fc2.weight", "fc2.bias"]
    opt = hp.DistributedOptimizer(torch.optim.SGD(params, lr=1.0), list(zip(names, params)),
                                  algorithm="dsl_terngrad4", topology=topo, comp_threshold=1024)
    outs = []
    for step in range(steps):
        for p, g in zip(params, _grads(rank, step)):
            p.grad = g.clone()
        opt.synchronize()
        outs.append([p.grad.clone() for p in params])
        opt._synchronized = False
    sd = opt.state_dict()["compressor_state"]
    return {"outs": outs, "backend": opt.engine.backend, "state": sd}


@pytest.mark.parametrize("topo", ["ring", "ps"])
def test_registered_dsl_algorithm_trains_through_the_runtime(topo):
    world, steps = 2, 5
    res = _spawn(_run_registered_algorithm, world, topo, steps)
    assert res[0]["backend"] == "host"
    for s in range(steps):
        for a, b in zip(res[0]["outs"][s], res[1]["outs"][s]):
            assert torch.equal(a, b)                        # replicas identical
        exact = sum(_grads(r, s)[0] for r in range(world)) / world
        got = res[0]["outs"][s][0]
        # 16 levels between min and max of ~N(0, 1e-3) data: close, but not exact
        assert (got - exact).abs().max().item() < 2e-3 and not torch.equal(got, exact)
        small = sum(_grads(r, s)[1] for r in range(world)) / world
        assert torch.allclose(res[0]["outs"][s][1], small, atol=1e-8)
    if topo == "ring":   # error feedback: delivered + pending residuals == exact mean
        delivered = sum(res[0]["outs"][s][0] for s in range(steps)).reshape(-1)
        exact = sum(sum(_grads(r, s)[0] for r in range(world)) / world for s in range(steps)).reshape(-1)
        pending = sum(r["state"]["tensors"]["fc1.weight"]["residual"] for r in res) / world
        assert torch.allclose(delivered + pending, exact, atol=1e-6)


def test_builtin_names_cannot_be_registered():
    import hipress_b200 as hp
    with pytest.raises(ValueError):
        hp.register_algorithm("tbq", encode=None, decode=None, payload_bytes=None)


def test_machines_of_different_sizes_fall_back_to_the_host_transport():
    res = _spawn(_run_two_machines, 3, "tbq", "ring", 2, 2)      # machines of 2 and 1 ranks
    assert all(r["backend"] == "host" and not r["hier"] and r["N"] == 3 for r in res)
    for s in range(2):
        for a, b in zip(res[0]["outs"][s], res[2]["outs"][s]):
            assert torch.equal(a, b)
