"""Fused sparse parameter-server kernels (DGC / GradDrop) with the N ranks played
phase by phase on one GPU, against the lock-step simulation on the CPU oracle."""
import pytest
import torch

from hipress_b200.ops import Compressor
from hipress_b200.parallel.fused_sparse import FusedSparseBucket
from hipress_b200.parallel.simulate import chunk_elems, simulate_ps, simulate_ring

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("N", [1, 2, 4, 8])
@pytest.mark.parametrize("name", ["dgc", "graddrop"])
def test_sparse_ps_emulated(name, N):
    torch.manual_seed(99 + N)
    sizes = [200003, 8192, 300, 1 << 18]
    c = Compressor(name, ratio=0.01)
    b = FusedSparseBucket(c.spec, sizes, N, 0, ctas=8, emulate=True).bind_local("cuda")
    total = sum(sizes)
    chunks = [chunk_elems(s, N) for s in sizes]
    offs = [sum(sizes[:i]) for i in range(len(sizes))]
    coffs = [sum(chunks[:i]) for i in range(len(sizes))]
    G = torch.zeros(N, total, device="cuda")
    A = torch.zeros(N, total, device="cuda")
    U = torch.zeros(N, total, device="cuda") if name == "dgc" else None
    O = torch.zeros(N, total, device="cuda")
    SR = torch.zeros(N, sum(chunks), device="cuda")
    cpu_states = [[c.new_state(s, "cpu") for s in sizes] for _ in range(N)]
    cpu_server = [[{"residual": torch.zeros(ch)} for ch in chunks] for _ in range(N)]
    for step in range(3):
        Gc = torch.randn(N, total)
        G.copy_(Gc)
        b.launch_ptrs([G[0, o:].data_ptr() for o in offs], [A[0, o:].data_ptr() for o in offs],
                      [U[0, o:].data_ptr() for o in offs] if U is not None else None,
                      [O[0, o:].data_ptr() for o in offs], [SR[0, o:].data_ptr() for o in coffs],
                      strides=(total, total, total, sum(chunks)))
        torch.cuda.synchronize()
        b.check_status()
        for i, (o, s) in enumerate(zip(offs, sizes)):
            gl = [Gc[r, o:o + s].contiguous() for r in range(N)]
            ref = simulate_ps(c, gl, [cpu_states[r][i] for r in range(N)],
                              [cpu_server[r][i] for r in range(N)])
            for r in range(N):
                got = O[r, o:o + s].cpu()
                assert torch.allclose(got, ref[r], rtol=1e-5, atol=1e-7), (name, N, step, i, r,
                                                                          (got - ref[r]).abs().max())
                assert torch.equal(O[r, o:o + s], O[0, o:o + s])
                acc_name = "accum_v" if name == "dgc" else "residual"
                assert torch.allclose(A[r, o:o + s].cpu(), cpu_states[r][i][acc_name], rtol=1e-5,
                                      atol=1e-7)
            ch = chunks[i]
            for r in range(N):
                assert torch.allclose(SR[r, coffs[i]:coffs[i] + ch].cpu(), cpu_server[r][i]["residual"],
                                      rtol=1e-5, atol=1e-7)
        assert (O[0] != 0).sum().item() > 0


@pytest.mark.parametrize("N", [1, 2, 3, 8])
@pytest.mark.parametrize("name", ["dgc", "graddrop"])
def test_sparse_ring_emulated(name, N):
    torch.manual_seed(7 + N)
    sizes = [150001, 8192, 300, 1 << 17]
    c = Compressor(name, ratio=0.01)
    b = FusedSparseBucket(c.spec, sizes, N, 0, ctas=8, emulate=True, topology="ring").bind_local("cuda")
    total = sum(sizes)
    offs = [sum(sizes[:i]) for i in range(len(sizes))]
    G = torch.zeros(N, total, device="cuda")
    A = torch.zeros(N, total, device="cuda")
    U = torch.zeros(N, total, device="cuda") if name == "dgc" else None
    O = torch.zeros(N, total, device="cuda")
    cpu_states = [[c.new_state(s, "cpu") for s in sizes] for _ in range(N)]
    acc_name = "accum_v" if name == "dgc" else "residual"
    for step in range(3):
        Gc = torch.randn(N, total)
        G.copy_(Gc)
        b.launch_ptrs([G[0, o:].data_ptr() for o in offs], [A[0, o:].data_ptr() for o in offs],
                      [U[0, o:].data_ptr() for o in offs] if U is not None else None,
                      [O[0, o:].data_ptr() for o in offs], [None] * len(sizes),
                      strides=(total, total, total, 0))
        torch.cuda.synchronize()
        b.check_status()
        for i, (o, s) in enumerate(zip(offs, sizes)):
            gl = [Gc[r, o:o + s].contiguous() for r in range(N)]
            ref = simulate_ring(c, gl, [cpu_states[r][i] for r in range(N)])
            for r in range(N):
                got = O[r, o:o + s].cpu()
                assert torch.allclose(got, ref[r], rtol=1e-5, atol=1e-7), (name, N, step, i, r)
                assert torch.equal(O[r, o:o + s], O[0, o:o + s])
                assert torch.allclose(A[r, o:o + s].cpu(), cpu_states[r][i][acc_name], rtol=1e-5, atol=1e-7)


def test_sparse_ps_through_the_optimizer_single_rank():
    import hipress_b200 as hp
    torch.manual_seed(3)
    p = torch.nn.Parameter(torch.zeros(100000, device="cuda"))
    opt = hp.DistributedOptimizer(torch.optim.SGD([p], lr=1.0), [("w", p)], algorithm="dgc",
                                  topology="ps", comp_threshold=1024, ratio=0.01)
    assert opt.engine.backend == "fused" and opt.engine.buckets[0].impl is not None
    g = torch.randn(100000, device="cuda")
    p.grad = g.clone()
    opt.step()
    torch.cuda.synchronize()
    opt.engine.check()
    sent = (p.detach() != 0)
    assert sent.sum().item() == 1000
    top = torch.topk(g.abs(), 1000).indices
    assert sent[top].all()
    assert torch.allclose(-p.detach()[top], g[top])
    opt.close()


def test_timeline_and_sm_partition_paths(tmp_path, monkeypatch):
    """Chrome-trace timeline of bucket launches, and the green-context stream that
    confines fused kernels to a few SMs (off by default): both paths run a step."""
    import json
    import hipress_b200 as hp
    trace = tmp_path / "timeline.json"
    monkeypatch.setenv("HIPRESS_TIMELINE", str(trace))
    torch.manual_seed(1)
    ps = [torch.nn.Parameter(torch.zeros(n, device="cuda")) for n in (300000, 70000, 500000, 10)]
    named = [(f"p{i}", p) for i, p in enumerate(ps)]
    opt = hp.DistributedOptimizer(torch.optim.SGD(ps, lr=1.0), named, algorithm="tbq", topology="ring",
                                  comp_threshold=1024, bucket_bytes=1 << 21, partition_sms=16,
                                  partition_ctas=32)
    eng = opt.engine
    assert sum(b.fused for b in eng.buckets) >= 2
    for step in range(2):
        for p in ps:
            p.grad = torch.full_like(p, 0.025)
        opt.step()
    torch.cuda.synchronize()
    eng.check()
    # two steps of 0.025 with threshold 0.01: 0.01 then 0.01 sent (residual 0.03 left)
    assert torch.allclose(ps[0].detach(), torch.full_like(ps[0], -0.02))
    assert torch.allclose(ps[3].detach(), torch.full_like(ps[3], -0.05))
    opt.close()
    events = json.loads(trace.read_text())["traceEvents"]
    assert len(events) >= 4 and all(e["dur"] >= 0 for e in events)


def test_overlapped_optimizer_step_on_the_communication_stream():
    """overlap_optimizer updates each bucket behind its fused kernel, during backward;
    parameters and momenta equal those of a single step() after synchronize()."""
    import hipress_b200 as hp

    def run(overlap):
        torch.manual_seed(0)
        model = torch.nn.Sequential(torch.nn.Linear(512, 1024), torch.nn.ReLU(),
                                    torch.nn.Linear(1024, 768), torch.nn.ReLU(),
                                    torch.nn.Linear(768, 16)).cuda()
        inner = torch.optim.SGD(model.parameters(), lr=0.1, momentum=0.9, fused=True)
        opt = hp.DistributedOptimizer(inner, list(model.named_parameters()), algorithm="tbq",
                                      topology="ring", comp_threshold=1024, threshold=1e-4,
                                      bucket_bytes=3 << 20, overlap_optimizer=overlap)
        assert opt.engine.backend == "fused" and sum(b.fused for b in opt.engine.buckets) >= 2
        gen = torch.Generator(device="cuda").manual_seed(5)
        for _ in range(4):
            x = torch.randn(64, 512, device="cuda", generator=gen)
            opt.zero_grad()
            model(x).square().mean().backward()
            opt.step()
        torch.cuda.synchronize()
        opt.engine.check()
        sd = inner.state_dict()["state"]
        out = [p.detach().clone() for p in model.parameters()] + \
              [sd[i]["momentum_buffer"].clone() for i in sorted(sd)]
        opt.close()
        return out

    plain, over = run(False), run(True)
    assert len(plain) == len(over) == 12
    for a, b in zip(plain, over):
        assert torch.equal(a, b)


@pytest.mark.parametrize("topology", ["ps", "ring"])
def test_sparse_auto_grid_and_heavy_ties(topology):
    """Grid sized from the bucket (ctas=0) and a gradient made of few distinct
    magnitudes, so the candidate list of the threshold bin overflows and the
    full-array passes (the extra, conditional phases of the launch) decide."""
    torch.manual_seed(21)
    N, n = 2, 600000
    c = Compressor("graddrop", ratio=0.01)
    b = FusedSparseBucket(c.spec, [n], N, 0, ctas=0, emulate=True, topology=topology).bind_local("cuda")
    G = (torch.randint(0, 3, (N, n)).float() - 1.0).cuda()        # values -1, 0, +1: massive ties
    A = torch.zeros(N, n, device="cuda")
    O = torch.zeros(N, n, device="cuda")
    SR = torch.zeros(N, chunk_elems(n, N), device="cuda")
    b.launch_ptrs([G.data_ptr()], [A.data_ptr()], None, [O.data_ptr()],
                  [SR.data_ptr() if topology == "ps" else None], strides=(n, n, n, SR.shape[1]))
    torch.cuda.synchronize()
    b.check_status()
    assert torch.equal(O[0], O[1])
    k = c.kmax(chunk_elems(n, N))
    sent = int((O[0] != 0).sum())
    assert 0 < sent <= 2 * k
    # conservation: what was delivered plus what every rank (and owner) kept is the input
    kept = A.sum(0)
    if topology == "ps":
        kept[:SR.shape[1]] += SR[0][:min(n, SR.shape[1])]
        kept[SR.shape[1]:] += SR[1][:n - SR.shape[1]]
    assert torch.allclose(O[0] * N + kept, G.sum(0), atol=1e-5)


def test_sparse_kernel_gives_up_cleanly_when_a_peer_never_sends():
    """Rank 0 of a two-rank job whose peer does not exist: the flag it waits for is
    never set.  The waits and the phase barriers are bounded, the launch ends by
    itself and the status word names the wait."""
    import time
    from hipress_b200.parallel.fused import HipressTimeoutError
    c = Compressor("graddrop", ratio=0.01)
    n = 50000
    b = FusedSparseBucket(c.spec, [n], 2, 0, ctas=8, timeout_s=0.3, topology="ps")
    arena = torch.zeros(2 * b.region_bytes(), dtype=torch.uint8, device="cuda")
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    b.bind([arena.data_ptr(), arena.data_ptr() + b.region_bytes()], status, "cuda")
    g = torch.randn(n, device="cuda")
    a = torch.zeros(n, device="cuda")
    out = torch.full((n,), 5.0, device="cuda")
    sr = torch.zeros(chunk_elems(n, 2), device="cuda")
    t0 = time.time()
    b.launch_ptrs([g.data_ptr()], [a.data_ptr()], None, [out.data_ptr()], [sr.data_ptr()])
    torch.cuda.synchronize()
    assert time.time() - t0 < 10.0
    with pytest.raises(HipressTimeoutError):
        b.check_status()
    # still usable afterwards
    b1 = FusedSparseBucket(c.spec, [n], 1, 0, ctas=8).bind_local("cuda")
    b1.launch_ptrs([g.data_ptr()], [torch.zeros_like(g).data_ptr()], None, [out.data_ptr()],
                   [torch.zeros(chunk_elems(n, 1), device="cuda").data_ptr()])
    torch.cuda.synchronize()
    b1.check_status()
