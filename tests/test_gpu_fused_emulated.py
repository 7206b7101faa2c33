"""Fused ring / PS kernels with all N ranks emulated by one cooperative launch on
one GPU, against the lock-step simulation built from CPU-oracle primitives."""
import pytest
import torch

from hipress_b200.ops import Compressor
from hipress_b200.parallel.fused import FusedDenseBucket, HipressTimeoutError
from hipress_b200.parallel.simulate import chunk_elems, simulate_ps, simulate_ring

pytestmark = pytest.mark.gpu

ALGS = [("tbq", {}), ("onebit", {}), ("terngrad", {"bitwidth": 2}), ("terngrad", {"bitwidth": 8})]


def _run(topology, name, kw, N, sizes, steps=2, ctas=8):
    torch.manual_seed(1234 + N)
    c = Compressor(name, **kw)
    ef = "residual" in c.spec.state_names()
    bucket = FusedDenseBucket(c.spec, topology, sizes, N, 0, ctas=ctas, emulate=True).bind_local("cuda")
    total = sum(sizes)
    G = torch.zeros(N, total, device="cuda")
    Rr = torch.zeros(N, total, device="cuda") if ef else None
    O = torch.zeros(N, total, device="cuda")
    chunks = [chunk_elems(s, N) for s in sizes]
    SR = torch.zeros(N, sum(chunks), device="cuda") if (ef and topology == "ps") else None
    offs = [sum(sizes[:i]) for i in range(len(sizes))]
    coffs = [sum(chunks[:i]) for i in range(len(sizes))]
    cpu_states = [[c.new_state(s, "cpu") for s in sizes] for _ in range(N)]
    cpu_sstates = [[({"residual": torch.zeros(ch)} if SR is not None else {}) for ch in chunks]
                   for _ in range(N)]
    for step in range(steps):
        Gc = torch.randn(N, total) * 0.02
        G.copy_(Gc)
        grads = [G[:, o:o + s] for o, s in zip(offs, sizes)]
        res = [Rr[:, o:o + s] for o, s in zip(offs, sizes)] if ef else None
        outs = [O[:, o:o + s] for o, s in zip(offs, sizes)]
        srs = [SR[:, o:o + ch] for o, ch in zip(coffs, chunks)] if SR is not None else None
        bucket.launch(grads, res, outs, srs, step=step, salt=0, tensor_ids=list(range(len(sizes))))
        torch.cuda.synchronize()
        bucket.check_status()
        for i, (o, s) in enumerate(zip(offs, sizes)):
            gl = [Gc[r, o:o + s].contiguous() for r in range(N)]
            sts = [cpu_states[r][i] for r in range(N)]
            if topology == "ring":
                ref = simulate_ring(c, gl, sts, step=step, tensor_id=i)
            else:
                ref = simulate_ps(c, gl, sts, [cpu_sstates[r][i] for r in range(N)], step=step,
                                  tensor_id=i)
            for r in range(N):
                got = O[r, o:o + s].cpu()
                assert torch.allclose(got, ref[r], rtol=1e-5, atol=1e-9), \
                    f"{topology} {name} N={N} step={step} tensor={i} rank={r}: " \
                    f"{(got - ref[r]).abs().max().item()}"
                assert torch.equal(O[r, o:o + s], O[0, o:o + s]), "ranks disagree"
                if ef:
                    assert torch.allclose(Rr[r, o:o + s].cpu(), sts[r]["residual"], rtol=1e-5, atol=1e-8)


@pytest.mark.parametrize("N", [1, 2, 4, 8])
@pytest.mark.parametrize("name,kw", ALGS)
def test_ring_emulated(name, kw, N):
    _run("ring", name, kw, N, [70001, 4096, 300, 1 << 17])


@pytest.mark.parametrize("N", [1, 2, 4, 8])
@pytest.mark.parametrize("name,kw", ALGS)
def test_ps_emulated(name, kw, N):
    _run("ps", name, kw, N, [70001, 4096, 300, 1 << 17])


@pytest.mark.parametrize("topology", ["ring", "ps"])
@pytest.mark.parametrize("N", [1, 2, 8])
@pytest.mark.parametrize("name,kw", ALGS[:3])
def test_emulated_aligned_tensors_use_bulk_prefetch(name, kw, N, topology):
    """Every tile is full and 16-byte aligned, so all loads go through the
    shared-memory prefetch pipeline (several tiles per CTA, across phases)."""
    _run(topology, name, kw, N, [1 << 19, 65536 + 4096 * 3, 8192 * N], steps=3, ctas=4)


def test_mean_of_many_steps_tracks_uncompressed_average():
    """Error feedback: over many steps the compressed ring delivers the same total."""
    torch.manual_seed(0)
    N, n = 4, 50000
    c = Compressor("tbq", threshold=0.01)
    b = FusedDenseBucket(c.spec, "ring", [n], N, 0, ctas=4, emulate=True).bind_local("cuda")
    G = torch.zeros(N, n, device="cuda")
    Rr = torch.zeros(N, n, device="cuda")
    O = torch.zeros(N, n, device="cuda")
    tot_ref = torch.zeros(n, device="cuda")
    tot = torch.zeros(n, device="cuda")
    for step in range(30):
        G.normal_(0, 0.004)
        tot_ref += G.mean(0)
        b.launch([G], [Rr], [O], step=step)
        tot += O[0]
    torch.cuda.synchronize()
    b.check_status()
    # what has not been delivered yet sits in the residuals
    pending = Rr.sum(0) / N
    assert torch.allclose(tot + pending, tot_ref, atol=2e-6)


def test_residency_guard():
    c = Compressor("tbq")
    b = FusedDenseBucket(c.spec, "ring", [1 << 24], 8, 0, ctas=4000, emulate=True).bind_local("cuda")
    G = torch.zeros(8, 1 << 24, device="cuda")
    from hipress_b200._native.lib import NativeLibraryError
    with pytest.raises(NativeLibraryError):
        b.launch([G], None, [G])


def test_device_side_trace_reports_phase_times():
    c = Compressor("tbq")
    n = 1 << 22
    b = FusedDenseBucket(c.spec, "ring", [n], 1, 0, ctas=128, trace=True).bind_local("cuda")
    g = torch.randn(n, device="cuda")
    r = torch.zeros(n, device="cuda")
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    b.launch([g], [r], [g])
    torch.cuda.synchronize()
    ev0.record()
    b.launch([g], [r], [g])
    ev1.record()
    torch.cuda.synchronize()
    enc_ms, total_ms = b.last_trace()[0]
    assert 0 < enc_ms <= total_ms
    # the stamps bracket the kernel itself: no longer than the event-timed launch
    assert total_ms <= ev0.elapsed_time(ev1) + 0.01
    assert int(b.trace[3]) == b.epoch


@pytest.mark.parametrize("topology", ["ring", "ps"])
def test_more_ctas_than_tiles_per_phase(topology):
    """Work items rotate over the grid from phase to phase: with more CTAs than a
    chunk has tiles, different hops run on different CTAs (and wait for one another
    across the emulated ranks) and the result is still the simulated one."""
    _run(topology, "tbq", {}, 4, [70001, 4096, 300, 1 << 17], steps=2, ctas=100)
    _run(topology, "onebit", {}, 2, [9000], steps=2, ctas=20)


def test_trace_splits_the_launch_into_phases():
    c = Compressor("tbq")
    N, n = 4, 1 << 20
    b = FusedDenseBucket(c.spec, "ring", [n], N, 0, ctas=32, emulate=True, trace=True).bind_local("cuda")
    G = torch.randn(N, n, device="cuda") * 0.02
    Rr = torch.zeros(N, n, device="cuda")
    b.launch([G], [Rr], [G])
    torch.cuda.synchronize()
    b.check_status()
    per_rank = b.last_trace_phases()
    assert len(per_rank) == N
    for phases, (enc_ms, total_ms) in zip(per_rank, b.last_trace()):
        assert len(phases) == 2 * N
        ends = [p["end_ms"] for p in phases]
        assert all(e > 0 for e in ends) and max(ends) <= total_ms + 1e-6
        assert ends[N - 1] <= enc_ms + 1e-6          # the hops end before the gathers do
        assert all(p["mean_poll_ms"] >= 0 for p in phases)


def test_fused_kernel_gives_up_cleanly_when_a_peer_never_sends():
    """Rank 0 of a two-rank ring whose peer does not exist: nothing ever fills the
    slots it polls.  Every wait is bounded, so the launch ends by itself; the status
    word names the wait; the sends of a CTA that gave up carry the mark that lets its
    receivers give up at once; and neither the gradient nor the error-feedback state
    of the chunks that needed the missing input is touched."""
    import time
    c = Compressor("tbq")
    n = 20000
    b = FusedDenseBucket(c.spec, "ring", [n], 2, 0, ctas=16, timeout_s=0.3)
    arena = torch.zeros(2 * b.region_bytes(), dtype=torch.uint8, device="cuda")
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    b.bind([arena.data_ptr(), arena.data_ptr() + b.region_bytes()], status)
    torch.manual_seed(5)
    g = torch.randn(n, device="cuda") * 0.02
    g0 = g.clone()
    r = torch.zeros(n, device="cuda")
    t0 = time.time()
    b.launch_ptrs([g.data_ptr()], [r.data_ptr()], [g.data_ptr()], [None])
    torch.cuda.synchronize()
    assert time.time() - t0 < 5.0
    with pytest.raises(HipressTimeoutError):
        b.check_status()
    ch = chunk_elems(n, 2)
    assert torch.equal(g, g0), "no averaged gradient is written from input that never arrived"
    assert bool((r[:ch] != 0).any()), "hop 0 needs no input: its error feedback is kept"
    assert bool((r[ch:] == 0).all()), "the hop that waited in vain leaves its state alone"
    # the context is still usable and the bucket works again once the status is cleared
    b1 = FusedDenseBucket(c.spec, "ring", [n], 1, 0, ctas=16).bind_local("cuda")
    b1.launch([g], [torch.zeros_like(g)], [g])
    torch.cuda.synchronize()
    b1.check_status()
