"""Fault injection on the host: corrupted, misrouted and missing messages among
CPU (gloo) ranks.  Nothing here touches a GPU."""
import pytest
import torch

from hipress_b200.ops import Compressor, PayloadError

SIZES = [5000, 3001]


def _spawn(fn, world, *args, **kw):
    from _mp import spawn
    return spawn(fn, world, *args, backend="gloo", **kw)


# ----------------------------------------------------------------- payload check
@pytest.mark.parametrize("alg", ["onebit", "tbq", "terngrad"])
def test_dense_payload_check_names_the_corrupted_field(alg):
    c = Compressor(alg)
    n = 10001
    g = torch.randn(n)
    pay = c.encode(g, c.new_state(n, "cpu"))
    c.check_payload(pay, n)
    for offset, what in [(0, "element count"), (4, "algorithm id"), (5, "bit width"),
                         (12, "tile size")]:
        bad = pay.clone()
        bad[offset] ^= 0x40
        with pytest.raises(PayloadError, match=what):
            c.check_payload(bad, n)
    with pytest.raises(PayloadError, match="shorter"):
        c.check_payload(pay[:-16], n)
    with pytest.raises(PayloadError, match="element count"):
        c.check_payload(pay, n + 1)           # a payload meant for another chunk
    other = Compressor("tbq" if alg != "tbq" else "onebit")
    with pytest.raises(PayloadError):
        other.check_payload(pay, n)


@pytest.mark.parametrize("alg", ["dgc", "graddrop"])
def test_sparse_payload_check_catches_bad_counts_and_indices(alg):
    c = Compressor(alg, ratio=0.01)
    n = 20000
    pay = c.encode(torch.randn(n), c.new_state(n, "cpu"))
    kmax = c.kmax(n)
    c.check_payload(pay, n)
    bad = pay.clone()
    bad[12:16] = torch.tensor([kmax + 1], dtype=torch.int32).view(torch.uint8)
    with pytest.raises(PayloadError, match="pair count"):
        c.check_payload(bad, n)
    bad = pay.clone()
    bad[16:20] = torch.tensor([n], dtype=torch.int32).view(torch.uint8)   # first index = n
    with pytest.raises(PayloadError, match="index out of range"):
        c.check_payload(bad, n)
    with pytest.raises(PayloadError, match="shorter"):
        c.check_payload(pay[:-8], n)
    # the decoder itself refuses the same faults instead of writing out of bounds
    out = torch.zeros(n)
    from hipress_b200._native.lib import NativeLibraryError
    with pytest.raises(NativeLibraryError):
        c.decode(bad, out)


# -------------------------------------------------- faults on the wire (gloo ranks)
def _run_with_fault(rank, world, alg, topo, fault):
    from hipress_b200.parallel.host_schedule import HostSchedule, SegView
    comp = Compressor(alg, ratio=0.01)
    sched = HostSchedule(comp, topo)
    torch.manual_seed(rank)
    segs = []
    for i, n in enumerate(SIZES):
        from hipress_b200.parallel.simulate import chunk_elems
        st = comp.new_state(n, "cpu")
        sst = {"residual": torch.zeros(chunk_elems(n, world))} if topo == "ps" else {}
        segs.append(SegView(torch.randn(n) * 0.05, st, sst, i))
    before = [s.g.clone() for s in segs]
    import torch.distributed as dist
    real_batch = dist.batch_isend_irecv
    if rank == 1 and fault == "flip-header":
        if topo == "ring":
            exchange = sched._exchange

            def faulty(send, dst, recv, src):
                exchange(send, dst, recv, src)
                recv[4] ^= 0x7                    # algorithm id of the first payload

            sched._exchange = faulty
        else:
            def damaged(ops):
                works = real_batch(ops)

                class AfterArrival:
                    def wait(self):
                        for w in works:
                            w.wait()
                        sched._bufs[("i", 0)][4] ^= 0x7   # rank 0's push, once it has arrived

                return [AfterArrival()]

            dist.batch_isend_irecv = damaged
    try:
        sched.sync(segs, step=0)
        return ("ok", [torch.equal(a, b.g) for a, b in zip(before, segs)])
    except PayloadError as e:
        return ("payload-error", str(e), [torch.equal(a, b.g) for a, b in zip(before, segs)])
    except RuntimeError as e:   # the peer that found the fault left: its connection closes
        return ("peer-left", str(e)[:200])
    finally:
        dist.batch_isend_irecv = real_batch


@pytest.mark.parametrize("alg,topo", [("tbq", "ring"), ("dgc", "ring"), ("onebit", "ps")])
def test_corrupted_message_is_detected_before_it_reaches_the_gradients(alg, topo):
    res = _spawn(_run_with_fault, 2, alg, topo, "flip-header")
    kind, msg = res[1][:2]
    assert kind == "payload-error", res[1]
    assert "rank 1" in msg and "algorithm id" in msg
    assert ("ring hop 1 from rank 0" in msg) if topo == "ring" else ("PS push from rank 0" in msg)
    assert res[0][0] in ("peer-left", "ok")       # the healthy rank ends with an error or had finished
    clean = _spawn(_run_with_fault, 2, alg, topo, "none")
    assert clean[0][0] == clean[1][0] == "ok"


def _run_missing_rank(rank, world):
    """Rank 1 never joins the step; rank 0's exchange ends with an error inside the
    process group's (short) timeout instead of waiting for ever."""
    import time
    from hipress_b200.parallel.host_schedule import HostSchedule, SegView
    comp = Compressor("tbq")
    sched = HostSchedule(comp, "ring")
    seg = SegView(torch.randn(4096) * 0.05, comp.new_state(4096, "cpu"), {}, 0)
    if rank == 1:
        time.sleep(4.0)
        return "absent"
    t0 = time.time()
    try:
        sched.sync([seg], step=0)
        return "completed"
    except Exception as e:  # gloo reports a timeout or a closed connection
        return ("error", type(e).__name__, round(time.time() - t0, 1))


def test_a_rank_that_never_joins_ends_the_exchange_with_an_error():
    res = _spawn(_run_missing_rank, 2, env={"HIPRESS_PG_TIMEOUT_S": "2"})
    assert res[1] == "absent"
    assert res[0][0] == "error" and res[0][2] < 4.0, res[0]
