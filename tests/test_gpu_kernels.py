"""CUDA kernels against the CPU oracle (plain fp32 restatement of the same op)."""
import pytest
import torch

from hipress_b200.ops import Compressor, sparse_pairs

pytestmark = pytest.mark.gpu

SIZES = [1, 7, 4095, 4096, 4097, 70001, 1 << 20]
DENSE = [("tbq", {}), ("onebit", {}), ("terngrad", {"bitwidth": 1}), ("terngrad", {"bitwidth": 2}),
         ("terngrad", {"bitwidth": 4}), ("terngrad", {"bitwidth": 8})]


def _meta_region(c, n):
    nt = (n + 4095) // 4096
    mf = {1: 1, 2: 0, 3: 2}[c.spec.alg]
    return 16, 16 + (nt * mf * 4 + 15) // 16 * 16


@pytest.mark.parametrize("n", SIZES)
@pytest.mark.parametrize("name,kw", DENSE)
def test_dense_encode_matches_oracle(name, kw, n):
    torch.manual_seed(n)
    c = Compressor(name, **kw)
    g = torch.randn(n) * 0.02
    r0 = torch.randn(n) * 0.005
    st_c, st_g = c.new_state(n, "cpu"), c.new_state(n, "cuda")
    if "residual" in st_c:
        st_c["residual"].copy_(r0)
        st_g["residual"].copy_(r0)
    pc = c.encode(g, st_c, step=7, salt=3, tensor_id=5)
    pg = c.encode(g.cuda(), st_g, step=7, salt=3, tensor_id=5)
    torch.cuda.synchronize()
    lo, hi = _meta_region(c, n)
    pgc = pg.cpu()
    # codes and header are bit exact; per-tile scales agree to the last bits
    assert torch.equal(pgc[:lo], pc[:lo])
    assert torch.equal(pgc[hi:], pc[hi:]), "packed codes differ"
    mg, mc = pgc[lo:hi].view(torch.float32), pc[lo:hi].view(torch.float32)
    assert torch.allclose(mg, mc, rtol=1e-6, atol=0)
    if "residual" in st_c:
        assert torch.allclose(st_g["residual"].cpu(), st_c["residual"], atol=1e-8, rtol=1e-5)
    # decode and decode-accumulate
    out_c, out_g = torch.empty(n), torch.empty(n, device="cuda")
    c.decode(pc, out_c, scale=0.25)
    c.decode(pg, out_g, scale=0.25)
    assert torch.allclose(out_g.cpu(), out_c, rtol=1e-6, atol=0)
    base = torch.randn(n)
    acc_c, acc_g = base.clone(), base.cuda()
    c.decode(pc, acc_c, accumulate=True)
    c.decode(pg, acc_g, accumulate=True)
    assert torch.allclose(acc_g.cpu(), acc_c, rtol=1e-6, atol=1e-9)


@pytest.mark.parametrize("name,kw", DENSE)
def test_dense_merge_incoming(name, kw):
    torch.manual_seed(11)
    c = Compressor(name, **kw)
    n = 50000
    g0, g1 = torch.randn(n) * 0.02, torch.randn(n) * 0.02
    p0 = c.encode(g0, c.new_state(n, "cpu"))
    st_c, st_g = c.new_state(n, "cpu"), c.new_state(n, "cuda")
    pc = c.encode(g1, st_c, incoming=p0, elem_offset=8192)
    pg = c.encode(g1.cuda(), st_g, incoming=p0.cuda(), elem_offset=8192)
    lo, hi = _meta_region(c, n)
    assert torch.equal(pg.cpu()[hi:], pc[hi:])


def test_unaligned_views():
    c = Compressor("tbq")
    base = torch.randn(10001) * 0.02
    g = base[1:]  # 4-byte aligned only
    st_c, st_g = c.new_state(10000, "cpu"), c.new_state(10000, "cuda")
    pc = c.encode(g.contiguous(), st_c)
    gg = base.cuda()[1:]
    pg = c.encode(gg, st_g)
    assert torch.equal(pg.cpu(), pc)
    out = torch.zeros(10001, device="cuda")
    c.decode(pg, out[1:])
    ref = torch.empty(10000)
    c.decode(pc, ref)
    assert torch.equal(out[1:].cpu(), ref) and out[0].item() == 0


@pytest.mark.parametrize("name", ["dgc", "graddrop"])
@pytest.mark.parametrize("n", [1, 10, 4097, 100003, 3_000_001])
def test_sparse_encode_matches_oracle(name, n):
    torch.manual_seed(n)
    c = Compressor(name, ratio=0.001 if n > 10000 else 0.05)
    g = torch.randn(n)
    v0 = torch.randn(n) * 0.3
    st_c, st_g = c.new_state(n, "cpu"), c.new_state(n, "cuda")
    for st in (st_c, st_g):
        for k_ in st:
            st[k_].copy_(v0 if k_ != "momentum_u" else v0 * 0.5)
    pc = c.encode(g, st_c)
    pg = c.encode(g.cuda(), st_g)
    torch.cuda.synchronize()
    k = c.kmax(n)
    ic, vc = sparse_pairs(pc, k)
    ig, vg = sparse_pairs(pg, k)
    assert torch.equal(ig, ic)
    assert torch.equal(vg, vc)
    for k_ in st_c:
        assert torch.equal(st_g[k_].cpu(), st_c[k_]), k_
    assert pg.cpu()[8:12].view(torch.float32).item() == pc[8:12].view(torch.float32).item()
    out_c, out_g = torch.ones(n), torch.ones(n, device="cuda")
    c.decode(pc, out_c, scale=0.5)
    c.decode(pg, out_g, scale=0.5)
    assert torch.equal(out_g.cpu(), out_c)
    c.decode(pc, out_c, scale=2.0, accumulate=True)
    c.decode(pg, out_g, scale=2.0, accumulate=True)
    assert torch.equal(out_g.cpu(), out_c)


def test_sparse_degenerate_inputs():
    c = Compressor("graddrop", ratio=0.01)
    n = 100000
    # all zeros: nothing is sent
    st = c.new_state(n, "cuda")
    p = c.encode(torch.zeros(n, device="cuda"), st)
    assert sparse_pairs(p, c.kmax(n))[0].numel() == 0
    # many equal magnitudes: exactly k are sent, all of them valid choices
    g = torch.ones(n, device="cuda")
    g[::2] = -1.0
    st = c.new_state(n, "cuda")
    p = c.encode(g, st)
    idx, val = sparse_pairs(p, c.kmax(n))
    assert idx.numel() == c.kmax(n) and idx.unique().numel() == idx.numel()
    assert torch.all(val.abs() == 1.0)
    assert int((st["residual"] == 0).sum()) == c.kmax(n)
    # select-only mode on a prepared accumulator
    acc = torch.randn(n, device="cuda")
    ref = torch.topk(acc.abs().cpu(), c.kmax(n)).indices.sort().values
    p = c.encode(acc, {"residual": acc}, update=False)
    assert torch.equal(sparse_pairs(p, c.kmax(n))[0], ref)


def test_bounded_wait_reports_and_returns():
    """A wait on a flag nobody sets must end with a status word, not a hang."""
    import time
    from hipress_b200._native import lib
    L = lib.cuda()
    flag = torch.zeros(4, dtype=torch.int32, device="cuda")
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    t0 = time.time()
    lib.check(L.hp_cuda_wait_probe(flag.data_ptr(), 5, int(0.2e9), status.data_ptr(), lib.stream_ptr()))
    torch.cuda.synchronize()
    dt = time.time() - t0
    w = status[0].item() & 0xFFFFFFFF
    assert w == (lib.STATUS_TIMEOUT | (7 << 16))
    assert 0.15 < dt < 1.5  # one timeout, the second wait returns at once
    # when the flag is set the wait passes and reports nothing
    status.zero_()
    lib.check(L.hp_cuda_set_flag(flag.data_ptr(), 5, lib.stream_ptr()))
    lib.check(L.hp_cuda_wait_probe(flag.data_ptr(), 5, int(0.2e9), status.data_ptr(), lib.stream_ptr()))
    torch.cuda.synchronize()
    assert status[0].item() == 0
    # the context is still usable
    assert torch.ones(8, device="cuda").sum().item() == 8


def test_arena_guard_words_detect_an_overrun():
    from hipress_b200.parallel.symm import SymmetricArena
    import hipress_b200 as hp
    hp.init()
    arena = SymmetricArena(1 << 16)
    a = arena.carve(1000)[0]
    b = arena.carve(512)[0]
    assert b - a == 1024 + SymmetricArena.GUARD_BYTES
    arena.check_guards()
    # a writer that runs past its region (here: 8 bytes into the guard of region 0)
    over = arena._view(1024, 2)
    over.fill_(7)
    with pytest.raises(RuntimeError, match="regions \\[0\\]"):
        arena.check_guards()
    arena.close()
