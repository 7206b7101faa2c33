"""CUDA kernels against a plain PyTorch fp32 restatement of each algorithm.

The other GPU tests compare the kernels with the C++ oracle, which includes the same
header of per-element formulas as the kernels do; a wrong formula there would pass
them all.  Nothing in this file touches the native math: the algorithms are restated
from their definitions (onebit: sign + mean |x| per 4096-element tile; TBQ: +-tau
threshold codes with error feedback; TernGrad: 2^b levels between the tile's min and
max; DGC: momentum correction + exact top-k), the payload is unpacked with tensor
ops, and the CUDA outputs are held against that.
"""
import math

import pytest
import torch

from hipress_b200.ops import Compressor, sparse_pairs

pytestmark = pytest.mark.gpu

TILE = 4096
SIZES = [1, 7, 4095, 4096, 4097, 70001, 1 << 20]


def _tiles(n):
    return (n + TILE - 1) // TILE


def _split(payload: torch.Tensor, n: int, meta_floats: int):
    """(header bytes, per-tile metadata [tiles, meta_floats], code bytes) of a dense payload."""
    p = payload.cpu()
    nt = _tiles(n)
    mb = (nt * meta_floats * 4 + 15) // 16 * 16
    meta = p[16:16 + nt * meta_floats * 4].view(torch.float32).view(nt, meta_floats) if meta_floats \
        else torch.empty(nt, 0)
    return p[:16], meta, p[16 + mb:]


def _unpack(codes: torch.Tensor, n: int, bits: int) -> torch.Tensor:
    """Element i of tile t sits at bit i*bits (LSB first) of the tile's code region,
    which starts at byte t * 4096 * bits / 8."""
    out = torch.empty(n, dtype=torch.int64)
    per = 8 // bits
    for t in range(_tiles(n)):
        m = min(TILE, n - t * TILE)
        reg = codes[t * TILE * bits // 8: t * TILE * bits // 8 + (m * bits + 7) // 8].to(torch.int64)
        i = torch.arange(m)
        out[t * TILE: t * TILE + m] = (reg[i // per] >> ((i % per) * bits)) & ((1 << bits) - 1)
    return out


@pytest.mark.parametrize("n", SIZES)
def test_tbq_against_definition(n):
    torch.manual_seed(100 + n)
    tau = 0.01
    c = Compressor("tbq", threshold=tau)
    g, r0 = torch.randn(n) * 0.02, torch.randn(n) * 0.005
    st = c.new_state(n, "cuda")
    st["residual"].copy_(r0)
    p = c.encode(g.cuda(), st)
    torch.cuda.synchronize()
    x = g + r0
    code = torch.where(x >= tau, 3, torch.where(x <= -tau, 2, 0))
    value = torch.where(code == 3, tau, torch.where(code == 2, -tau, 0.0)).float()
    _, _, cb = _split(p, n, 0)
    assert torch.equal(_unpack(cb, n, 2), code), "TBQ codes"
    assert torch.equal(st["residual"].cpu(), x - value), "error feedback: r' = x - Q(x)"
    out = torch.full((n,), 7.0, device="cuda")
    c.decode(p, out, scale=0.5)
    assert torch.equal(out.cpu(), value * 0.5)
    # the invariant of error feedback: what was sent plus what was kept is the input
    full = torch.empty(n, device="cuda")
    c.decode(p, full)
    assert torch.allclose(full.cpu() + st["residual"].cpu(), x, atol=1e-8, rtol=0)


@pytest.mark.parametrize("n", SIZES)
def test_onebit_against_definition(n):
    torch.manual_seed(200 + n)
    c = Compressor("onebit")
    g, r0 = torch.randn(n) * 0.02, torch.randn(n) * 0.005
    st = c.new_state(n, "cuda")
    st["residual"].copy_(r0)
    p = c.encode(g.cuda(), st)
    torch.cuda.synchronize()
    x = g + r0
    _, meta, cb = _split(p, n, 1)
    bit = _unpack(cb, n, 1)
    assert torch.equal(bit, (x < 0).to(torch.int64)), "sign bits"
    scale = torch.stack([x[t * TILE:(t + 1) * TILE].abs().double().mean().float()
                         for t in range(_tiles(n))])
    assert torch.allclose(meta[:, 0], scale, rtol=1e-6, atol=0), "per-tile scale = mean |x|"
    value = torch.where(bit == 1, -1.0, 1.0) * meta[:, 0].repeat_interleave(TILE)[:n]
    assert torch.allclose(st["residual"].cpu(), x - value, rtol=1e-6, atol=1e-9)
    out = torch.empty(n, device="cuda")
    c.decode(p, out)
    assert torch.equal(out.cpu(), value)


@pytest.mark.parametrize("bits", [1, 2, 4, 8])
@pytest.mark.parametrize("n", [7, 4096, 70001, 1 << 20])
def test_terngrad_against_definition(n, bits):
    torch.manual_seed(300 + n + bits)
    c = Compressor("terngrad", bitwidth=bits)
    g = torch.randn(n) * 0.02
    p = c.encode(g.cuda(), c.new_state(n, "cuda"), step=3, tensor_id=2)
    torch.cuda.synchronize()
    _, meta, cb = _split(p, n, 2)
    q = _unpack(cb, n, bits)
    levels = (1 << bits) - 1
    mn = torch.stack([g[t * TILE:(t + 1) * TILE].min() for t in range(_tiles(n))])
    mx = torch.stack([g[t * TILE:(t + 1) * TILE].max() for t in range(_tiles(n))])
    assert torch.equal(meta[:, 0], mn) and torch.equal(meta[:, 1], mx), "tile min / max"
    gap = ((mx - mn) / levels).repeat_interleave(TILE)[:n]
    lo = mn.repeat_interleave(TILE)[:n]
    assert int(q.min()) >= 0 and int(q.max()) <= levels
    value = q.float() * gap + lo
    # stochastic rounding picks one of the two levels around the element ...
    assert bool(((value - g).abs() <= gap * 1.0001 + 1e-12).all()), "level placement"
    # ... and is unbiased: the mean error over many elements is far below one step
    if n >= 70001:
        assert abs(float((value - g).mean())) < 0.02 * float(gap.mean())
        up = (value > g).float().mean().item()
        assert 0.3 < up < 0.7, "rounds up about as often as down"
    out = torch.empty(n, device="cuda")
    c.decode(p, out)
    assert torch.allclose(out.cpu(), value, rtol=1e-6, atol=3e-8), "decode = q * gap + min"


@pytest.mark.parametrize("n", [4097, 100003, 3_000_001])
def test_dgc_against_definition(n):
    torch.manual_seed(400 + n)
    ratio, m = 0.001 if n > 10000 else 0.05, 0.9
    c = Compressor("dgc", ratio=ratio, momentum=m)
    g, u0, v0 = torch.randn(n), torch.randn(n) * 0.15, torch.randn(n) * 0.3
    st = c.new_state(n, "cuda")
    st["momentum_u"].copy_(u0)
    st["accum_v"].copy_(v0)
    p = c.encode(g.cuda(), st)
    torch.cuda.synchronize()
    u = m * u0 + g
    v = v0 + u
    k = math.ceil(ratio * n)
    assert c.kmax(n) == k
    top = torch.topk(v.abs(), k).indices.sort().values
    idx, val = sparse_pairs(p, k)
    assert torch.equal(idx, top), "the k largest |v| are sent"
    assert torch.allclose(val, v[top], rtol=1e-6, atol=1e-6)
    keep = torch.ones(n, dtype=torch.bool)
    keep[top] = False
    gu, gv = st["momentum_u"].cpu(), st["accum_v"].cpu()
    assert torch.allclose(gv[keep], v[keep], rtol=1e-6, atol=1e-6) and bool((gv[top] == 0).all())
    assert torch.allclose(gu[keep], u[keep], rtol=1e-6, atol=1e-6) and bool((gu[top] == 0).all())
    out = torch.zeros(n, device="cuda")
    c.decode(p, out, scale=0.25)
    ref = torch.zeros(n)
    ref[top] = val * 0.25
    assert torch.equal(out.cpu(), ref)


@pytest.mark.parametrize("n", [4097, 100003])
def test_graddrop_against_definition(n):
    torch.manual_seed(500 + n)
    ratio = 0.001 if n > 10000 else 0.05
    c = Compressor("graddrop", ratio=ratio)
    g, r0 = torch.randn(n), torch.randn(n) * 0.3
    st = c.new_state(n, "cuda")
    st["residual"].copy_(r0)
    p = c.encode(g.cuda(), st)
    torch.cuda.synchronize()
    x = g + r0
    k = math.ceil(ratio * n)
    top = torch.topk(x.abs(), k).indices.sort().values
    idx, val = sparse_pairs(p, k)
    assert torch.equal(idx, top) and torch.equal(val, x[top])
    rest = x.clone()
    rest[top] = 0
    assert torch.equal(st["residual"].cpu(), rest), "residual = what was not sent"
