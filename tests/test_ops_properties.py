"""Property tests (hypothesis) of the CPU oracle: wire sizes, error-feedback
conservation, top-k count and threshold, determinism."""
import math

import pytest
import torch
from hypothesis import given, settings, strategies as st

from hipress_b200.ops import Compressor, sparse_pairs

sizes = st.integers(min_value=1, max_value=20000)
seeds = st.integers(min_value=0, max_value=2 ** 31 - 1)


@settings(max_examples=40, deadline=None)
@given(n=sizes, seed=seeds, name=st.sampled_from(["tbq", "onebit"]), scale=st.floats(1e-4, 10.0))
def test_error_feedback_conserves_the_signal(n, seed, name, scale):
    g = torch.randn(n, generator=torch.Generator().manual_seed(seed)) * scale
    c = Compressor(name, threshold=0.01)
    state = c.new_state(n, "cpu")
    r0 = torch.randn(n, generator=torch.Generator().manual_seed(seed + 1)) * 0.1 * scale
    state["residual"].copy_(r0)
    p = c.encode(g, state)
    assert p.numel() == c.payload_bytes(n)
    out = torch.empty(n)
    c.decode(p, out)
    assert torch.allclose(out + state["residual"], g + r0, rtol=1e-5, atol=1e-6 * scale)
    assert torch.equal(p, c.encode(g, {"residual": r0.clone()}))  # same input, same bytes


@settings(max_examples=40, deadline=None)
@given(n=sizes, seed=seeds, bits=st.sampled_from([1, 2, 4, 8]), step=st.integers(0, 1000))
def test_terngrad_stays_inside_one_gap(n, seed, bits, step):
    g = torch.randn(n, generator=torch.Generator().manual_seed(seed))
    c = Compressor("terngrad", bitwidth=bits)
    out = torch.empty(n)
    c.decode(c.encode(g, {}, step=step), out)
    for t0 in range(0, n, 4096):
        tile, dec = g[t0:t0 + 4096], out[t0:t0 + 4096]
        gap = (tile.max() - tile.min()) / (2 ** bits - 1)
        assert (dec - tile).abs().max() <= gap * (1 + 1e-4) + 1e-6
        assert dec.min() >= tile.min() - 1e-6 and dec.max() <= tile.max() + 1e-5 + gap * 1e-4


@settings(max_examples=40, deadline=None)
@given(n=sizes, seed=seeds, ratio=st.floats(0.0005, 0.5), name=st.sampled_from(["dgc", "graddrop"]))
def test_topk_sends_exactly_the_largest(n, seed, ratio, name):
    g = torch.randn(n, generator=torch.Generator().manual_seed(seed))
    c = Compressor(name, ratio=ratio)
    k = c.kmax(n)
    assert k == min(n, max(1, math.ceil(float(torch.tensor(ratio, dtype=torch.float32)) * n)))
    state = c.new_state(n, "cpu")
    idx, val = sparse_pairs(c.encode(g, state), k)
    assert idx.numel() == k and idx.unique().numel() == k
    thr = val.abs().min()
    rest = torch.ones(n, dtype=torch.bool)
    rest[idx] = False
    if rest.any():
        assert g[rest].abs().max() <= thr
    acc = state["accum_v"] if name == "dgc" else state["residual"]
    assert torch.all(acc[idx] == 0) and torch.equal(acc[rest], g[rest])
