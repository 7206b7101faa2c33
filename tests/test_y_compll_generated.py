"""CompLL-generated operators run: the C++ target everywhere, the sm_100a kernels
on a GPU, against plain PyTorch restatements of the DSL semantics.  (Front end
and emitter structure: tests/test_compll.py.)"""
import importlib.util
from pathlib import Path

import pytest
import torch

from hipress_b200.compll import generate, generate_files

PSE = Path(__file__).resolve().parents[1] / "hipress_b200" / "compll" / "pse"
REF_PSE = Path(__file__).resolve().parents[1] / "baseline" / "_ref" / "src" / "CompLL" / "GCGen" / "pse"

# ------------------------------------------------- generated code, both targets
DEVICES = ["cpu", pytest.param("cuda", marks=pytest.mark.gpu)]


def _sync(device):
    if device == "cuda":
        torch.cuda.synchronize()


def _load(tmp_path, name, src_dir=PSE, device="cuda"):
    generate_files(src_dir / f"{name}.pse", tmp_path, build=True,
                   target="cpu" if device == "cpu" else "cuda")
    spec = importlib.util.spec_from_file_location(name, tmp_path / name / f"{name}.py")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return getattr(mod, name)


@pytest.mark.parametrize("device", DEVICES)
@pytest.mark.parametrize("bits", [1, 2, 4, 8])
@pytest.mark.parametrize("n", [7, 4096, 100003])
def test_generated_terngrad_roundtrip(tmp_path, bits, n, device):
    enc = _load(tmp_path, "TernGradEncode", device=device)
    dec = _load(tmp_path, "TernGradDecode", device=device)
    torch.manual_seed(n)
    g = torch.randn(n, device=device)
    per = 8 // bits
    comp = torch.zeros(10 + (n + per - 1) // per, dtype=torch.uint8, device=device)
    enc(g, comp, bits, seed=3)
    out = torch.full((n,), 7.0, device=device)
    dec(comp, out)
    _sync(device)
    hdr = comp[:10].cpu()
    assert hdr[0].item() == bits and hdr[1].item() == (per - n % per) % per
    import struct
    lo, hi = struct.unpack("<ff", bytes(hdr[2:10].tolist()))
    assert lo == g.min().item() and hi == g.max().item()
    gap = (hi - lo) / (2 ** bits - 1)
    assert (out - g).abs().max().item() <= gap * (1 + 1e-5) + 1e-6
    # decoded values sit on the quantisation grid
    lv = (out - lo) / gap
    assert (lv - lv.round()).abs().max().item() < 1e-3
    # same seed, same payload; the stochastic rounding is unbiased on average
    comp2 = torch.zeros_like(comp)
    enc(g, comp2, bits, seed=3)
    assert torch.equal(comp, comp2)
    if bits == 2 and n > 50000:
        assert abs((out - g).mean().item()) < 0.02 * gap


@pytest.mark.parametrize("device", DEVICES)
def test_generated_onebit_and_tbq_with_error_feedback(tmp_path, device):
    n = 50001
    torch.manual_seed(0)
    g = torch.randn(n, device=device) * 0.02
    r0 = torch.randn(n, device=device) * 0.005
    x = g + r0
    # onebit
    enc = _load(tmp_path, "OnebitEncode", device=device)
    dec = _load(tmp_path, "OnebitDecode", device=device)
    r = r0.clone()
    comp = torch.zeros(4 + (n + 7) // 8, dtype=torch.uint8, device=device)
    enc(g, r, comp)
    out = torch.empty(n, device=device)
    dec(comp, out)
    scale = comp[:4].cpu().clone().view(torch.float32).item()
    assert scale == pytest.approx(x.abs().mean().item(), rel=1e-4)
    assert torch.equal(out < 0, x < 0)
    assert torch.allclose(out + r, x, atol=1e-6)
    # tbq
    enc = _load(tmp_path, "TbqEncode", device=device)
    dec = _load(tmp_path, "TbqDecode", device=device)
    r = r0.clone()
    comp = torch.zeros(4 + (n + 3) // 4, dtype=torch.uint8, device=device)
    enc(g, r, comp, 0.01)
    dec(comp, out)
    want = torch.where(x >= 0.01, 0.01, torch.where(x <= -0.01, -0.01, 0.0))
    assert torch.allclose(out, want.float())
    assert torch.allclose(out + r, x, atol=1e-7)


@pytest.mark.parametrize("device", DEVICES)
@pytest.mark.skipif(not REF_PSE.exists(), reason="reference tree not present")
def test_reference_dsl_sources_run(tmp_path, device):
    """The reference's own TernGrad sources, generated and run unchanged (n is a
    multiple of 4 and bitwidth 2, the case its tail arithmetic covers)."""
    enc = _load(tmp_path, "TernGradEncode", REF_PSE, device=device)
    dec = _load(tmp_path, "TernGradDecode", REF_PSE, device=device)
    n = 4096 * 3
    g = torch.randn(n, device=device)
    comp = torch.zeros(10 + n // 4, dtype=torch.uint8, device=device)
    enc(g, comp, 2)
    out = torch.empty(n, device=device)
    dec(comp, out)
    gap = (g.max() - g.min()).item() / 3
    inside = g < g.max() - gap  # the source does not clamp a round-up at the maximum
    assert (out - g)[inside].abs().max().item() <= gap * 1.001


@pytest.mark.parametrize("device", DEVICES)
def test_generated_decode_accumulate(tmp_path, device):
    enc = _load(tmp_path, "TbqEncode", device=device)
    acc = _load(tmp_path, "TbqDecodeAccumulate", device=device)
    n = 30001
    torch.manual_seed(4)
    g = torch.randn(n, device=device) * 0.02
    r = torch.zeros(n, device=device)
    comp = torch.zeros(4 + (n + 3) // 4, dtype=torch.uint8, device=device)
    enc(g, r, comp, 0.01)
    base = torch.randn(n, device=device)
    out = base.clone()
    acc(comp, out, 0.25)
    want = base + 0.25 * torch.where(g >= 0.01, 0.01, torch.where(g <= -0.01, -0.01, 0.0))
    assert torch.allclose(out, want.float(), atol=1e-7)


@pytest.mark.parametrize("device", DEVICES)
def test_generated_graddrop_and_dgc_use_the_library_topk(tmp_path, device):
    import math
    n, ratio = 200003, 0.001
    k = max(int(math.ceil(torch.tensor(ratio, dtype=torch.float32).item() * n)), 1)
    nbytes = 16 + 2 * ((4 * k + 15) // 16 * 16)
    torch.manual_seed(9)
    g = torch.randn(n, device=device)
    # GradDrop
    enc, dec = _load(tmp_path, "GradDropEncode", device=device), _load(tmp_path, "GradDropDecode", device=device)
    r0 = torch.randn(n, device=device) * 0.3
    r = r0.clone()
    comp = torch.zeros(nbytes, dtype=torch.uint8, device=device)
    enc(g, r, comp, ratio)
    out = torch.ones(n, device=device)
    dec(comp, out, 0.5)
    _sync(device)
    x = g + r0
    top = torch.topk(x.abs(), k).indices
    assert int((out != 0).sum()) == k
    assert torch.allclose(out[top], 0.5 * x[top])
    assert torch.all(r[top] == 0)
    mask = torch.ones(n, dtype=torch.bool, device=device)
    mask[top] = False
    assert torch.allclose(r[mask], x[mask])
    # DGC
    enc = _load(tmp_path, "DgcEncode", device=device)
    u = torch.randn(n, device=device) * 0.1
    v = torch.randn(n, device=device) * 0.1
    u_ref = 0.9 * u + g
    v_ref = v + u_ref
    comp.zero_()
    enc(g, u, v, comp, ratio, 0.9)
    dec(comp, out, 1.0)
    _sync(device)
    top = torch.topk(v_ref.abs(), k).indices
    assert torch.allclose(out[top], v_ref[top], rtol=1e-6)
    assert torch.all(v[top] == 0) and torch.all(u[top] == 0)
    mask = torch.ones(n, dtype=torch.bool, device=device)
    mask[top] = False
    assert torch.allclose(v[mask], v_ref[mask], rtol=1e-6) and torch.allclose(u[mask], u_ref[mask], rtol=1e-6)


def test_decode_accumulate_for_every_format(tmp_path):
    """The fused decode + merge of each wire format, generated from the DSL and run
    on the CPU target: target += decode(payload) * weight."""
    device = "cpu"
    n = 20011
    torch.manual_seed(11)
    g = torch.randn(n) * 0.02
    base = torch.randn(n)
    # onebit
    enc = _load(tmp_path, "OnebitEncode", device=device)
    dec = _load(tmp_path, "OnebitDecode", device=device)
    acc = _load(tmp_path, "OnebitDecodeAccumulate", device=device)
    comp = torch.zeros(4 + (n + 7) // 8, dtype=torch.uint8)
    enc(g, torch.zeros(n), comp)
    plain = torch.empty(n)
    dec(comp, plain)
    out = base.clone()
    acc(comp, out, 0.125)
    assert torch.allclose(out, base + 0.125 * plain, atol=1e-7)
    # terngrad, 4 bits
    enc = _load(tmp_path, "TernGradEncode", device=device)
    dec = _load(tmp_path, "TernGradDecode", device=device)
    acc = _load(tmp_path, "TernGradDecodeAccumulate", device=device)
    comp = torch.zeros(10 + (n + 1) // 2, dtype=torch.uint8)
    enc(g, comp, 4, seed=5)
    dec(comp, plain)
    out = base.clone()
    acc(comp, out, 0.5)
    assert torch.allclose(out, base + 0.5 * plain, atol=1e-7)
    # sparse (GradDrop payload), scatter_add keeps what the target held
    import math
    ratio = 0.01
    k = max(int(math.ceil(torch.tensor(ratio, dtype=torch.float32).item() * n)), 1)
    enc = _load(tmp_path, "GradDropEncode", device=device)
    acc = _load(tmp_path, "SparseDecodeAccumulate", device=device)
    comp = torch.zeros(16 + 2 * ((4 * k + 15) // 16 * 16), dtype=torch.uint8)
    enc(g, torch.zeros(n), comp, ratio)
    out = base.clone()
    acc(comp, out, 0.25)
    top = torch.topk(g.abs(), k).indices
    want = base.clone()
    want[top] += 0.25 * g[top]
    assert torch.allclose(out, want, atol=1e-7)
    em = generate((PSE / "SparseDecodeAccumulate.pse").read_text())
    assert "n_gradient,\n" in em.wrapper_source() and ", 1, stream)" in em.wrapper_source()
    assert ", 0, stream)" in generate((PSE / "GradDropDecode.pse").read_text()).wrapper_source()
