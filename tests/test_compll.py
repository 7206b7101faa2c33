"""CompLL: DSL front end, CUDA and CPU emitters, the operator library and the worked
example.  (The generated operators are run in tests/test_y_compll_generated.py.)"""
import os
import shutil
import sys
from pathlib import Path

import pytest
import torch

from hipress_b200.compll import CompileError, generate, generate_files, parse, tokenize
from hipress_b200.compll import frontend as F

PSE = Path(__file__).resolve().parents[1] / "hipress_b200" / "compll" / "pse"
REF_PSE = Path(__file__).resolve().parents[1] / "baseline" / "_ref" / "src" / "CompLL" / "GCGen" / "pse"
HAVE_NVCC = shutil.which("nvcc") is not None or os.path.exists("/usr/local/cuda/bin/nvcc")


def test_lexer_float_literals_and_operators():
    toks = [(t.kind, t.text) for t in tokenize("x = 0.01 + 3e-2 << 2; // c\n y>=1")]
    assert ("float", "0.01") in toks and ("float", "3e-2") in toks
    assert ("op", "<<") in toks and ("op", ">=") in toks
    assert all(t[1] != "c" for t in toks)  # comment stripped


def test_parser_builds_typed_tree():
    fn = parse((PSE / "TernGradEncode.pse").read_text())
    assert fn.name == "TernGradEncode"
    assert [(t.name, t.vector, n) for t, n in fn.params] == [
        ("float", True, "gradient"), ("uint8", True, "compressed"), ("uint8", False, "bitwidth")]
    kinds = [type(s).__name__ for s in fn.body]
    assert kinds.count("Decl") >= 7 and kinds[-1] == "Assign"
    q = [s for s in fn.body if isinstance(s, F.Decl) and s.name == "Q"][0]
    assert q.type.vector and isinstance(q.type.bits, F.Name) and isinstance(q.init, F.Map)


def test_literal_bitwidth_and_precedence():
    fn = parse("void f(float* g, uint8* c){ uint<2>* Q = map(range(g.size), h); int a = 1 + 2 * 3 << 1; }")
    q = fn.body[0]
    assert isinstance(q.type.bits, F.Num) and q.type.bits.text == "2"
    a = fn.body[1].init
    assert isinstance(a, F.Binary) and a.op == "<<" and a.a.op == "+" and a.a.b.op == "*"


@pytest.mark.parametrize("src,msg", [
    ("void f(float* g){ foo x = 1; }", "unrecognized|expected|typename"),
    ("void f(float* g){ float a = reduce(g, 0); }", "three arguments"),
    ("void f(float* g, uint8* c){ uint<2>* Q = map(range(g.size), nolambda); c = concat(Q); }", "lambda"),
    ("void f(float* g){ float a = $; }", "unexpected character"),
])
def test_errors_carry_a_message(src, msg):
    import re
    with pytest.raises(CompileError) as e:
        generate(src).body_source()
    assert re.search(msg, str(e.value))


def test_unsupported_framework_is_an_error_not_ignored():
    em = generate((PSE / "TernGradDecode.pse").read_text())
    with pytest.raises(CompileError):
        em.register_source("mxnet")
    assert "def TernGradDecode(" in em.register_source("torch")


def test_emitter_structure():
    em = generate((PSE / "OnebitEncode.pse").read_text())
    # source order is kept: map, reduce, map, map
    assert [s[0] for s in em.stages] == ["map", "reduce", "map", "map"]
    body = em.body_source()
    assert "compll_rand01" not in body and "__shfl_xor_sync" in body
    em2 = generate((PSE / "TernGradEncode.pse").read_text())
    # two reduces fused into one pass; header offsets 0,1,2,6 then codes at 10
    assert [s[0] for s in em2.stages] == ["reduce", "map"] and len(em2.stages[0][1]) == 2
    assert em2.concats[0][1] == [("bitwidth", 0), ("pad", 1), ("lo", 2), ("hi", 6)]
    assert em2.syms["Q"].alias == ("compressed", 10)
    assert "compll_rand01" in em2.body_source()


@pytest.mark.skipif(not REF_PSE.exists(), reason="reference tree not present")
def test_reference_sources_are_accepted_unchanged(tmp_path):
    for name in ("TernGradEncode", "TernGradDecode"):
        em = generate((REF_PSE / f"{name}.pse").read_text())
        assert em.fn.name == name
        assert "__global__" in em.body_source()
    enc = generate((REF_PSE / "TernGradEncode.pse").read_text())
    # the 10-byte header of the reference: bitwidth, tail, min, max at 0,1,2,6
    assert enc.concats[0][1] == [("bitwidth", 0), ("tail", 1), ("min", 2), ("max", 6)]


@pytest.mark.skipif(not HAVE_NVCC, reason="nvcc not available")
def test_generated_code_compiles_for_sm100a(tmp_path):
    for f in sorted(PSE.glob("*.pse")):
        files = generate_files(f, tmp_path, build=True)
        assert files[-1].name.startswith("lib") and files[-1].exists()


def test_topk_and_scatter_lower_to_library_stages():
    em = generate((PSE / "DgcEncode.pse").read_text())
    assert [s[0] for s in em.stages] == ["map", "map", "topk"] and em.uses_library
    w = em.wrapper_source()
    assert "hp_cuda_sparse_encode(4, nullptr, p_accum_v, p_momentum_u" in w
    em = generate((PSE / "GradDropDecode.pse").read_text())
    assert [s[0] for s in em.stages] == ["scatter"]
    with pytest.raises(CompileError):
        generate("void f(float* g, uint8* c){ float x = 1.0; x = topk(g, 3); }")


def test_operator_library_builds_on_first_use_and_runs_on_cpu_tensors():
    from hipress_b200.compll import available, load_op
    names = available()
    assert {"TbqEncode", "TbqDecode", "OnebitEncode", "TernGradEncode", "DgcEncode",
            "GradDropEncode", "SparseDecodeAccumulate"} <= set(names)
    enc, dec = load_op("TbqEncode"), load_op("TbqDecode")
    assert load_op("TbqEncode") is enc                   # cached
    n = 1000
    g = torch.linspace(-0.03, 0.03, n)
    r = torch.zeros(n)
    comp = torch.zeros(4 + (n + 3) // 4, dtype=torch.uint8)
    enc(g, r, comp, 0.01)
    out = torch.empty(n)
    dec(comp, out)
    assert torch.allclose(out + r, g, atol=1e-7)
    levels = torch.tensor([-0.01, 0.0, 0.01])
    assert (out.unsqueeze(1) - levels).abs().min(dim=1).values.max().item() < 1e-9
    with pytest.raises(ValueError):
        enc(g[::2], r, comp, 0.01)                       # not contiguous
    with pytest.raises(KeyError):
        load_op("NoSuchOperator")


def test_new_algorithm_example_trains_on_two_cpu_ranks(tmp_path):
    """The worked example: DSL source -> operators -> registered algorithm ->
    data-parallel training, launched the way its docstring says."""
    import json
    import subprocess
    from _mp import free_port
    root = Path(__file__).resolve().parents[1]
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nproc-per-node", "2",
                        "--master-addr", "127.0.0.1", "--master-port", str(free_port()), "-m",
                        "hipress_b200.compll.examples.train_with_new_algorithm", "--steps", "25",
                        "--topo", "ps", "--out", str(tmp_path)],
                       capture_output=True, text=True, cwd=root, timeout=600,
                       env={**os.environ, "CUDA_VISIBLE_DEVICES": ""})
    assert r.returncode == 0, r.stderr[-2000:]
    line = json.loads([row for row in r.stdout.splitlines() if row.startswith("{")][-1])
    assert line["replicas_identical"] and line["backend"] == "host" and line["ranks"] == 2
    assert line["last_loss"] < 0.2 * line["first_loss"] and line["compressed_fraction"] > 0.9


# ------------------------------------------------------------ fused target: phase plans
def _phases(name):
    from hipress_b200.compll.emit_cuda import generate as gen
    pse = Path(__file__).resolve().parents[1] / "hipress_b200" / "compll" / "pse"
    plan = gen((pse / f"{name}.pse").read_text()).fused_plan()
    if plan is None:
        return None
    return [[(it.target if it.kind == "map" else "reduce:" + it.sym.name) for it in ph.items]
            for ph in plan.phases]


def test_fused_plans_of_the_shipped_operators():
    """One launch per function: maps that only need their own element of what an earlier
    map wrote share a phase (TBQ: all three), a stage that needs a reduction's result
    waits behind a barrier (onebit's leftover map, TernGrad's quantising map), and
    functions with a library-lowered stage keep the staged target."""
    assert _phases("TbqEncode") == [["residual", "Q", "residual"]]
    assert _phases("OnebitEncode") == [["residual", "reduce:total", "S"], ["residual"]]
    assert _phases("TernGradEncode") == [["reduce:hi", "reduce:lo"], ["Q"]]
    for dec in ("TbqDecode", "OnebitDecode", "TernGradDecode", "TbqDecodeAccumulate"):
        assert _phases(dec) == [["gradient"]]
    assert _phases("DgcEncode") is None and _phases("SparseDecodeAccumulate") is None


def test_maps_around_a_library_stage_still_share_a_kernel():
    """DgcEncode = two state-update maps + the library's exact top-k: the maps are one
    kernel (one pass over u, v and g), launched right before the library call."""
    from hipress_b200.compll.emit_cuda import generate as gen
    pse = Path(__file__).resolve().parents[1] / "hipress_b200" / "compll" / "pse"
    em = gen((pse / "DgcEncode.pse").read_text())
    segs = em.segments()
    assert [(i0, cnt) for i0, cnt, _ in segs] == [(0, 2)]
    assert [[it.target for it in ph.items] for ph in segs[0][2].phases] == [["momentum_u", "accum_v"]]
    body, wrap = em.body_source(), em.wrapper_source()
    assert "DgcEncode_seg0_kernel" in body and "_map0_kernel" not in body and "_map1_kernel" not in body
    assert wrap.index("DgcEncode_seg0_kernel") < wrap.index("hp_cuda_sparse_encode(4")
    assert "cudaLaunchCooperativeKernel" not in wrap        # one phase: no grid barrier
    # a single map next to the library call stays as it was
    one = gen((pse / "GradDropEncode.pse").read_text())
    assert one.segments() == [] and "_map0_kernel" in one.body_source()
    # and the staged target is still available
    staged = gen((pse / "DgcEncode.pse").read_text(), fuse=False)
    assert staged.segments() == [] and "_map1_kernel" in staged.body_source()


def test_fused_target_starts_a_new_phase_for_reads_at_another_index():
    from hipress_b200.compll.emit_cuda import generate as gen
    src = """
void Shift(float* a, float* b, float* c) {
    lambda_func first = [&](int i) -> float { return a[i] * 2.0; };
    b = map(range(a.size), first);
    lambda_func second = [&](int i) -> float { return b[a.size - 1 - i] + 1.0; };
    c = map(range(a.size), second);
}
"""
    em = gen(src)
    plan = em.fused_plan()
    assert plan is not None and len(plan.phases) == 2      # b is read back to front: barrier
    body = em.body_source()
    assert "compll_grid_sync" in body and "Shift_fused_kernel" in body
    assert "cudaLaunchCooperativeKernel" in em.wrapper_source()
    staged = gen(src, fuse=False)
    assert "Shift_map0_kernel" in staged.body_source() and "fused" not in staged.body_source()
