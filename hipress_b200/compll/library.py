"""The shipped CompLL operators, generated and compiled in-tree.

``hipress_b200/compll/pse/*.pse`` holds the DSL sources of the library (encode,
decode and fused decode-accumulate for the five algorithms).  ``build_all()``
runs the generator on each of them and compiles both targets into
``hipress_b200/compll/_built/<Name>/``; ``load_op(name)`` returns the generated
PyTorch binding, building it first when its sources changed.

    from hipress_b200.compll import load_op
    encode = load_op("TbqEncode")          # encode(gradient, residual, compressed, threshold)

This is the counterpart of the reference's step "copy the generated operator into
the framework and rebuild it" (README.md:262-270 of mark14wu/hipress): here the
generated operator is a self-contained shared library next to its binding.
"""
from __future__ import annotations

import hashlib
import importlib.util
import shutil
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

from .generator import INCLUDE, generate_files

HERE = Path(__file__).resolve().parent
PSE = HERE / "pse"
BUILT = HERE / "_built"
_ops: dict = {}


def available() -> list[str]:
    """Names of the shipped operators."""
    return sorted(p.stem for p in PSE.glob("*.pse"))


def _have_nvcc() -> bool:
    from .._native.build import nvcc_path
    return nvcc_path() is not None


def _digest(name: str, target: str) -> str:
    h = hashlib.sha256()
    for p in [PSE / f"{name}.pse", HERE / "frontend.py", HERE / "emit_cuda.py", HERE / "emit_host.py",
              HERE / "generator.py", INCLUDE / "hipress" / "compll_rt.cuh", INCLUDE / "hipress" / "common.h"]:
        h.update(p.read_bytes())
    h.update(target.encode())
    return h.hexdigest()


def build_op(name: str, target: str | None = None, force: bool = False) -> Path:
    """Generate and compile one shipped operator; returns its directory.  ``target``
    defaults to both ("all") when nvcc is present and to "cpu" otherwise."""
    if name not in available():
        raise KeyError(f"no shipped operator {name!r}; have {available()}")
    target = target or ("all" if _have_nvcc() else "cpu")
    d = BUILT / name
    stamp = d / f".{target}.sha"
    dg = _digest(name, target)
    if not force and stamp.exists() and stamp.read_text() == dg:
        return d
    generate_files(PSE / f"{name}.pse", BUILT, build=True, target=target)
    stamp.write_text(dg)
    _ops.pop(name, None)
    return d


def build_all(target: str | None = None, force: bool = False, jobs: int = 8) -> dict:
    """Build every shipped operator (in parallel); name -> directory."""
    names = available()
    with ThreadPoolExecutor(max_workers=max(1, min(jobs, len(names)))) as ex:
        dirs = list(ex.map(lambda n: build_op(n, target, force), names))
    return dict(zip(names, dirs))


def load_op(name: str, target: str | None = None):
    """The generated binding ``name(*tensors_and_scalars, seed=0, stream=None)``.  It
    dispatches on the tensors' device: CPU tensors run the C++ target, CUDA tensors
    the sm_100a kernels (which need the operator built with nvcc present)."""
    if name in _ops:
        return _ops[name]
    d = build_op(name, target)
    spec = importlib.util.spec_from_file_location(f"hipress_b200.compll._built.{name}", d / f"{name}.py")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    _ops[name] = getattr(mod, name)
    return _ops[name]


def clean() -> None:
    """Remove every built operator."""
    if BUILT.exists():
        shutil.rmtree(BUILT)
    _ops.clear()
