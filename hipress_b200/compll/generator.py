"""File-level driver of the generator: DSL file -> ``<out>/<Name>/<Name>_body.cuh``,
``<Name>_wrapper.cu``, ``<Name>.py`` and (optionally) ``lib<Name>.so``."""
from __future__ import annotations

import subprocess
from pathlib import Path

from .emit_cuda import generate

ROOT = Path(__file__).resolve().parents[2]
INCLUDE = ROOT / "csrc" / "include"
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-fmad=false", "-Xcompiler", "-fPIC"]


def generate_files(path, outdir="output", *, body=True, wrapper=True, register=True,
                   framework="torch", build=False):
    em = generate(Path(path).read_text())
    name = em.fn.name
    d = Path(outdir) / name
    d.mkdir(parents=True, exist_ok=True)
    written = []
    if body or build:
        (d / f"{name}_body.cuh").write_text(em.body_source())
        written.append(d / f"{name}_body.cuh")
    if wrapper or build:
        (d / f"{name}_wrapper.cu").write_text(em.wrapper_source())
        written.append(d / f"{name}_wrapper.cu")
    if register:
        (d / f"{name}.py").write_text(em.register_source(framework))
        written.append(d / f"{name}.py")
    if build:
        written.append(compile_generated(d, name, uses_library=em.uses_library))
    return written


def compile_generated(d: Path, name: str, nvcc: str = "nvcc", uses_library: bool = False) -> Path:
    out = d / f"lib{name}.so"
    cmd = [nvcc, *NVCC_FLAGS, "-shared", "-I", str(INCLUDE), "-I", str(d), "-o", str(out),
           str(d / f"{name}_wrapper.cu")]
    if uses_library:  # top-k / scatter stages call into the run-time library
        libdir = ROOT / "hipress_b200" / "_native"
        cmd += ["-L", str(libdir), "-lhipress_cuda", "-Xlinker", f"-rpath={libdir}"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("nvcc failed on generated code:\n" + r.stderr[-4000:])
    return out
