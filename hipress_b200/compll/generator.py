"""File-level driver of the generator: DSL file -> ``<out>/<Name>/<Name>_body.cuh``,
``<Name>_wrapper.cu`` (CUDA target), ``<Name>_cpu.cpp`` (CPU target), ``<Name>.py``
(binding that dispatches on the tensors' device) and, optionally, ``lib<Name>.so`` /
``lib<Name>_cpu.so``."""
from __future__ import annotations

import subprocess
from pathlib import Path

from .emit_cuda import generate

ROOT = Path(__file__).resolve().parents[2]
INCLUDE = ROOT / "csrc" / "include"
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-fmad=false", "-Xcompiler", "-fPIC"]


CXX_FLAGS = ["-O2", "-std=c++17", "-ffp-contract=off", "-fPIC", "-shared", "-Wno-unknown-pragmas"]
TARGETS = ("cuda", "cpu", "all")


def generate_files(path, outdir="output", *, body=True, wrapper=True, register=True,
                   framework="torch", build=False, target="all"):
    """``target``: "cuda", "cpu" or "all".  With ``build`` the CUDA library is the
    last entry of the returned list."""
    if target not in TARGETS:
        raise ValueError(f"target must be one of {TARGETS}")
    em = generate(Path(path).read_text())
    name = em.fn.name
    d = Path(outdir) / name
    d.mkdir(parents=True, exist_ok=True)
    written = []
    if target in ("cpu", "all") and (body or build):
        (d / f"{name}_cpu.cpp").write_text(em.host_source())
        written.append(d / f"{name}_cpu.cpp")
        if build:
            written.append(compile_host(d, name, uses_library=em.uses_library))
    if target == "cpu":
        if register:
            (d / f"{name}.py").write_text(em.register_source(framework))
            written.append(d / f"{name}.py")
        return written
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


def compile_host(d: Path, name: str, cxx: str = "g++", uses_library: bool = False) -> Path:
    out = d / f"lib{name}_cpu.so"
    cmd = [cxx, *CXX_FLAGS, "-I", str(INCLUDE), "-o", str(out), str(d / f"{name}_cpu.cpp")]
    if uses_library:  # top-k / scatter stages call into the run-time library
        from .._native import lib as _lib
        _lib.cpu()    # builds libhipress_cpu.so when it is missing
        libdir = ROOT / "hipress_b200" / "_native"
        cmd += ["-L", str(libdir), "-lhipress_cpu", f"-Wl,-rpath={libdir}"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("g++ failed on generated code:\n" + r.stderr[-4000:])
    return out


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
