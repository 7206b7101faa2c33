"""Builds the two native libraries in-tree.

``libhipress_cpu.so``  g++   CPU oracle, planner cost model, host runtime
``libhipress_cuda.so`` nvcc  sm_100a kernels (``-gencode arch=compute_100a,code=sm_100a``)

Both expose a plain C ABI that :mod:`hipress_b200._native.lib` binds with ctypes,
so neither needs the PyTorch headers and a full rebuild takes well under a minute.
Run ``python -m hipress_b200._native.build`` (add ``--force`` to rebuild).
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

HERE = Path(__file__).resolve().parent
ROOT = HERE.parent.parent
CSRC = ROOT / "csrc"
OBJ = HERE / "build"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-fmad=false", "-Xcompiler", "-fPIC", "-Xptxas", "-v",
]
GXX_FLAGS = ["-O2", "-std=c++17", "-fPIC", "-ffp-contract=off", "-Wall"]


def _sources():
    cpu = sorted((CSRC / "cpu").glob("*.cpp"))
    cuda = sorted((CSRC / "cuda").glob("*.cu"))
    return cpu, cuda


def _digest(paths) -> str:
    h = hashlib.sha256()
    deps = list(paths) + sorted((CSRC / "include" / "hipress").glob("*")) + \
        sorted((CSRC / "cuda").glob("*.cuh"))
    for p in deps:
        h.update(p.name.encode())
        h.update(p.read_bytes())
    h.update(" ".join(NVCC_FLAGS + GXX_FLAGS).encode())
    return h.hexdigest()


def _run(cmd, log):
    r = subprocess.run(cmd, capture_output=True, text=True)
    log.write(" ".join(map(str, cmd)) + "\n" + r.stdout + r.stderr + "\n")
    if r.returncode != 0:
        raise RuntimeError("native build failed:\n" + " ".join(map(str, cmd)) + "\n" + r.stderr[-4000:])
    return r


def nvcc_path() -> str | None:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    return None


def build_debug(force: bool = False, verbose: bool = False):
    """The CUDA library once more with ``-DHIPRESS_DEBUG``: the kernels check every
    payload-slot index against its inbox, record a violation in the status word and
    skip the access (what stands in for compute-sanitizer where that tool is not
    available).  Loaded instead of the normal library when HIPRESS_DEBUG=1."""
    nv = nvcc_path()
    if nv is None:
        return None
    _, cuda_src = _sources()
    obj = OBJ / "debug"
    obj.mkdir(parents=True, exist_ok=True)
    out = HERE / "libhipress_cuda_debug.so"
    stamp = obj / "cuda.sha"
    dg = _digest(cuda_src) + "-debug"
    if not force and out.exists() and stamp.exists() and stamp.read_text() == dg:
        return out
    inc = ["-I", str(CSRC / "include"), "-I", str(CSRC / "cuda")]
    with open(OBJ / "build.log", "a") as log:
        objs = [obj / (s.stem + ".o") for s in cuda_src]

        def one(pair):
            s, o = pair
            return _run([nv, *NVCC_FLAGS, "-DHIPRESS_DEBUG", *inc, "-c", str(s), "-o", str(o)], log)

        with ThreadPoolExecutor(max_workers=min(8, len(cuda_src))) as ex:
            list(ex.map(one, zip(cuda_src, objs)))
        _run([nv, "-shared", "-o", str(out), *map(str, objs), "-lcudart"], log)
    stamp.write_text(dg)
    if verbose:
        print("built", out)
    return out


def build(force: bool = False, verbose: bool = False) -> dict:
    """Compile whatever is out of date; returns the paths of the libraries."""
    cpu_src, cuda_src = _sources()
    OBJ.mkdir(exist_ok=True)
    out = {"cpu": HERE / "libhipress_cpu.so", "cuda": HERE / "libhipress_cuda.so"}
    inc = ["-I", str(CSRC / "include")]
    with open(OBJ / "build.log", "a") as log:
        stamp = OBJ / "cpu.sha"
        dg = _digest(cpu_src)
        if force or not out["cpu"].exists() or not stamp.exists() or stamp.read_text() != dg:
            _run(["g++", *GXX_FLAGS, *inc, "-shared", "-o", str(out["cpu"]), *map(str, cpu_src)], log)
            stamp.write_text(dg)
            if verbose:
                print("built", out["cpu"])
        nv = nvcc_path()
        if nv is None:
            if not out["cuda"].exists():
                out["cuda"] = None
            return out
        stamp = OBJ / "cuda.sha"
        dg = _digest(cuda_src)
        if force or not out["cuda"].exists() or not stamp.exists() or stamp.read_text() != dg:
            objs = [OBJ / (s.stem + ".o") for s in cuda_src]

            def one(pair):
                s, o = pair
                return _run([nv, *NVCC_FLAGS, *inc, "-I", str(CSRC / "cuda"), "-c", str(s), "-o", str(o)], log)

            with ThreadPoolExecutor(max_workers=min(8, len(cuda_src))) as ex:
                list(ex.map(one, zip(cuda_src, objs)))
            _run([nv, "-shared", "-o", str(out["cuda"]), *map(str, objs), "-lcudart"], log)
            stamp.write_text(dg)
            if verbose:
                print("built", out["cuda"])
    return out


def main():
    print(build(force="--force" in sys.argv, verbose=True))
    if "--debug" in sys.argv:
        print(build_debug(force="--force" in sys.argv, verbose=True))


if __name__ == "__main__":
    main()
