"""In-tree build of the native libraries.

Two shared objects are produced under ``kharon_b200/_lib``:

* ``libkharon_rt.so``   -- host runtime (C++17, g++), no CUDA dependency;
* ``libkharon_cuda.so`` -- every CUDA kernel, compiled by nvcc for ``sm_100a`` only
  (``-gencode arch=compute_100a,code=sm_100a``); cross-compiles without a GPU.

Objects are rebuilt only when a source or header is newer than the object.  Run
``python -m kharon_b200._build`` to build everything; ``--verbose`` adds ``-Xptxas -v``.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

ROOT = Path(__file__).resolve().parent
CSRC = ROOT / "csrc"
LIB = ROOT / "_lib"
OBJ = LIB / "obj"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr",
]
# --use_fast_math (approximate division / sqrt / tanh, flush-to-zero) only where exponentials and
# tanh sit in a hot loop: GEMM epilogues (GELU), attention, the decode kernels.  The optimizer
# (fp32 master weights, Adam moments), LayerNorm statistics, the loss and the ZeRO step are
# compiled with IEEE division and square root; their softmax exponentials call __expf explicitly.
FAST_MATH_FILES = {"gemm_tcgen05.cu", "gemm_skinny.cu", "flash_tcgen05.cu", "paged.cu", "fused_tp.cu"}


def _newer(srcs, target: Path) -> bool:
    if not target.exists():
        return True
    t = target.stat().st_mtime
    return any(Path(s).stat().st_mtime > t for s in srcs)


def _run(cmd, verbose=False):
    p = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if p.returncode != 0:
        raise RuntimeError("build failed: %s\n%s" % (" ".join(map(str, cmd)), p.stdout))
    if verbose and p.stdout.strip():
        print(p.stdout)
    return p.stdout


def build_runtime(force: bool = False) -> Path:
    LIB.mkdir(exist_ok=True)
    out = LIB / "libkharon_rt.so"
    srcs = [p for p in sorted((CSRC / "runtime").glob("*.cpp")) if not p.name.endswith("_selftest.cpp")]
    deps = srcs + sorted((CSRC / "runtime").glob("*.h"))
    if force or _newer(deps, out):
        cxx = os.environ.get("CXX", "g++")
        tmp = out.with_suffix(".so.tmp%d" % os.getpid())
        _run([cxx, "-O2", "-std=c++17", "-fPIC", "-shared", "-Wall", "-o", str(tmp)] + [str(s) for s in srcs])
        os.replace(tmp, out)
    return out


def nvcc_path() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    raise RuntimeError("nvcc not found")


def cuda_sources():
    return sorted((CSRC / "kernels").glob("*.cu")) + sorted((CSRC / "comm").glob("*.cu"))


def build_cuda(force: bool = False, verbose: bool = False) -> Path:
    LIB.mkdir(exist_ok=True)
    OBJ.mkdir(exist_ok=True)
    out = LIB / "libkharon_cuda.so"
    nvcc = nvcc_path()
    headers = sorted(CSRC.glob("**/*.cuh")) + sorted(CSRC.glob("**/*.h"))
    jobs = []
    objs = []
    for src in cuda_sources():
        obj = OBJ / (src.stem + ".o")
        objs.append(obj)
        if force or _newer([src] + headers, obj):
            fast = ["--use_fast_math"] if src.name in FAST_MATH_FILES else []
            cmd = [nvcc] + NVCC_FLAGS + fast + (["-Xptxas", "-v"] if verbose else []) + [
                "-I", str(CSRC), "-c", str(src), "-o", str(obj)]
            jobs.append(cmd)
    if jobs:
        with ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            list(ex.map(lambda c: _run(c, verbose), jobs))
    if force or jobs or _newer(objs, out):
        tmp = out.with_suffix(".so.tmp%d" % os.getpid())
        _run([nvcc, "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", str(tmp)]
             + [str(o) for o in objs])
        os.replace(tmp, out)
    return out


def build_all(force: bool = False, verbose: bool = False):
    return build_runtime(force), build_cuda(force, verbose)


if __name__ == "__main__":
    rt, cu = build_all(force="--force" in sys.argv, verbose="--verbose" in sys.argv)
    print(rt)
    print(cu)
