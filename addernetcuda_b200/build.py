"""Builds libadder_b200.so in-tree with nvcc for sm_100a (no libtorch, no Python headers).

    python -m addernetcuda_b200.build [--force] [--verbose]

The library is placed next to this file so that it travels with the source tree.  It links the
CUDA runtime statically and exports only the extern "C" entry points of include/adder_b200.h.
"""
from __future__ import annotations

import argparse
import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
INCLUDE = PKG.parent / "include"
LIB = PKG / "libadder_b200.so"
SOURCES = ["api.cu", "adder_fwd.cu", "adder_bwd_input.cu", "adder_bwd_weight.cu", "adder_bwd_weight_1x1.cu", "adder_pointwise.cu", "static_scratch.cu", "batchnorm.cu"]
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]


def find_nvcc() -> str:
    cand = os.environ.get("NVCC") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(cand).exists():
        raise RuntimeError("nvcc not found (set NVCC or add it to PATH)")
    return cand


def _stale() -> bool:
    if not LIB.exists():
        return True
    t = LIB.stat().st_mtime
    deps = list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h")) + list(INCLUDE.glob("*.h"))
    return any(d.stat().st_mtime > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compile every translation unit (in parallel) and link the shared library."""
    if not force and not _stale():
        return LIB
    nvcc = find_nvcc()
    objdir = PKG / "build"
    objdir.mkdir(exist_ok=True)
    common = [nvcc, "-O3", "-std=c++17", "-lineinfo", *ARCH_FLAGS, "-Xcompiler", "-fPIC,-fvisibility=hidden",
              "-I", str(INCLUDE), "-I", str(CSRC)]
    if verbose:
        common += ["-Xptxas", "-v"]
    procs = []
    objs = []
    for src in SOURCES:
        obj = objdir / (src[:-3] + ".o")
        objs.append(str(obj))
        procs.append((src, subprocess.Popen(common + ["-c", str(CSRC / src), "-o", str(obj)],
                                            stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    failed = False
    for src, p in procs:
        out, _ = p.communicate()
        if p.returncode != 0:
            failed = True
            sys.stderr.write(f"--- nvcc failed on {src} ---\n{out}\n")
        elif verbose or out.strip():
            sys.stderr.write(f"--- {src} ---\n{out}\n")
    if failed:
        raise RuntimeError("nvcc compilation failed")
    link = [nvcc, "-shared", *ARCH_FLAGS, "-o", str(LIB), *objs, "-cudart", "static"]
    subprocess.run(link, check=True)
    return LIB


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true", help="print ptxas register/shared-memory usage")
    a = ap.parse_args()
    print(build(force=a.force, verbose=a.verbose))
