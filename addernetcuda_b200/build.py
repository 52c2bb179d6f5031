"""Builds libadder_b200.so in-tree with nvcc for sm_100a (no libtorch, no Python headers).

    python -m addernetcuda_b200.build [--force] [--verbose]

The library is placed next to this file so that it travels with the source tree.  It links the
CUDA runtime statically and exports only the extern "C" entry points of include/adder_b200.h.
A second library, libadder_b200_tuning.so, is linked from the same objects with the C-ABI layer compiled
with -DADDER_B200_TUNING: it adds the tile-override setters that parameter sweeps and some tests use and
that the product library deliberately lacks.
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
TUNING_LIB = PKG / "libadder_b200_tuning.so"   # same objects, api.cu compiled with -DADDER_B200_TUNING
SOURCES = ["api.cu", "adder_fwd.cu", "adder_bwd_input.cu", "adder_bwd_weight.cu", "adder_bwd_weight_pipe.cu", "adder_bwd_weight_tma.cu", "tma_host.cu", "adder_bwd_weight_1x1.cu", "adder_pointwise.cu", "static_scratch.cu", "batchnorm.cu", "peer_allreduce.cu"]
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]


def find_nvcc() -> str:
    cand = os.environ.get("NVCC") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(cand).exists():
        raise RuntimeError("nvcc not found (set NVCC or add it to PATH)")
    return cand


def _stale() -> bool:
    if not LIB.exists() or not TUNING_LIB.exists():
        return True
    t = min(LIB.stat().st_mtime, TUNING_LIB.stat().st_mtime)
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
    # the tuning variant of the C-ABI layer: the only translation unit that differs between the two libraries
    api_tuning = objdir / "api_tuning.o"
    procs.append(("api.cu (tuning)", subprocess.Popen(common + ["-DADDER_B200_TUNING", "-c", str(CSRC / "api.cu"), "-o", str(api_tuning)],
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
    tuning_objs = [str(api_tuning) if o.endswith("/api.o") else o for o in objs]
    subprocess.run([nvcc, "-shared", *ARCH_FLAGS, "-o", str(TUNING_LIB), *tuning_objs, "-cudart", "static"], check=True)
    return LIB


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true", help="print ptxas register/shared-memory usage")
    a = ap.parse_args()
    print(build(force=a.force, verbose=a.verbose))
