"""Installs the unmodified reference (LingYeAI/AdderNetCUDA) into baseline/_ref/ (git-ignored).

    python baseline/install_ref.py [--reference /path/to/AdderNetCUDA] [--no-extension]

Two things land in baseline/_ref/:

  * the reference's Python files (adder.py, resnet20.py, resnet50.py, vgg.py, densenet.py), copied
    byte for byte.  The GPU tests import the model files from there and run them on top of this
    package's drop-in `adder` module; the layer benchmark imports adder.py itself from there to time
    the reference's own path (unfold + its CUDA kernels).
  * its CUDA extension `adder_cuda`, built for sm_100 with the reference's own setup.py through
    `pip install --target`.  The sources are first copied to a scratch directory (the checkout may
    be read-only) and four tokens are changed there: `AT_DISPATCH_ALL_TYPES(x.type(), ...)` ->
    `AT_DISPATCH_ALL_TYPES(x.scalar_type(), ...)` at adder.cu:310,344,391,453, without which the file
    does not compile against PyTorch >= 2.0.  Nothing else is touched; no kernel line changes.

Nothing in baseline/_ref/ is part of the product or of its history.
"""
from __future__ import annotations

import argparse
import os
import shutil
import subprocess
import sys
import tempfile
from pathlib import Path

HERE = Path(__file__).resolve().parent
DEST = HERE / "_ref"
PY_FILES = ["adder.py", "resnet20.py", "resnet50.py", "vgg.py", "densenet.py"]


def install_python_files(ref: Path) -> None:
    DEST.mkdir(parents=True, exist_ok=True)
    for name in PY_FILES:
        shutil.copyfile(ref / name, DEST / name)


def extension_present() -> bool:
    return any(DEST.glob("adder_cuda*.so"))


def install_extension(ref: Path, log=sys.stderr) -> bool:
    """Build the reference's adder_cuda extension into baseline/_ref/.  Returns True when it is there."""
    if extension_present():
        return True
    with tempfile.TemporaryDirectory(prefix="addernet_ref_") as tmp:
        src = Path(tmp) / "adder_cuda"
        shutil.copytree(ref / "adder_cuda", src)
        cu = src / "adder.cu"
        text = cu.read_text()
        patched = text.replace("AT_DISPATCH_ALL_TYPES(x.type(),", "AT_DISPATCH_ALL_TYPES(x.scalar_type(),")
        if text.count("AT_DISPATCH_ALL_TYPES(x.type(),") != 4:
            log.write("install_ref: unexpected adder.cu (dispatch lines not found); extension not built\n")
            return False
        cu.write_text(patched)
        env = dict(os.environ, TORCH_CUDA_ARCH_LIST="10.0", MAX_JOBS="4")
        cmd = [sys.executable, "-m", "pip", "install", "--no-index", "--no-build-isolation", "--no-deps",
               "--find-links", "/opt/wheelhouse", "--target", str(DEST), str(src)]
        r = subprocess.run(cmd, env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
        if r.returncode != 0:
            log.write("install_ref: building the reference extension failed:\n" + r.stdout[-2000:] + "\n")
            return False
    return extension_present()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=os.environ.get("ADDERNET_REFERENCE_DIR", ""))
    ap.add_argument("--no-extension", action="store_true")
    a = ap.parse_args()
    if not a.reference or not Path(a.reference, "adder.py").exists():
        raise SystemExit("give the reference checkout with --reference or ADDERNET_REFERENCE_DIR")
    ref = Path(a.reference)
    install_python_files(ref)
    print("python files ->", DEST)
    if not a.no_extension:
        print("extension:", "built" if install_extension(ref) else "NOT built")


if __name__ == "__main__":
    main()
