"""Builds oracle/_ref/libref_kernels.so: the reference's OWN CUDA kernels (its header-only
device code, compiled from the reference checkout where it lies) behind the extern "C"
launchers of oracle/ref_kernels.cu, for sm_100a.  Checker only -- the product never loads
it.  Needs the reference checkout; on a GPU box the prebuilt file is used.

    python oracle/build_ref.py /path/to/reference

Without an argument the checkout is looked for in $SUPERL8_REFERENCE_ROOT and then in a
directory named ``reference`` beside this repository.
"""

import os
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
OUT_DIR = HERE / "_ref"
LIB = OUT_DIR / "libref_kernels.so"


def find_reference(reference_root=None):
    """The reference checkout: the argument, $SUPERL8_REFERENCE_ROOT, or ../reference; None if absent."""
    cands = [reference_root, os.environ.get("SUPERL8_REFERENCE_ROOT"), HERE.parent.parent / "reference"]
    for c in cands:
        if c and (Path(c) / "csrc" / "include").is_dir():
            return Path(c)
    return None


def build_ref(reference_root=None, force=False):
    root = find_reference(reference_root)
    if root is None:
        return None
    inc = root / "csrc" / "include"
    src = HERE / "ref_kernels.cu"
    if LIB.exists() and not force and LIB.stat().st_mtime > src.stat().st_mtime:
        return LIB
    OUT_DIR.mkdir(exist_ok=True)
    cmd = ["nvcc", "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-lineinfo",
           "-Xcompiler", "-fPIC", "-shared", "-I", str(inc), str(src), "-o", str(LIB)]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("reference kernel build failed:\n" + r.stdout + r.stderr)
    return LIB


if __name__ == "__main__":
    lib = build_ref(sys.argv[1] if len(sys.argv) > 1 else None, force=True)
    if lib is None:
        sys.exit("no reference checkout: pass its path or set SUPERL8_REFERENCE_ROOT")
    print(lib)
