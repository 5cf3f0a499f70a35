"""In-tree build of the sm_100a shared library (``libsuperl8_b200.so``).

``python -m superl8_b200.build`` compiles every ``csrc/*.cu`` with nvcc for
``sm_100a`` and links one C-ABI shared library next to this file.  nvcc
cross-compiles, so no GPU is needed to build.  Objects are rebuilt only when a
source or header is newer than the object.

``python -m superl8_b200.build --trace [-DSL8_TRACE_BASE=n -DSL8_TRACE_STRIDE=m ...]`` builds a SECOND
library, ``libsuperl8_b200_trace.so`` (objects under ``csrc/build_trace``), with ``-DSL8_TRACE``: the
forward and backward tensor-memory kernels then stamp ``clock64()`` at the points marked ``TR(slot)``
in their sources for eight blocks of a launch (csrc/sl8_common.cuh), and the library exports
``sl8_dbg_read_trace`` / ``sl8_dbg_read_trace2`` / ``sl8_dbg_read_trace_bwd``.  ``superl8_b200.trace``
loads that library and reads the stamps back.  The shipped library never carries any of it.
"""

from __future__ import annotations

import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
CSRC = PKG_DIR / "csrc"
BUILD_DIR = PKG_DIR / "csrc" / "build"
LIB_PATH = PKG_DIR / "libsuperl8_b200.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
    "--expt-relaxed-constexpr",
]


def _nvcc() -> str:
    cand = os.environ.get("NVCC") or "/usr/local/cuda/bin/nvcc"
    return cand if os.path.exists(cand) else "nvcc"


def _newest_header_mtime() -> float:
    hdrs = list(CSRC.glob("*.cuh")) + [PKG_DIR.parent / "include" / "superl8_b200.h"]
    return max(h.stat().st_mtime for h in hdrs if h.exists())


TRACE_BUILD_DIR = PKG_DIR / "csrc" / "build_trace"
TRACE_LIB_PATH = PKG_DIR / "libsuperl8_b200_trace.so"


def build(force: bool = False, verbose: bool = False, trace: bool = False, defines=()) -> Path:
    """Compiles and links the library; ``trace=True`` builds the clock-stamp variant (always from
    scratch: its defines are not part of the staleness check) beside it."""
    build_dir, lib_path = (TRACE_BUILD_DIR, TRACE_LIB_PATH) if trace else (BUILD_DIR, LIB_PATH)
    extra = ["-DSL8_TRACE", *defines] if trace else list(defines)
    force = force or trace
    build_dir.mkdir(parents=True, exist_ok=True)
    sources = sorted(CSRC.glob("*.cu"))
    hdr_m = _newest_header_mtime()
    jobs = []
    objs = []
    for src in sources:
        obj = build_dir / (src.stem + ".o")
        objs.append(obj)
        stale = force or not obj.exists() or obj.stat().st_mtime < max(src.stat().st_mtime, hdr_m)
        if stale:
            cmd = [_nvcc(), *NVCC_FLAGS, *extra, "-c", str(src), "-o", str(obj)]
            if verbose:
                cmd.insert(1, "-Xptxas=-v")
            jobs.append(cmd)

    def run(cmd):
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("nvcc failed: " + " ".join(cmd) + "\n" + r.stdout + r.stderr)
        if verbose:
            sys.stderr.write(r.stderr)

    with ThreadPoolExecutor(max_workers=min(8, max(1, len(jobs)))) as ex:
        list(ex.map(run, jobs))

    relink = force or jobs or not lib_path.exists() or any(o.stat().st_mtime > lib_path.stat().st_mtime for o in objs)
    if relink:
        run([_nvcc(), "-shared", "-o", str(lib_path), *map(str, objs), "-gencode", "arch=compute_100a,code=sm_100a"])
    return lib_path


EXT_SRC = CSRC / "torch_ext" / "sl8_torch_ext.cpp"
EXT_NAME = "_C_ext"


def ext_path() -> Path:
    import sysconfig
    return PKG_DIR / (EXT_NAME + (sysconfig.get_config_var("EXT_SUFFIX") or ".so"))


def build_torch_ext(force: bool = False) -> Path:
    """Compiles the thin torch extension (csrc/torch_ext) with g++ against the installed torch and
    links it to libsuperl8_b200.so; the result sits beside the library (in-tree, nothing goes to a
    JIT cache).  Needs no GPU and no nvcc, only the CUDA headers torch's own headers include."""
    import sysconfig

    import torch
    from torch.utils import cpp_extension as ce

    out = ext_path()
    hdr = PKG_DIR.parent / "include" / "superl8_b200.h"
    if out.exists() and not force and out.stat().st_mtime > max(EXT_SRC.stat().st_mtime, hdr.stat().st_mtime):
        return out
    build()  # the extension links against the library
    cuda_home = os.environ.get("CUDA_HOME") or "/usr/local/cuda"
    incs = [*ce.include_paths(), sysconfig.get_paths()["include"], str(Path(cuda_home) / "include")]
    torch_lib = str(Path(torch.__file__).resolve().parent / "lib")
    cmd = [os.environ.get("CXX", "g++"), "-O2", "-std=c++17", "-fPIC", "-shared", "-fvisibility=hidden",
           f"-DTORCH_EXTENSION_NAME={EXT_NAME}", "-DTORCH_API_INCLUDE_EXTENSION_H",
           f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}",
           *[f"-I{i}" for i in incs], str(EXT_SRC), "-o", str(out),
           f"-L{torch_lib}", f"-L{PKG_DIR}", "-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch", "-ltorch_python",
           "-l:libsuperl8_b200.so",
           "-Wl,-rpath,$ORIGIN", f"-Wl,-rpath,{torch_lib}"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("torch extension build failed: " + " ".join(cmd) + "\n" + r.stdout + r.stderr)
    return out


if __name__ == "__main__":
    if "--trace" in sys.argv:
        print(build(trace=True, verbose="-v" in sys.argv, defines=[a for a in sys.argv[1:] if a.startswith("-D")]))
        sys.exit(0)
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
    if "--no-ext" not in sys.argv:
        print(build_torch_ext(force="--force" in sys.argv))
