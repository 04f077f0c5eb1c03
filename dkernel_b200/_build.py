"""In-tree build of libbsa_b200.so with nvcc for sm_100a.

``python -m dkernel_b200._build`` (or ``build()``) compiles every translation
unit under ``csrc/`` in parallel and links them into ``dkernel_b200/libbsa_b200.so``;
``--debug`` (``build(debug=True)``) makes the bounds-checking ``libbsa_b200_debug.so``.
Objects are cached under ``dkernel_b200/csrc/build/`` and rebuilt when the
source or any header is newer.  nvcc cross-compiles without a GPU.
"""
from __future__ import annotations

import concurrent.futures as cf
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(CSRC, "build")
LIB = os.path.join(HERE, "libbsa_b200.so")
LIB_DEBUG = os.path.join(HERE, "libbsa_b200_debug.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC",
]


def _nvcc() -> str:
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        raise RuntimeError("nvcc not found: cannot build libbsa_b200.so")
    return nvcc


def _sources():
    return sorted(f for f in os.listdir(CSRC) if f.endswith(".cu"))


def _headers_mtime() -> float:
    hs = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))]
    hs.append(os.path.join(HERE, "..", "include", "bsa.h"))
    return max(os.path.getmtime(h) for h in hs)


def _compile(nvcc: str, src: str, verbose: bool, extra, objdir: str = OBJ) -> str:
    obj = os.path.join(objdir, src[:-3] + ".o")
    srcp = os.path.join(CSRC, src)
    if os.path.exists(obj) and os.path.getmtime(obj) > max(os.path.getmtime(srcp), _headers_mtime()) \
            and not (verbose and extra):
        return obj
    cmd = [nvcc, *NVCC_FLAGS, *extra, "-c", srcp, "-o", obj]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if verbose or r.returncode != 0:
        sys.stderr.write(" ".join(cmd) + "\n" + r.stdout + r.stderr)
    if r.returncode != 0:
        raise RuntimeError(f"nvcc failed on {src}")
    return obj


def build(verbose: bool = False, extra_flags=(), debug: bool = False) -> str:
    """Release library, or with ``debug=True`` the bounds-checking build ``libbsa_b200_debug.so``
    (``-DBSA_DEBUG_BOUNDS``: index invariants checked in the kernels, violations recorded in the
    wait-status block, nothing traps).  Select it at run time with ``BSA_B200_LIB=<path>``."""
    objdir = OBJ + ("_debug" if debug else "")
    lib = LIB_DEBUG if debug else LIB
    os.makedirs(objdir, exist_ok=True)
    nvcc = _nvcc()
    srcs = _sources()
    flags = list(extra_flags) + (["-DBSA_DEBUG_BOUNDS"] if debug else [])
    with cf.ThreadPoolExecutor(max_workers=min(8, len(srcs))) as ex:
        objs = list(ex.map(lambda s: _compile(nvcc, s, verbose, flags, objdir), srcs))
    if os.path.exists(lib) and all(os.path.getmtime(lib) > os.path.getmtime(o) for o in objs):
        return lib
    cmd = [nvcc, "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", lib, *objs]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        sys.stderr.write(" ".join(cmd) + "\n" + r.stdout + r.stderr)
        raise RuntimeError(f"link of {os.path.basename(lib)} failed")
    return lib


if __name__ == "__main__":
    v = "-v" in sys.argv
    print(build(verbose=v, extra_flags=["-Xptxas", "-v"] if v else (), debug="--debug" in sys.argv))
