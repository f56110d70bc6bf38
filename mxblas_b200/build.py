"""Build libmxblas_b200.so in-tree with nvcc for sm_100a.

The reference compiles one kernel per problem at run time (mxblas/jit/compiler.py:131-243, nvcc
per candidate configuration); here every kernel variant is compiled once, ahead of time, into one
shared library with a C ABI (include/mxblas_b200.h). nvcc cross-compiles without a GPU.

    python mxblas_b200/build.py [--force] [--verbose]
"""

from __future__ import annotations

import argparse
import hashlib
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
CSRC = PKG_DIR / "csrc"
OBJ_DIR = PKG_DIR / "build"
LIB_PATH = PKG_DIR / "libmxblas_b200.so"

SOURCES = [
    "mxb_host.cu",
    "mxb_hostmem.cu",
    "mxb_noalloc.cu",
    "mxb_quant.cu",
    "mxb_push.cu",
    "mxb_inst_epilogue.cu",
    "mxb_inst_promote.cu",
    "mxb_inst_mx.cu",
    "mxb_inst_pair.cu",
    "mxb_inst_quant2d.cu",
    "mxb_inst_general.cu",
    "mxb_inst_general_pair.cu",
]

NVCC_FLAGS = [
    "-gencode",
    "arch=compute_100a,code=sm_100a",
    "-lineinfo",
    "-O3",
    "-std=c++17",
    "-Xcompiler",
    "-fPIC",
]


def _nvcc() -> str:
    exe = os.environ.get("MXBLAS_NVCC_COMPILER") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found; set MXBLAS_NVCC_COMPILER")
    return exe


def _sources() -> list[str]:
    return [s for s in SOURCES if (CSRC / s).exists()]


def _fingerprint() -> str:
    h = hashlib.sha256()
    for path in sorted(CSRC.iterdir()) + [PKG_DIR.parent / "include" / "mxblas_b200.h"]:
        if path.suffix in (".cu", ".cuh", ".h"):
            h.update(path.name.encode())
            h.update(path.read_bytes())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compile (if sources changed) and return the path of the shared library."""
    OBJ_DIR.mkdir(exist_ok=True)
    stamp = OBJ_DIR / "fingerprint.txt"
    fp = _fingerprint()
    if not force and LIB_PATH.exists() and stamp.exists() and stamp.read_text() == fp:
        return LIB_PATH
    nvcc = _nvcc()
    extra = ["-Xptxas", "-v"] if verbose or os.environ.get("MXBLAS_PTXAS_VERBOSE") else []

    def compile_one(src: str) -> Path:
        obj = OBJ_DIR / (Path(src).stem + ".o")
        cmd = [nvcc, *NVCC_FLAGS, *extra, "-c", str(CSRC / src), "-o", str(obj)]
        if os.environ.get("MXBLAS_JIT_PRINT_NVCC_COMMAND"):
            print(" ".join(cmd), file=sys.stderr)
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"nvcc failed for {src}:\n{res.stdout}\n{res.stderr}")
        if extra:
            print(res.stderr, file=sys.stderr)
        return obj

    with ThreadPoolExecutor(max_workers=len(SOURCES)) as pool:
        objs = list(pool.map(compile_one, _sources()))
    cmd = [nvcc, "-shared", "-o", str(LIB_PATH), *map(str, objs)]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"link failed:\n{res.stdout}\n{res.stderr}")
    stamp.write_text(fp)
    return LIB_PATH


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    a = ap.parse_args()
    print(build(force=a.force, verbose=a.verbose))
