"""Build recipe for libint8kv_b200.so (nvcc, sm_100a only).

The shared library is built in-tree next to this file so that it travels with a copy of the
repository; it is never installed into site-packages.  `python -m` style use:

    python int8-kvcache_b200/build.py            # build if sources are newer than the library
    python int8-kvcache_b200/build.py --force
"""

from __future__ import annotations

import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
CSRC = PKG_DIR / "csrc"
LIB_PATH = PKG_DIR / "libint8kv_b200.so"
SOURCES = ["c_api.cu", "cache_write.cu", "paged_attn.cu"]
HEADERS = ["common.cuh", "kernels.h", "../../include/int8kv_b200.h"]

NVCC_FLAGS = [
    "-gencode",
    "arch=compute_100a,code=sm_100a",
    "-O3",
    "-std=c++17",
    "-lineinfo",
    "--shared",
    "-Xcompiler",
    "-fPIC",
    "--cudart",
    "static",
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    raise RuntimeError("nvcc not found; set NVCC or put it on PATH")


def sources() -> list:
    return [CSRC / s for s in SOURCES if (CSRC / s).exists()]


def is_stale() -> bool:
    if not LIB_PATH.exists():
        return True
    built = LIB_PATH.stat().st_mtime
    deps = sources() + [CSRC / h for h in HEADERS]
    return any(d.exists() and d.stat().st_mtime > built for d in deps)


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compile the CUDA sources into libint8kv_b200.so; returns the library path."""
    if not force and not is_stale():
        return LIB_PATH
    cmd = [_nvcc(), *NVCC_FLAGS]
    if verbose:
        cmd += ["-Xptxas", "-v"]
    cmd += [str(s) for s in sources()] + ["-o", str(LIB_PATH)]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError("nvcc failed:\n" + " ".join(cmd) + "\n" + proc.stdout + proc.stderr)
    if verbose:
        sys.stderr.write(proc.stdout + proc.stderr)
    return LIB_PATH


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose="-v" in sys.argv)
    print(path)
