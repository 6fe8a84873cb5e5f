"""Builds libgeorefine_b200.so (host coder + CUDA kernels + C ABI) in-tree for sm_100a with nvcc.

    python -m georefine_b200.build [--force] [--verbose]

The library is written to georefine_b200/_build/ and is rebuilt when any source under csrc/ or include/ is
newer than it.  nvcc cross-compiles without a GPU.
"""
from __future__ import annotations

import shutil
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
OUT = PKG / "_build" / "libgeorefine_b200.so"
SOURCES = [CSRC / "capi.cu", CSRC / "bcx_host.cpp", CSRC / "bxr_build.cpp"]
FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "-Xcompiler", "-fPIC",
         "-Xcompiler", "-pthread", "-shared"]


def _inputs():
    return list(CSRC.glob("*")) + list((PKG.parent / "include").glob("*.h"))


def needs_build() -> bool:
    if not OUT.exists():
        return True
    stamp = OUT.stat().st_mtime
    return any(p.stat().st_mtime > stamp for p in _inputs())


def build(force: bool = False, verbose: bool = False) -> Path:
    if not force and not needs_build():
        return OUT
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(nvcc).exists():
        raise RuntimeError("nvcc not found: the CUDA library cannot be built here and no prebuilt copy is up to date")
    OUT.parent.mkdir(parents=True, exist_ok=True)
    cmd = [nvcc, *FLAGS, *(["-Xptxas", "-v"] if verbose else []), *map(str, SOURCES), "-o", str(OUT)]
    run = subprocess.run(cmd, capture_output=True, text=True)
    if verbose:
        sys.stderr.write(run.stderr)
    if run.returncode:
        raise RuntimeError("nvcc failed:\n" + run.stderr[-4000:])
    return OUT


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
