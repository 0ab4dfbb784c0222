"""Build libfftopk.so (the C-ABI library of the sm_100a top-2048 selector) with nvcc.

The library has no torch / ATen dependency, so a cold build takes seconds (the reference
JIT-compiles its pybind11 module against the ATen headers at first call,
jit_kernel/topk_indexer.py:24-39, which takes minutes).

Usage:  python build.py [--force] [--verbose]
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent
CSRC = ROOT / "csrc"
LIB_DIR = ROOT / "lib"
LIB_PATH = LIB_DIR / "libfftopk.so"
SOURCES = [CSRC / "fftopk_select.cu", CSRC / "fftopk_cp.cu", CSRC / "fftopk_hostio.cu"]
HEADERS = [CSRC / "fftopk_device.cuh", CSRC / "fftopk_key.h", CSRC / "fftopk_host.h", CSRC / "fftopk_trace.cuh",
           ROOT.parent / "include" / "fftopk.h"]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "-shared", "-Xcompiler", "-fPIC",
]


def find_nvcc() -> str | None:
    cand = os.environ.get("NVCC") or shutil.which("nvcc")
    if cand:
        return cand
    p = Path(os.environ.get("CUDA_HOME", "/usr/local/cuda")) / "bin" / "nvcc"
    return str(p) if p.exists() else None


def is_stale() -> bool:
    if not LIB_PATH.exists():
        return True
    built = LIB_PATH.stat().st_mtime
    return any(f.stat().st_mtime > built for f in SOURCES + HEADERS if f.exists())


def build_library(force: bool = False, verbose: bool = False, extra_flags: list[str] | None = None,
                  out: Path | None = None) -> Path:
    """Compile the library if it is missing or older than its sources; return its path."""
    out = Path(out) if out else LIB_PATH
    if out == LIB_PATH and not force and not is_stale():
        return out
    nvcc = find_nvcc()
    if nvcc is None:
        raise RuntimeError("nvcc not found: cannot build libfftopk.so (set NVCC or CUDA_HOME)")
    out.parent.mkdir(parents=True, exist_ok=True)
    cmd = [nvcc, *NVCC_FLAGS, *(extra_flags or []), "-o", str(out), *map(str, SOURCES)]
    if verbose:
        cmd[1:1] = ["-Xptxas", "-v"]
        print(" ".join(cmd), file=sys.stderr)
    res = subprocess.run(cmd, capture_output=True, text=True)
    if verbose or res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
    if res.returncode != 0:
        raise RuntimeError(f"nvcc failed with exit code {res.returncode}")
    return out


if __name__ == "__main__":
    path = build_library(force="--force" in sys.argv, verbose="--verbose" in sys.argv)
    print(path)
