"""Build libfftopk.so (the C-ABI library of the sm_100a top-2048 selector) with nvcc.

The library has no torch / ATen dependency, so a cold build takes seconds (the reference
JIT-compiles its pybind11 module against the ATen headers at first call,
jit_kernel/topk_indexer.py:24-39, which takes minutes).

Usage:  python build.py [--force] [--verbose]
"""
from __future__ import annotations

import contextlib
import fcntl
import os
import shutil
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent
CSRC = ROOT / "csrc"
LIB_DIR = ROOT / "lib"
LIB_PATH = LIB_DIR / "libfftopk.so"
SOURCES = [CSRC / "fftopk_select.cu", CSRC / "fftopk_cp.cu", CSRC / "fftopk_hostio.cu", CSRC / "fftopk_indexer.cu"]
HEADERS = [CSRC / "fftopk_device.cuh", CSRC / "fftopk_key.h", CSRC / "fftopk_host.h", CSRC / "fftopk_trace.cuh",
           CSRC / "fftopk_internal.h", CSRC / "fftopk_decide.h", CSRC / "fftopk_merge.cuh", ROOT.parent / "include" / "fftopk.h"]

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


CHECKED_LIB_PATH = LIB_DIR / "libfftopk_checked.so"


def is_stale(path: Path = LIB_PATH) -> bool:
    if not path.exists():
        return True
    built = path.stat().st_mtime
    return any(f.stat().st_mtime > built for f in SOURCES + HEADERS if f.exists())


@contextlib.contextmanager
def build_lock():
    """One builder at a time across processes (the ranks of a multi-GPU job all import the package)."""
    LIB_DIR.mkdir(parents=True, exist_ok=True)
    with open(LIB_DIR / ".build.lock", "w") as f:
        fcntl.flock(f, fcntl.LOCK_EX)
        try:
            yield
        finally:
            fcntl.flock(f, fcntl.LOCK_UN)


def build_library(force: bool = False, verbose: bool = False, extra_flags: list[str] | None = None,
                  out: Path | None = None) -> Path:
    """Compile the library if it is missing or older than its sources; return its path.

    Safe when several processes call it at once: builders take turns under a file lock (the second
    one finds the library fresh and returns), and the library appears under its name by an atomic
    rename, so a process that is loading it never sees a half-written file."""
    out = Path(out) if out else LIB_PATH
    if not force and not is_stale(out):
        return out
    nvcc = find_nvcc()
    if nvcc is None:
        raise RuntimeError("nvcc not found: cannot build libfftopk.so (set NVCC or CUDA_HOME)")
    out.parent.mkdir(parents=True, exist_ok=True)
    with build_lock():
        if not force and not is_stale(out):
            return out  # another process built it while this one waited for the lock
        tmp = out.with_name(f".{out.name}.{os.getpid()}.tmp")
        cmd = [nvcc, *NVCC_FLAGS, *(extra_flags or []), "-o", str(tmp), *map(str, SOURCES)]
        if verbose:
            cmd[1:1] = ["-Xptxas", "-v"]
            print(" ".join(cmd), file=sys.stderr)
        res = subprocess.run(cmd, capture_output=True, text=True)
        if verbose or res.returncode != 0:
            sys.stderr.write(res.stdout + res.stderr)
        if res.returncode != 0:
            with contextlib.suppress(OSError):
                tmp.unlink()
            raise RuntimeError(f"nvcc failed with exit code {res.returncode}")
        os.replace(tmp, out)
    return out


def build_checked_library(force: bool = False) -> Path:
    """The same library with -DFFTOPK_CHECKED: every index the selection logic guarantees to be in
    range is tested on the device, a failing test raises FFTOPK_ST_CHECK in the status word and
    leaves a record for fftopk_checked_read(). Point FFTOPK_LIBRARY at it to run anything on it."""
    return build_library(force=force, extra_flags=["-DFFTOPK_CHECKED"], out=CHECKED_LIB_PATH)


if __name__ == "__main__":
    if "--checked" in sys.argv:
        print(build_checked_library(force="--force" in sys.argv))
    else:
        print(build_library(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
