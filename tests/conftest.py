import os
import sys
from pathlib import Path

import pytest

REPO = Path(__file__).resolve().parent.parent
PKG = REPO / "flash-float-jit-kernels_b200"
for p in (str(REPO), str(PKG)):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200 with -m gpu)")


def _has_cuda() -> bool:
    try:
        import torch
        return torch.cuda.is_available()
    except Exception:
        return False


def pytest_collection_modifyitems(config, items):
    if _has_cuda():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def golden_dir() -> Path:
    return REPO / "tests" / "golden"


def pytest_sessionfinish(session, exitstatus):
    """A checked build of the library (-DFFTOPK_CHECKED, chosen with FFTOPK_LIBRARY) keeps the first
    bound violation its kernels saw: print it, so that a failing status assertion can be traced."""
    if not os.environ.get("FFTOPK_LIBRARY") or not _has_cuda():
        return
    try:
        import ctypes

        from jit_kernel import _native
        lib = _native.lib()
        if hasattr(lib, "fftopk_checked_read"):
            rec = (ctypes.c_uint32 * 8)()
            if lib.fftopk_checked_read(rec) == 0:
                print(f"\nchecked build, first violation (site, index, limit, block): select {list(rec[:4])}, "
                      f"merge {list(rec[4:])}")
    except Exception as e:  # never turn a report into a failure
        print(f"\nchecked build: could not read the violation record: {e!r}")
