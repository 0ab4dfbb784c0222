"""CPU tests of the boundary: the C-ABI library loads and exports what include/fftopk.h declares,
and the Python op mirrors the reference's argument checking.  No kernel is launched here."""
import ctypes
import re
from pathlib import Path

import numpy as np
import pytest
import torch

from jit_kernel import _native
from jit_kernel.topk_indexer import fast_topk_v3
from oracle import topk_oracle as orc

REPO = Path(__file__).resolve().parent.parent


def declared_symbols():
    text = (REPO / "include" / "fftopk.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(fftopk_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    lib = _native.lib()
    names = declared_symbols()
    assert set(names) == set(_native.EXPORTS)
    for n in names:
        assert getattr(lib, n) is not None


def test_library_has_no_torch_dependency():
    import subprocess
    out = subprocess.run(["ldd", str(_native.LIB_PATH)], capture_output=True, text=True).stdout
    assert "torch" not in out and "c10" not in out


def test_version_and_strerror():
    lib = _native.lib()
    assert lib.fftopk_version() >= 100
    assert lib.fftopk_strerror(0) == b"ok"
    assert b"invalid" in lib.fftopk_strerror(-1)


def test_host_key_function_matches_oracle():
    lib = _native.lib()
    vals = [0.0, -0.0, 1.0, -1.0, 3.5, -7.25, float("inf"), float("-inf"), float("nan"), 1e-42, -1e-42]
    for v in vals:
        assert lib.fftopk_key_of(ctypes.c_float(v)) == int(orc.keys_of(np.array([v], np.float32))[0])


def test_argument_validation_without_a_device():
    lib = _native.lib()
    # null pointers / bad sizes are rejected before any CUDA call
    assert lib.fftopk_select2048(None, 0, 1, 10, None, None, None, None, 0, None, None) == -1
    assert lib.fftopk_select2048(None, 0, -1, 10, None, None, None, None, 0, None, None) == -1
    assert lib.fftopk_select2048(None, 0, 0, 10, None, None, None, None, 0, None, None) == 0  # B == 0: no-op
    assert lib.fftopk_merge2048(None, None, 0, 9, 1, None, None, None, None) == -4
    assert lib.fftopk_set_tuning(3, -1, -1, -1, 0) == -1
    assert lib.fftopk_set_tuning(-1, -1, -1, -1, 0) == 0


def test_python_op_mirrors_reference_assertions():
    s = torch.randn(2, 4096)
    ln = torch.full((2,), 4096, dtype=torch.int32)
    with pytest.raises(AssertionError):  # reference: topk must be 2048 (topk_indexer.py:62-64)
        fast_topk_v3(s, ln, 1024)
    with pytest.raises(AssertionError):  # reference: score.dim() == 2 (topk_indexer.py:65)
        fast_topk_v3(s[0], ln, 2048)
    with pytest.raises(RuntimeError):  # reference: CHECK_CUDA (topk_indexer_radix.cu:1049-1062)
        fast_topk_v3(s, ln, 2048)
