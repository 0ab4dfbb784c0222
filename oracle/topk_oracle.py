"""CPU oracle for the top-2048 selector.  TEST INFRASTRUCTURE ONLY.

Only tests/, ``__graft_entry__.smoke()`` and the CPU-baseline / reference legs of ``bench.py``
import this module; the product (``jit_kernel.topk_indexer``) never does and has no CPU path.

Three independent statements of the same contract live here and are checked against each other
and against the golden vectors in tests/golden:

* ``torch_oracle``  - the reference's own ground truth, ``torch.topk(score[:, :len], k,
  sorted=False)`` (benchmark/bench_topk.py:25-42), for the value multiset, plus
  ``torch.sort(descending=True, stable=True)[:k]`` for the index set (stable => the lower index
  first among equal values, the tie rule this build fixes; torch.topk leaves ties unspecified).
* ``numpy_oracle``  - composite-key partition: key = order-preserving uint32 map of the fp32
  bits (the map the reference defines as convert_to_uint32,
  jit_kernel/csrc/topk_indexer/topk_indexer_radix.cu:206-209), composite = key << 32 | ~index.
* ``c_oracle``      - oracle/topk_oracle.c through ctypes (build: ``make -C oracle``).

Parity status: pinned.  The reference ships no golden vectors for this path
(benchmark/bench_topk.py:90-132 compares against torch.topk at run time), so the pins are
torch.topk / stable-sort outputs generated in this image by tests/golden/make_golden.py.
"""
from __future__ import annotations

import ctypes
import subprocess
from pathlib import Path
from typing import Optional

import numpy as np

K = 2048
_HERE = Path(__file__).resolve().parent
_C_LIB = _HERE / "_build" / "libtopk_oracle.so"


# ----------------------------------------------------------------------------------------------
# key map (numpy)
# ----------------------------------------------------------------------------------------------
def keys_of(x: np.ndarray) -> np.ndarray:
    """Order-preserving uint32 keys of an fp32 array (-0.0 -> +0.0, NaN -> 0xFFFFFFFF)."""
    bits = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32).copy()
    nan = (bits & np.uint32(0x7FFFFFFF)) > np.uint32(0x7F800000)
    bits[bits == np.uint32(0x80000000)] = 0
    neg = (bits & np.uint32(0x80000000)) != 0
    keys = np.where(neg, ~bits, bits | np.uint32(0x80000000)).astype(np.uint32)
    keys[nan] = np.uint32(0xFFFFFFFF)
    return keys


def _row_bounds(L: int, length: int, row_start: int) -> tuple[int, int]:
    rs = min(max(int(row_start), 0), L)
    ln = min(max(int(length), 0), L - rs)
    return rs, ln


def identity_row(length: int, k: int = K) -> np.ndarray:
    """Rows with len <= k: 0..len-1 then -1 (topk_indexer_radix.cu:152-163)."""
    out = np.full(k, -1, dtype=np.int32)
    out[:length] = np.arange(length, dtype=np.int32)
    return out


# ----------------------------------------------------------------------------------------------
# numpy restatement
# ----------------------------------------------------------------------------------------------
def numpy_topk_row(row: np.ndarray, k: int = K) -> np.ndarray:
    """Sorted indices of the k largest entries of `row` under (value desc, index asc)."""
    n = row.shape[0]
    if n <= k:
        return identity_row(n, k)
    comp = (keys_of(row).astype(np.uint64) << np.uint64(32)) | \
        (np.uint64(0xFFFFFFFF) - np.arange(n, dtype=np.uint64))
    part = np.argpartition(comp, n - k)[n - k:]
    return np.sort(part).astype(np.int32)


def numpy_oracle(score: np.ndarray, lengths, k: int = K, row_starts=None) -> np.ndarray:
    """[B, k] expected indices; rows with len > k are sorted ascending, short rows are exact."""
    score = np.asarray(score, dtype=np.float32)
    B, L = score.shape
    out = np.empty((B, k), dtype=np.int32)
    for b in range(B):
        rs, ln = _row_bounds(L, lengths[b], 0 if row_starts is None else row_starts[b])
        out[b] = numpy_topk_row(score[b, rs:rs + ln], k)
    return out


# ----------------------------------------------------------------------------------------------
# torch ground truth (the reference's own)
# ----------------------------------------------------------------------------------------------
def torch_oracle(score, lengths, k: int = K, row_starts=None):
    """Returns (indices [B,k] int32 numpy, values list) using torch on CPU.

    values[b] is torch.topk's value multiset (sorted descending) or None for short rows;
    indices come from a stable descending sort and are asserted to carry the same values.
    """
    import torch

    score = torch.as_tensor(score, dtype=torch.float32).cpu()
    B, L = score.shape
    idx_out = np.empty((B, k), dtype=np.int32)
    vals_out = []
    for b in range(B):
        rs, ln = _row_bounds(L, int(lengths[b]), 0 if row_starts is None else int(row_starts[b]))
        if ln <= k:
            idx_out[b] = identity_row(ln, k)
            vals_out.append(None)
            continue
        x = score[b, rs:rs + ln]
        tv = torch.topk(x, k, dim=-1, sorted=False).values  # bench_topk.py:33
        order = torch.sort(x, descending=True, stable=True).indices[:k]
        sv = x[order]
        tv_sorted = torch.sort(tv, descending=True).values
        if not torch.equal(torch.nan_to_num(tv_sorted, nan=3e38), torch.nan_to_num(sv, nan=3e38)):
            raise AssertionError("stable-sort oracle disagrees with torch.topk on the value multiset")
        idx_out[b] = np.sort(order.numpy()).astype(np.int32)
        vals_out.append(tv_sorted.numpy())
    return idx_out, vals_out


# ----------------------------------------------------------------------------------------------
# C restatement through ctypes
# ----------------------------------------------------------------------------------------------
def build_c_oracle() -> Path:
    subprocess.run(["make", "-s", "-C", str(_HERE)], check=True)
    return _C_LIB


def _c_lib() -> ctypes.CDLL:
    if not _C_LIB.exists():
        build_c_oracle()
    lib = ctypes.CDLL(str(_C_LIB))
    lib.oracle_topk.restype = ctypes.c_int
    lib.oracle_topk.argtypes = [ctypes.c_void_p, ctypes.c_int64, ctypes.c_int32, ctypes.c_int64,
                                ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int32, ctypes.c_void_p]
    lib.oracle_ref_floor_radix.restype = ctypes.c_int
    lib.oracle_ref_floor_radix.argtypes = [ctypes.c_void_p, ctypes.c_int32, ctypes.c_int32,
                                           ctypes.c_int32, ctypes.c_void_p]
    lib.oracle_key_of.restype = ctypes.c_uint32
    lib.oracle_key_of.argtypes = [ctypes.c_float]
    return lib


def c_oracle(score: np.ndarray, lengths, k: int = K, row_starts=None) -> np.ndarray:
    """oracle_topk from topk_oracle.c; rows with len > k are returned sorted ascending."""
    score = np.ascontiguousarray(score, dtype=np.float32)
    B, L = score.shape
    lengths = np.ascontiguousarray(lengths, dtype=np.int32)
    rs = None if row_starts is None else np.ascontiguousarray(row_starts, dtype=np.int32)
    out = np.empty((B, k), dtype=np.int32)
    rc = _c_lib().oracle_topk(score.ctypes.data, L, B, L, lengths.ctypes.data,
                              None if rs is None else rs.ctypes.data, k, out.ctypes.data)
    if rc != 0:
        raise MemoryError("oracle_topk failed")
    for b in range(B):
        _, ln = _row_bounds(L, lengths[b], 0 if rs is None else rs[b])
        if ln > k:
            out[b] = np.sort(out[b])
    return out


def c_ref_floor_radix(row: np.ndarray, k: int = K, max_rounds: int = 4) -> np.ndarray:
    """The reference kernel's floor-bin scheme (valid for inputs in [0,256)); sorted indices."""
    row = np.ascontiguousarray(row, dtype=np.float32)
    out = np.empty(k, dtype=np.int32)
    n = _c_lib().oracle_ref_floor_radix(row.ctypes.data, row.shape[0], k, max_rounds, out.ctypes.data)
    if n != k:
        raise AssertionError(f"oracle_ref_floor_radix wrote {n} of {k}")
    return np.sort(out) if row.shape[0] > k else out


def c_key_of(x: float) -> int:
    return int(_c_lib().oracle_key_of(ctypes.c_float(x)))


# ----------------------------------------------------------------------------------------------
# the checker tests and smoke() use on a CUDA result
# ----------------------------------------------------------------------------------------------
def check_result(score_cpu, lengths_cpu, got_indices, row_starts_cpu=None, k: int = K,
                 expected: Optional[np.ndarray] = None, what: str = "") -> None:
    """Bit-exact comparison of a [B,k] index result with the oracle.

    Rows with len > k are compared as index SETS (the op's order is unspecified); short rows must
    match the identity layout exactly.  Raises AssertionError naming the first differing row.
    """
    score_np = np.asarray(score_cpu, dtype=np.float32)
    lengths_np = np.asarray(lengths_cpu, dtype=np.int64)
    rs_np = None if row_starts_cpu is None else np.asarray(row_starts_cpu, dtype=np.int64)
    got = np.asarray(got_indices, dtype=np.int32)
    B, L = score_np.shape
    assert got.shape == (B, k), f"{what}: result shape {got.shape} != {(B, k)}"
    exp = numpy_oracle(score_np, lengths_np, k, rs_np) if expected is None else expected
    for b in range(B):
        _, ln = _row_bounds(L, lengths_np[b], 0 if rs_np is None else rs_np[b])
        g = got[b] if ln <= k else np.sort(got[b])
        if not np.array_equal(g, exp[b]):
            extra = np.setdiff1d(g, exp[b])[:8]
            missing = np.setdiff1d(exp[b], g)[:8]
            raise AssertionError(
                f"{what}: row {b} (len {ln}) differs from the oracle: "
                f"{np.count_nonzero(~np.isin(g, exp[b]))} wrong; extra {extra}, missing {missing}")
