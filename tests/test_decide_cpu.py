"""CPU tests of the selector's decision rules. The kernels take every guess / fall-back decision
through csrc/fftopk_decide.h; here the same header is compiled by g++ and driven with generated
inputs, and a numpy restatement of the sampled attempt (sample -> histogram -> rank bound -> key
guess -> float edge -> filter -> keep-or-fall-back) is run end to end on the host:

  * whatever the data and the sample, the attempt is either abandoned or admits a superset of the
    true top k; on i.i.d. rows it is practically never abandoned and admits few extras;
  * finish digits are monotone over the candidate range, stay inside the bin count, agree between
    the key-only and the full form, and bin ranges tile the range;
  * the fused indexer's work split visits every tile of every row exactly once, whatever the rows'
    lengths and the number of CTAs, and no CTA gets more than one tile more than another.
"""
import ctypes
import subprocess
from pathlib import Path

import numpy as np
import pytest
from hypothesis import given, settings, strategies as st

from oracle import topk_oracle as orc

REPO = Path(__file__).resolve().parent.parent
CSRC = REPO / "flash-float-jit-kernels_b200" / "csrc"
K = 2048
u32, u64, f32, i32 = ctypes.c_uint32, ctypes.c_uint64, ctypes.c_float, ctypes.c_int


@pytest.fixture(scope="module")
def dh(tmp_path_factory):
    out = tmp_path_factory.mktemp("decide") / "libdecide.so"
    subprocess.run(["g++", "-O2", "-std=c++17", "-shared", "-fPIC", "-I", str(CSRC), "-o", str(out),
                    str(REPO / "tests" / "decide_harness.cpp")], check=True)
    lib = ctypes.CDLL(str(out))
    sigs = {
        "dh_key_from_bits": (u32, [u32]), "dh_bits_from_key": (u32, [u32]),
        "dh_sample_lower_rank": (u32, [u32, u32, f32]), "dh_sample_upper_rank": (u32, [u32, u32, f32]),
        "dh_sample_bin_too_coarse": (i32, [u32, u32, f32, u32, f32]),
        "dh_fine_histogram_usable": (i32, [i32, u32, u32]),
        "dh_guess_key": (u32, [i32, u32, u32]), "dh_guess_edge_bits": (u32, [u32]), "dh_guess_low_key": (u32, [u32]),
        "dh_sampled_attempt_ok": (i32, [u32, u32, u32, u32]),
        "dh_finish_bins": (i32, []), "dh_finish_shift": (i32, [u64, u64]), "dh_finish_key_only": (i32, [u64, u64]),
        "dh_finish_digit": (u32, [u64, u64, u64]), "dh_finish_digit_of_key": (u32, [u64, u64, u32]),
        "dh_finish_bin_range": (None, [u64, u64, u64, i32, ctypes.POINTER(u64), ctypes.POINTER(u64)]),
        "dh_single_key_floor": (u64, [u64, i32]),
        "dh_walk_tile_split": (i32, [ctypes.c_void_p, i32, u32, ctypes.c_void_p, ctypes.c_void_p]),
        "dh_tile_run": (None, [u32, u32, u32, ctypes.POINTER(u32), ctypes.POINTER(u32)]),
    }
    for name, (res, args) in sigs.items():
        getattr(lib, name).restype = res
        getattr(lib, name).argtypes = args
    return lib


def test_host_key_map_is_the_oracles(dh):
    vals = np.array([0.0, -0.0, 1.0, -1.0, 3.5, np.inf, -np.inf, np.nan, 1e-42, -1e-42, 255.0], np.float32)
    for v, k in zip(vals.view(np.uint32), orc.keys_of(vals)):
        assert dh.dh_key_from_bits(int(v)) == int(k)
        if not np.isnan(np.array([v], np.uint32).view(np.float32)[0]) and int(v) != 0x80000000:
            assert dh.dh_bits_from_key(int(k)) == int(v)


def test_rank_bounds_bracket_the_expected_rank(dh):
    for n_s in (2048, 8192, 16384, 65536):
        for length in (n_s, 3 * n_s, 40 * n_s):
            m = K * n_s / length
            lo, hi = dh.dh_sample_lower_rank(K, n_s, length), dh.dh_sample_upper_rank(K, n_s, length)
            assert lo <= n_s and lo >= min(n_s, int(m))
            assert hi <= m and (hi == 0 or hi >= 1)
            assert hi < lo


def _edge_admits(dh, row, gkey):
    """The filter's test, !(x < edge), and the claim it stands for: key(x) >= low key of the guess."""
    edge = np.array([dh.dh_guess_edge_bits(gkey)], np.uint32).view(np.float32)[0]
    with np.errstate(invalid="ignore"):
        admitted = ~(row < edge)
    assert np.array_equal(admitted, orc.keys_of(row) >= np.uint32(dh.dh_guess_low_key(gkey)))
    return admitted


def sampled_attempt(dh, row, positions, k=K, room=1 << 30):
    """numpy restatement of one sampled attempt; returns (kept, admitted mask)."""
    keys = orc.keys_of(row)
    sample = keys[positions]
    n_s, length = sample.size, float(row.size)
    need = dh.dh_sample_lower_rank(k, n_s, length)
    hist_a = np.bincount(sample >> 20, minlength=4096)
    # the finer histogram applies when one value of the top four key bits holds the whole sample
    nib = np.bincount(sample >> 28, minlength=16)
    fine = bool(dh.dh_fine_histogram_usable(1, n_s, int(nib.max())))
    hist = np.bincount((sample >> 16) & 0xFFF, minlength=4096) if fine else hist_a
    suffix = np.cumsum(hist[::-1])[::-1]  # elements in bins >= b
    if need == 0 or suffix[0] < need:
        return False, None
    t = int(np.nonzero(suffix >= need)[0].max())
    gkey = dh.dh_guess_key(int(fine), int(nib.argmax()), t)
    pbits = 16 if fine else 12
    if dh.dh_sample_bin_too_coarse(int(hist[t]), n_s, length, k, 2.0):
        rem = need - (int(suffix[t + 1]) if t + 1 < 4096 else 0)
        sb = 32 - pbits - 12
        inside = sample[(sample >> (32 - pbits)) == (gkey >> (32 - pbits))]
        h2 = np.bincount((inside >> sb) & 0xFFF, minlength=4096)
        s2 = np.cumsum(h2[::-1])[::-1]
        if s2[0] < rem:
            return False, None
        gkey |= int(np.nonzero(s2 >= rem)[0].max()) << sb
    admitted = _edge_admits(dh, row, gkey)
    return bool(dh.dh_sampled_attempt_ok(0, int(admitted.sum()), k, room)), admitted


def _rows(rng, length):
    heads = np.maximum(rng.standard_normal((16, length)), 0).astype(np.float32) * rng.random((16, 1), np.float32)
    yield "normal", rng.standard_normal(length).astype(np.float32)
    yield "relu heads", heads.sum(0, dtype=np.float32)
    yield "lognormal+zeros", np.where(rng.random(length) < 0.7, 0, np.exp(rng.standard_normal(length))).astype(np.float32)
    yield "bf16-rounded", (rng.standard_normal(length).astype(np.float32).view(np.uint32) & 0xFFFF0000).view(np.float32)
    yield "all negative", (-rng.random(length) - 1).astype(np.float32)
    yield "sorted", np.sort(rng.standard_normal(length)).astype(np.float32)
    yield "all equal", np.full(length, 2.5, np.float32)
    yield "specials", np.where(rng.random(length) < 0.01, np.nan, np.where(rng.random(length) < 0.01, -np.inf,
                               rng.standard_normal(length))).astype(np.float32)
    r = rng.standard_normal(length).astype(np.float32)
    r[1000:2900] += 100  # a window of winners the sample may miss entirely
    yield "window", r


@pytest.mark.parametrize("length,n_s", [(9000, 8192), (40000, 8192), (131072, 8192), (1 << 20, 16384)])
def test_sampled_attempt_is_a_superset_or_is_abandoned(dh, length, n_s):
    rng = np.random.default_rng(length)
    for name, row in _rows(rng, length):
        for slab_sampling in (True, False):
            if slab_sampling:  # what the kernel does: evenly spaced runs of 128 elements
                starts = (np.arange(n_s // 128) * (length // (n_s // 128)))[:, None]
                pos = np.minimum(starts + np.arange(128)[None, :], length - 1).reshape(-1)
            else:
                pos = rng.choice(length, n_s, replace=False)
            kept, admitted = sampled_attempt(dh, row, pos)
            if not kept:
                continue  # the kernel falls back to full histograms: always exact
            top = orc.numpy_oracle(row[None, :], np.array([length]), K)[0]
            assert admitted[top].all(), f"{name}: a true winner was filtered out although the attempt was kept"
            assert admitted.sum() >= K


def test_sampled_attempt_is_rarely_abandoned_on_iid_rows(dh):
    rng = np.random.default_rng(7)
    abandoned, extra = 0, []
    for _ in range(300):
        row = rng.standard_normal(65536).astype(np.float32)
        kept, admitted = sampled_attempt(dh, row, rng.choice(row.size, 8192, replace=False))
        abandoned += 0 if kept else 1
        if kept:
            extra.append(int(admitted.sum()) - K)
    assert abandoned == 0
    assert np.median(extra) < 2 * K  # the safety margin costs a bounded number of extra candidates


def test_abandon_conditions(dh):
    assert dh.dh_sampled_attempt_ok(0, K, K, 4096) == 1
    assert dh.dh_sampled_attempt_ok(0, K - 1, K, 4096) == 0  # guess too high
    assert dh.dh_sampled_attempt_ok(1, 3000, K, 4096) == 0   # a list overflowed
    assert dh.dh_sampled_attempt_ok(0, 5000, K, 4096) == 0   # more than the gather buffer holds


comp = st.integers(min_value=0, max_value=(1 << 64) - 1)


@settings(max_examples=400, deadline=None)
@given(a=comp, b=comp, c=comp, d=comp, e=comp)
def test_finish_digit_is_monotone_and_bounded(dh, a, b, c, d, e):
    lo, x, y, focus, cap = sorted((a, b, c, d, e))
    if focus < x:  # keep lo <= focus <= cap with two probes anywhere in [lo, cap]
        focus = cap
    nb = dh.dh_finish_bins()
    dx, dy = dh.dh_finish_digit(lo, focus, x), dh.dh_finish_digit(lo, focus, y)
    assert dx <= dy < nb
    assert dh.dh_finish_digit(lo, focus, lo) == 0
    # everything up to the focus stays below the last bin unless the range is that narrow
    if focus - lo >= nb:
        assert dh.dh_finish_digit(lo, focus, focus) <= nb - 2
    # the bin of a composite contains it, and consecutive bins tile [lo, cap]
    t_lo, t_hi = u64(), u64()
    dh.dh_finish_bin_range(lo, focus, cap, dx, ctypes.byref(t_lo), ctypes.byref(t_hi))
    assert t_lo.value <= x <= t_hi.value <= cap
    if dx + 1 < nb and t_hi.value < cap:
        n_lo, n_hi = u64(), u64()
        dh.dh_finish_bin_range(lo, focus, cap, dx + 1, ctypes.byref(n_lo), ctypes.byref(n_hi))
        assert n_lo.value == t_hi.value + 1


@settings(max_examples=300, deadline=None)
@given(k0=st.integers(0, (1 << 32) - 1), k1=st.integers(0, (1 << 32) - 1), k2=st.integers(0, (1 << 32) - 1),
       low=st.integers(0, (1 << 32) - 1))
def test_key_only_digit_agrees_with_the_full_digit(dh, k0, k1, k2, low):
    klo, k, kfocus = sorted((k0, k1, k2))
    lo, focus = klo << 32, (kfocus << 32) | 0xFFFFFFFF
    if dh.dh_finish_key_only(lo, focus):
        assert dh.dh_finish_digit_of_key(lo, focus, k) == dh.dh_finish_digit(lo, focus, (k << 32) | low)
    else:
        assert dh.dh_finish_shift(lo, focus) < 32


def test_single_key_floor(dh):
    lo = 0x12345678 << 32
    f = dh.dh_single_key_floor(lo, 17)
    assert f >> 32 == 0x12345678 and (f & 0xFFFFFFFF) == 0xFFFE0000
    assert dh.dh_single_key_floor(lo, 32) == lo


# ---- work split of the fused indexer's producer ---------------------------------------------------
def _walk(dh, tiles_per_row, ctas):
    first = np.concatenate([[0], np.cumsum(tiles_per_row)]).astype(np.uint32)
    visits = np.zeros(int(first[-1]) + 1, dtype=np.uint32)
    segs = np.zeros(ctas, dtype=np.uint32)
    rc = dh.dh_walk_tile_split(first.ctypes.data, len(tiles_per_row), ctas, visits.ctypes.data, segs.ctypes.data)
    return rc, first, visits, segs


@settings(max_examples=200, deadline=None)
@given(st.lists(st.integers(0, 2100), min_size=1, max_size=300), st.integers(1, 600))
def test_tile_split_visits_every_tile_once(dh, tiles_per_row, ctas):
    rc, first, visits, segs = _walk(dh, tiles_per_row, ctas)
    assert rc == 0
    total = int(first[-1])
    assert np.all(visits[:total] == 1) and visits[total] == 0
    # a CTA's segments: at most one per row it touches, and none for a CTA without tiles
    sizes = []
    for c in range(ctas):
        g0, g1 = u32(), u32()
        dh.dh_tile_run(total, ctas, c, ctypes.byref(g0), ctypes.byref(g1))
        sizes.append(g1.value - g0.value)
        assert (segs[c] == 0) == (g1.value == g0.value)
    assert sum(sizes) == total and max(sizes) - min(sizes) <= 1


def test_tile_split_edge_cases(dh):
    # no tile at all; one row; rows without tiles at both ends and in the middle; more CTAs than tiles
    for tiles, ctas in (([0], 296), ([0, 0, 0], 5), ([8192], 296), ([1], 296), ([0, 5, 0, 0, 7, 0], 3),
                        ([3] * 1024, 296), ([2048] * 64, 296), ([1, 1, 1], 296)):
        rc, first, visits, segs = _walk(dh, tiles, ctas)
        assert rc == 0
        assert np.all(visits[:int(first[-1])] == 1)
