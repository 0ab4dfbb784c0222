"""CPU tests: the oracle's three statements agree with each other and with the golden vectors."""
import numpy as np
import pytest
import torch

from helpers import GOLDEN_NAMES, crc, load_golden
from oracle import topk_oracle as orc

K = 2048


@pytest.mark.parametrize("name", GOLDEN_NAMES)
def test_oracles_match_golden(name):
    score, lengths, rs, expected, value_crc = load_golden(name)
    s = score.numpy()
    ln = lengths.numpy()
    r = None if rs is None else rs.numpy()
    assert np.array_equal(orc.numpy_oracle(s, ln, K, r), expected)
    assert np.array_equal(orc.c_oracle(s, ln, K, r), expected)
    # torch.topk (the reference's ground truth) still yields the pinned value multiset
    _, vals = orc.torch_oracle(score, ln, K, r)
    for b, v in enumerate(vals):
        assert (0 if v is None else crc(v)) == int(value_crc[b])


def test_golden_set_is_complete():
    assert len(GOLDEN_NAMES) >= 7


def test_key_map_is_order_preserving():
    g = torch.Generator().manual_seed(1)
    x = torch.randn(20000, generator=g).numpy()
    x = np.concatenate([x, np.array([0.0, -0.0, np.inf, -np.inf, 1e-45, -1e-45, 3.4e38, -3.4e38], np.float32)])
    k = orc.keys_of(x)
    order = np.argsort(x, kind="stable")
    assert np.all(np.diff(k[order].astype(np.int64)) >= 0)
    # equal values <=> equal keys
    xs, ks = x[order], k[order]
    same_val = xs[1:] == xs[:-1]
    assert np.array_equal(same_val, ks[1:] == ks[:-1])
    # any MSB digit is monotone: bin(x) >= bin(y) whenever x >= y
    for bits in (8, 11, 12, 16):
        assert np.all(np.diff((ks >> np.uint32(32 - bits)).astype(np.int64)) >= 0)


def test_key_map_special_values():
    z = orc.keys_of(np.array([0.0, -0.0], np.float32))
    assert z[0] == z[1] == 0x80000000
    n = orc.keys_of(np.array([np.nan, -np.nan, np.inf], np.float32))
    assert n[0] == n[1] == 0xFFFFFFFF and n[2] == 0xFF800000
    for v in (0.0, -0.0, 1.5, -2.25, float("inf"), float("-inf"), float("nan"), 1e-42):
        assert orc.c_key_of(v) == int(orc.keys_of(np.array([v], np.float32))[0])


def test_short_rows_identity_layout():
    s = torch.randn(3, 4096)
    ln = np.array([0, 100, 2048])
    for fn in (orc.numpy_oracle, orc.c_oracle):
        out = fn(s.numpy(), ln, K)
        for b, n in enumerate(ln):
            assert np.array_equal(out[b, :n], np.arange(n))
            assert np.all(out[b, n:] == -1)


def test_tie_rule_is_lower_index():
    row = np.zeros(10000, np.float32)
    row[[5, 77, 9000]] = 1.0
    exp = np.sort(np.concatenate([[5, 77, 9000], np.setdiff1d(np.arange(10000), [5, 77, 9000])[:K - 3]]))
    assert np.array_equal(orc.numpy_topk_row(row), exp)
    assert np.array_equal(orc.c_oracle(row[None], [10000])[0], exp)
    idx, _ = orc.torch_oracle(torch.from_numpy(row)[None], [10000])
    assert np.array_equal(idx[0], exp)


def test_row_starts_and_clamping():
    g = torch.Generator().manual_seed(3)
    s = torch.randn(2, 6000, generator=g)
    ln = np.array([5000, 5900])
    rs = np.array([500, 300])  # second row: 300 + 5900 > 6000 -> clamped to 5700
    a = orc.numpy_oracle(s.numpy(), ln, K, rs)
    b = orc.c_oracle(s.numpy(), ln, K, rs)
    t, _ = orc.torch_oracle(s, ln, K, rs)
    assert np.array_equal(a, b) and np.array_equal(a, t)
    assert a[1].max() < 5700


def test_reference_floor_radix_scheme_agrees_on_its_domain():
    """The reference kernel's floor-bin selection (valid on [0,256)) picks the same set."""
    for seed, L in ((42, 16384), (43, 65536), (44, 120000)):
        g = torch.Generator().manual_seed(seed)
        x = torch.randn(L, generator=g)
        x = ((x - x.min()) / (x.max() - x.min() + 1e-6) * 255).numpy()  # bench_topk.py:101-104
        assert np.array_equal(orc.c_ref_floor_radix(x), orc.numpy_topk_row(x))


def test_checker_detects_a_wrong_pick():
    s, l = torch.randn(1, 5000), np.array([5000])
    good = orc.numpy_oracle(s.numpy(), l)
    orc.check_result(s, l, good)
    bad = good.copy()
    missing = np.setdiff1d(np.arange(5000), good[0])[0]
    bad[0, 0] = missing
    with pytest.raises(AssertionError):
        orc.check_result(s, l, bad)
