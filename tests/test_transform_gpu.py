"""GPU parity tests of the fused output transforms (the reference's fast_topk_transform_fused and
fast_topk_transform_ragged_fused, topk_indexer_radix.cu:871-995, 1160-1250): the value multiset of
every output row must equal the transform applied to the oracle's index set; short rows keep the
reference's exact layout."""
import numpy as np
import pytest
import torch

import workloads
from jit_kernel.topk_indexer import fast_topk_transform_fused, fast_topk_transform_ragged_fused, kernel_status
from oracle import topk_oracle as orc

pytestmark = pytest.mark.gpu
K = 2048
DEV = "cuda:0"


def _expected_rows(score, lengths, row_starts, transform):
    exp_idx = orc.numpy_oracle(score.numpy(), lengths.numpy(), K, None if row_starts is None else row_starts.numpy())
    rows = []
    for b in range(score.size(0)):
        n = min(max(int(lengths[b]), 0), K) if int(lengths[b]) <= K else K
        idx = exp_idx[b]
        vals = np.where(idx >= 0, transform(b, np.maximum(idx, 0)), -1)
        rows.append((vals, int(lengths[b]) <= K))
    return rows


def _check(got, rows):
    for b, (vals, short) in enumerate(rows):
        if short:
            assert np.array_equal(got[b], vals), f"short row {b}"
        else:
            assert np.array_equal(np.sort(got[b]), np.sort(vals)), f"row {b}"


def test_page_table_decode():
    score, lengths = workloads.c3(B=6, L=70000, min_len=500)
    lengths[0] = 1200
    g = torch.Generator().manual_seed(1)
    table = torch.stack([torch.randperm(70016, generator=g)[:70016] for _ in range(6)]).to(torch.int32)
    cu = torch.arange(7, dtype=torch.int32)
    got = fast_topk_transform_fused(score.to(DEV), lengths.to(DEV), table.to(DEV), cu.to(DEV), K).cpu().numpy()
    _check(got, _expected_rows(score, lengths, None, lambda b, idx: table[b].numpy()[idx]))
    assert kernel_status() == 0


def test_page_table_prefill_with_cu_seqlens_and_row_starts():
    g = torch.Generator().manual_seed(2)
    B, L = 7, 300000
    score = torch.randn(B, L, generator=g)
    lengths = torch.tensor([250000, 90000, 2048, 40000, 40001, 3000, 100], dtype=torch.int32)
    row_starts = torch.tensor([0, 5, 100, 7, 0, 1, 2], dtype=torch.int32)
    cu = torch.tensor([0, 3, 4, 7], dtype=torch.int32)  # three requests: rows 0-2, 3, 4-6
    table = torch.randint(0, 1 << 30, (3, L + 8), generator=g, dtype=torch.int32)[:, :L]  # strided view
    req = [0, 0, 0, 1, 2, 2, 2]
    got = fast_topk_transform_fused(score.to(DEV), lengths.to(DEV), table.to(DEV), cu.to(DEV), K,
                                    row_starts=row_starts.to(DEV)).cpu().numpy()
    _check(got, _expected_rows(score, lengths, row_starts, lambda b, idx: table[req[b]].numpy()[idx]))


def test_ragged_offsets():
    score, lengths = workloads.c4(B=4, L=131072)
    lengths = torch.tensor([131072, 50000, 2000, 131072], dtype=torch.int32)
    off = torch.tensor([0, 131072, 181072, 183072], dtype=torch.int32)
    got = fast_topk_transform_ragged_fused(score.to(DEV), lengths.to(DEV), off.to(DEV), K).cpu().numpy()
    _check(got, _expected_rows(score, lengths, None, lambda b, idx: idx + int(off[b])))
    rs = torch.tensor([3, 0, 1, 2], dtype=torch.int32)
    l2 = torch.tensor([100000, 50000, 2000, 131070], dtype=torch.int32)
    got = fast_topk_transform_ragged_fused(score.to(DEV), l2.to(DEV), off.to(DEV), K, row_starts=rs.to(DEV)).cpu().numpy()
    _check(got, _expected_rows(score, l2, rs, lambda b, idx: idx + int(off[b])))


def test_long_rows_through_the_sampled_path():
    score, lengths = workloads.c5(B=2, L=1 << 20)
    off = torch.tensor([7, 1 << 20], dtype=torch.int32)
    got = fast_topk_transform_ragged_fused(score.to(DEV), lengths.to(DEV), off.to(DEV), K).cpu().numpy()
    _check(got, _expected_rows(score, lengths, None, lambda b, idx: idx + int(off[b])))
