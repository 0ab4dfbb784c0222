"""GPU parity tests of the candidate merge (context-parallel mode) on ONE device: the G shards of
a row are selected one after the other with the index offset of their slice, stacked the way the
all-gather delivers them, and merged; the result must equal the single-device oracle."""
import numpy as np
import pytest
import torch

import workloads
from jit_kernel.distributed import _cuda_select, local_lengths, merge_candidates
from jit_kernel.topk_indexer import kernel_status
from oracle import topk_oracle as orc

pytestmark = pytest.mark.gpu
K = 2048


def cp_on_one_device(score, lengths, G):
    dev = torch.device("cuda", 0)
    B, L = score.shape
    Ls = L // G
    parts = []
    for g in range(G):
        shard = score[:, g * Ls:(g + 1) * Ls].contiguous().to(dev)
        parts.append(_cuda_select(shard, local_lengths(lengths, Ls, g).to(dev), g * Ls))
    out = merge_candidates(torch.stack(parts).contiguous())
    torch.cuda.synchronize()
    return out.cpu().numpy()


@pytest.mark.parametrize("G", [2, 4, 8])
def test_c5_context_parallel_shards(G):
    score, lengths = workloads.c5(B=2, L=1 << 20)
    got = cp_on_one_device(score, lengths, G)
    orc.check_result(score.numpy(), lengths.numpy(), got, what=f"cp G={G}")
    assert kernel_status() == 0


@pytest.mark.parametrize("G", [2, 8])
def test_ties_across_shards_go_to_the_lower_global_index(G):
    score, lengths = workloads.c4(B=2, L=131072)
    got = cp_on_one_device(score, lengths, G)
    orc.check_result(score.numpy(), lengths.numpy(), got, what=f"cp ties G={G}")


def test_ragged_global_lengths_and_short_rows():
    g = torch.Generator().manual_seed(31)
    score = torch.randn(4, 32768, generator=g)
    lengths = torch.tensor([32768, 9000, 2048, 700], dtype=torch.int32)  # shards partly / fully empty
    got = cp_on_one_device(score, lengths, 4)
    exp = orc.numpy_oracle(score.numpy(), lengths.numpy(), K)
    for b in range(4):
        n = min(int(lengths[b]), K)
        assert np.array_equal(np.sort(got[b][got[b] >= 0]), np.sort(exp[b][exp[b] >= 0])), b
        assert (got[b] >= 0).sum() == n
        assert np.all(got[b][n:] == -1)  # -1 padding at the end
