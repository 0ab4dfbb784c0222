"""GPU parity tests of the host-buffer entry point (fftopk_select2048_host through
fast_topk_v3_host): same index sets as the oracle, only valid prefixes copied."""
import numpy as np
import pytest
import torch

import workloads
from jit_kernel.topk_indexer import fast_topk_v3_host, kernel_status
from oracle import topk_oracle as orc

pytestmark = pytest.mark.gpu
K = 2048


def _run(score, lengths, pinned=True, out=None):
    hs = score.pin_memory() if pinned else score
    hl = lengths.pin_memory() if pinned else lengths
    res = fast_topk_v3_host(hs, hl, K, out=out)
    torch.cuda.synchronize()
    assert not res.is_cuda
    return res.numpy()


@pytest.mark.parametrize("pinned", [True, False])
def test_ragged_batch_from_host_memory(pinned):
    s, ln = workloads.c3(B=16, L=50000)
    got = _run(s, ln, pinned)
    orc.check_result(s.numpy(), ln.numpy(), got, what=f"host ragged pinned={pinned}")
    assert kernel_status() == 0


def test_padding_in_host_memory_is_never_copied_or_read():
    s, ln = workloads.c3(B=8, L=30000)
    poisoned = s.clone()
    col = torch.arange(s.size(1)).unsqueeze(0)
    poisoned[col >= ln.unsqueeze(1)] = float("nan")  # NaN would win every comparison if it were read
    got = _run(poisoned, ln)
    orc.check_result(s.numpy(), ln.numpy(), got, what="host poisoned padding")


def test_full_rows_short_rows_strided_rows_and_given_output():
    g = torch.Generator().manual_seed(5)
    s = torch.randn(6, 9000, generator=g)
    ln = torch.tensor([9000, 9000, 0, 2048, 17, 9000], dtype=torch.int32)
    out = torch.full((6, K), -7, dtype=torch.int32).pin_memory()
    got = _run(s, ln, out=out)
    assert got.ctypes.data == out.numpy().ctypes.data
    orc.check_result(s.numpy(), ln.numpy(), got, what="host mixed rows")
    wide = torch.randn(4, 12000, generator=g)
    view = wide[:, 1000:11000]  # row stride 12000, 10000 columns
    ln2 = torch.tensor([10000, 5000, 2049, 9999], dtype=torch.int32)
    got = _run(view, ln2, pinned=False)
    orc.check_result(view.contiguous().numpy(), ln2.numpy(), got, what="host strided rows")


def test_two_calls_in_a_row_and_decode_row():
    s, ln = workloads.c2(L=300000)
    a = _run(s, ln).copy()
    b = _run(s, ln)
    orc.check_result(s.numpy(), ln.numpy(), a, what="host decode row")
    assert np.array_equal(np.sort(a, axis=1), np.sort(b, axis=1))


def test_argument_errors():
    s = torch.randn(2, 5000)
    ln = torch.full((2,), 5000, dtype=torch.int32)
    with pytest.raises(RuntimeError):
        fast_topk_v3_host(s.cuda(), ln, K)
    with pytest.raises(RuntimeError):
        fast_topk_v3_host(s.double(), ln, K)
    with pytest.raises(RuntimeError):
        fast_topk_v3_host(s, ln.long(), K)
    with pytest.raises(RuntimeError):
        fast_topk_v3_host(s, ln, K, out=torch.empty(2, 100, dtype=torch.int32))
