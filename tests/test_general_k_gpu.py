"""GPU parity tests of the general-k entry point (fftopk_select_topk through fast_topk_general):
k = 512, 1024, 4096 and odd values against the oracle, bit-exact, in both launch plans."""
import pytest
import torch

import workloads
from jit_kernel import _native
from jit_kernel.topk_indexer import fast_topk_general, fast_topk_v3, kernel_status
from oracle import topk_oracle as orc

pytestmark = pytest.mark.gpu


def _check(score, lengths, k, row_starts=None, what=""):
    dev = torch.device("cuda", 0)
    rs = None if row_starts is None else row_starts.to(dev)
    got = fast_topk_general(score.to(dev), lengths.to(dev), k, row_starts=rs)
    torch.cuda.synchronize()
    assert tuple(got.shape) == (score.size(0), k)
    orc.check_result(score.numpy(), lengths.numpy(), got.cpu().numpy(),
                     None if row_starts is None else row_starts.numpy(), k, None, what)
    assert kernel_status() == 0


@pytest.fixture(autouse=True)
def _reset():
    _native.set_tuning()
    _native.set_overlap(False)
    yield
    _native.set_tuning()
    _native.set_overlap(False)


@pytest.mark.parametrize("k", [1, 31, 512, 1024, 2048, 3000, 4096])
def test_decode_rows(k):
    for L in (20000, 300000):
        s, ln = workloads.c2(L=L)
        _check(s, ln, k, what=f"k={k} L={L}")


@pytest.mark.parametrize("k", [512, 1024, 4096])
@pytest.mark.parametrize("overlap", [False, True])
def test_ragged_batch(k, overlap):
    s, ln = workloads.c3(B=48, L=70000, min_len=100)
    _native.set_overlap(overlap)
    _check(s, ln, k, what=f"ragged k={k} overlap={overlap}")


@pytest.mark.parametrize("k", [512, 4096])
def test_ties_short_rows_and_row_starts(k):
    s, ln = workloads.c4(B=4, L=100000)
    _check(s, ln, k, what=f"ties k={k}")
    g = torch.Generator().manual_seed(k)
    s = torch.randn(5, 9000, generator=g)
    ln = torch.tensor([k, k - 1, k + 1, 0, 5000], dtype=torch.int32)
    rs = torch.tensor([0, 7, 100, 0, 4000], dtype=torch.int32)
    _check(s, ln, k, rs, what=f"short rows k={k}")
    eq = torch.full((2, 50000), 1.5)
    _check(eq, torch.tensor([50000, 4097], dtype=torch.int32), k, what=f"all equal k={k}")


@pytest.mark.parametrize("cluster", [1, 4, 16])
def test_every_path_with_k_4096(cluster):
    _native.set_tuning(cluster_ctas=cluster)
    s, ln = workloads.c5(B=2, L=200000)
    _check(s, ln, 4096, what=f"k=4096 C={cluster}")
    _native.set_tuning(cluster_ctas=cluster, force_full_histogram=True)
    _check(s, ln, 1024, what=f"k=1024 full-hist C={cluster}")


def test_same_as_the_fixed_entry_point_and_argument_errors():
    dev = torch.device("cuda", 0)
    s, ln = workloads.c3(B=8, L=30000)
    a = fast_topk_general(s.to(dev), ln.to(dev), 2048).cpu()
    b = fast_topk_v3(s.to(dev), ln.to(dev), 2048).cpu()
    assert torch.equal(a.sort(dim=1).values, b.sort(dim=1).values)
    with pytest.raises(ValueError):
        fast_topk_general(s.to(dev), ln.to(dev), 0)
    with pytest.raises(ValueError):
        fast_topk_general(s.to(dev), ln.to(dev), 4097)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("k", [512, 2048])
def test_16bit_scores(dtype, k):
    """fp16 / bf16 scores: same index set as the oracle on the widened values (many exact ties)."""
    dev = torch.device("cuda", 0)
    s, ln = workloads.c3(B=12, L=60000, min_len=100)
    s16 = s.to(dtype)
    got = fast_topk_general(s16.to(dev), ln.to(dev), k)
    torch.cuda.synchronize()
    orc.check_result(s16.to(torch.float32).numpy(), ln.numpy(), got.cpu().numpy(), None, k, None, f"{dtype} k={k}")
    # unaligned views, row_starts, a decode row
    wide = torch.randn(3, 50011, generator=torch.Generator().manual_seed(9)).to(dtype)
    view = wide[:, 3:50003]
    ln2 = torch.tensor([40000, 2049, 49990], dtype=torch.int32)
    rs = torch.tensor([5, 0, 9], dtype=torch.int32)
    got = fast_topk_general(wide.to(dev)[:, 3:50003], ln2.to(dev), k, row_starts=rs.to(dev))
    torch.cuda.synchronize()
    orc.check_result(view.to(torch.float32).contiguous().numpy(), ln2.numpy(), got.cpu().numpy(), rs.numpy(), k, None,
                     f"{dtype} k={k} row_starts")
    s1, l1 = workloads.c2(L=300000)
    got = fast_topk_general(s1.to(dtype).to(dev), l1.to(dev), k)
    torch.cuda.synchronize()
    orc.check_result(s1.to(dtype).to(torch.float32).numpy(), l1.numpy(), got.cpu().numpy(), None, k, None, f"{dtype} decode")
    assert kernel_status() == 0


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("cluster", [1, 2, 8, 16])
def test_16bit_every_path(dtype, cluster):
    """The 16-bit instantiation of the kernel on every path: register-resident and sampled rows,
    the full-histogram path, exact ties taken in index order, special values, every misalignment
    of the row start, rows of at most k elements."""
    dev = torch.device("cuda", 0)
    _native.set_tuning(cluster_ctas=cluster)
    try:
        g = torch.Generator().manual_seed(cluster)
        s = torch.randn(6, 90001, generator=g)
        s[0, ::3] = 0.0
        s[0, 1::5] = -0.0
        s[0, 11::501] = float("inf")
        s[0, 13::499] = float("-inf")
        s[0, 17::1009] = float("nan")
        s[1] = 2.5  # all equal: the first k indices win
        s[2, :] = (torch.arange(90001) % 97).to(torch.float32)  # 97 values, thousands of ties at the threshold
        ln = torch.tensor([90001, 80000, 70001, 2048, 2049, 300], dtype=torch.int32)
        s16 = s.to(dtype)
        for k in (2048, 100, 4096):
            got = fast_topk_general(s16.to(dev), ln.to(dev), k)
            torch.cuda.synchronize()
            orc.check_result(s16.to(torch.float32).numpy(), ln.numpy(), got.cpu().numpy(), None, k, None,
                             f"{dtype} C={cluster} k={k}")
        # long rows (the sampled path on every cluster size), bf16-/fp16-rounded heavy ties
        s1, l1 = workloads.c5(B=2, L=500000)
        got = fast_topk_general(s1.to(dtype).to(dev), l1.to(dev), 2048)
        orc.check_result(s1.to(dtype).to(torch.float32).numpy(), l1.numpy(), got.cpu().numpy(), None, 2048, None,
                         f"{dtype} C={cluster} long")
        # every misalignment of the row start relative to the 8-byte granule
        wide = torch.randn(2, 30016, generator=g).to(dtype)
        wd = wide.to(dev)
        for off in range(8):
            view = wd[:, off:off + 30000]
            ln3 = torch.tensor([30000, 29999 - off], dtype=torch.int32)
            got = fast_topk_general(view, ln3.to(dev), 2048)
            orc.check_result(wide[:, off:off + 30000].to(torch.float32).contiguous().numpy(), ln3.numpy(),
                             got.cpu().numpy(), None, 2048, None, f"{dtype} C={cluster} offset {off}")
        # the full-histogram path
        _native.set_tuning(cluster_ctas=cluster, force_full_histogram=True)
        got = fast_topk_general(s16.to(dev), ln.to(dev), 2048)
        orc.check_result(s16.to(torch.float32).numpy(), ln.numpy(), got.cpu().numpy(), None, 2048, None,
                         f"{dtype} C={cluster} full histogram")
        assert kernel_status() == 0
    finally:
        _native.set_tuning()
