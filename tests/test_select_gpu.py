"""GPU parity tests: fast_topk_v3 (CUDA, through the C ABI) against the oracle, bit-exact.

Index sets must be identical (ties to the lower index), short rows must have the identity
layout.  Cases follow the benchmark configs plus the edge cases the reference's own check
exercises (row_starts, several batch sizes; benchmark/bench_topk.py:90-146)."""
import numpy as np
import pytest
import torch

import workloads
from helpers import GOLDEN_NAMES, load_golden
from jit_kernel import _native
from jit_kernel.topk_indexer import fast_topk, fast_topk_v3, kernel_status
from oracle import topk_oracle as orc

pytestmark = pytest.mark.gpu
K = 2048


def run(score, lengths, row_starts=None):
    dev = torch.device("cuda", 0)
    s = score.to(dev)
    ln = lengths.to(dev)
    rs = None if row_starts is None else row_starts.to(dev)
    out = fast_topk_v3(s, ln, K, row_starts=rs)
    torch.cuda.synchronize()
    return out.cpu().numpy()


def check(score, lengths, row_starts=None, expected=None, what=""):
    got = run(score, lengths, row_starts)
    orc.check_result(score.numpy(), lengths.numpy(), got,
                     None if row_starts is None else row_starts.numpy(), K, expected, what)
    assert kernel_status() == 0
    return got


@pytest.fixture(autouse=True)
def _reset_tuning():
    _native.set_tuning()
    yield
    _native.set_tuning()


@pytest.mark.parametrize("name", GOLDEN_NAMES)
def test_golden_vectors(name):
    score, lengths, rs, expected, _ = load_golden(name)
    check(score, lengths, rs, expected, name)


def test_c1_cpu_runnable_case():
    check(*workloads.c1(), what="c1")


@pytest.mark.parametrize("L", [65536, 131072, 262144, 524288, 1048576])
def test_c2_decode_sweep(L):
    check(*workloads.c2(L=L), what=f"c2 L={L}")


def test_c3_ragged_batch_full_size():
    score, lengths = workloads.c3()
    assert int(lengths.min()) < K < int(lengths.max())  # some rows take the -1 padded path
    check(score, lengths, what="c3")


def test_c4_tie_stress_full_size():
    score, lengths = workloads.c4()
    keys = orc.keys_of(score[0].numpy())
    t = np.sort(keys)[-K]
    assert (keys == t).sum() > 10000  # thousands of exact duplicates of the threshold value
    check(score, lengths, what="c4")


def test_c5_planted_tail_single_device():
    check(*workloads.c5(), what="c5")


@pytest.mark.parametrize("bs", [1, 2, 4, 8])
@pytest.mark.parametrize("seq_len", [16384, 65536, 98304, 120000])
@pytest.mark.parametrize("has_row_starts", [False, True])
def test_reference_benchmark_grid(bs, seq_len, has_row_starts):
    """The 32 configurations of the reference's calculate_diff (bench_topk.py:135-146), same
    recipe: randn min-max normalised to [0,255), optional random row_starts - but with zero
    tolerated wrong picks instead of five."""
    g = torch.Generator().manual_seed(42)
    L = 131072 if has_row_starts else seq_len
    s = torch.randn(bs, L, generator=g)
    s = (s - s.min()) / (s.max() - s.min() + 1e-6) * 255
    ln = torch.full((bs,), seq_len, dtype=torch.int32)
    rs = torch.randint(0, 2048, (bs,), generator=g, dtype=torch.int32) if has_row_starts else None
    check(s, ln, rs, what=f"grid bs={bs} L={seq_len} rs={has_row_starts}")


@pytest.mark.parametrize("cluster", [1, 2, 4, 8, 16])
@pytest.mark.parametrize("threads", [256, 512, 1024])
def test_every_cluster_size(cluster, threads):
    _native.set_tuning(cluster_ctas=cluster, threads=threads)
    g = torch.Generator().manual_seed(cluster * 10 + threads)
    s = torch.randn(3, 70001, generator=g)
    ln = torch.tensor([70001, 33333, 2049], dtype=torch.int32)
    check(s, ln, what=f"cluster={cluster} threads={threads}")
    if cluster <= 2:  # long rows on few CTAs: the sampled path, single-CTA shortcut included
        check(*workloads.c5(B=2, L=400000), what=f"cluster={cluster} threads={threads} long")


def test_overlapped_back_to_back_calls():
    """Programmatic dependent launch between consecutive calls (opt-in): same results."""
    dev = torch.device("cuda", 0)
    s, ln = workloads.c3(B=32, L=60000)
    bufs = [torch.roll(s, i, 0).contiguous().to(dev) for i in range(4)]
    lens = [torch.roll(ln, i, 0).contiguous().to(dev) for i in range(4)]
    outs = [torch.empty(32, K, dtype=torch.int32, device=dev) for _ in range(4)]
    _native.set_overlap(True)
    try:
        for rep in range(3):
            for i in range(4):
                fast_topk(bufs[i], outs[i], lens[i])
        torch.cuda.synchronize()
    finally:
        _native.set_overlap(False)
    for i in range(4):
        orc.check_result(torch.roll(s, i, 0).numpy(), torch.roll(ln, i, 0).numpy(), outs[i].cpu().numpy(),
                         what=f"overlap buffer {i}")


@pytest.mark.parametrize("cluster", [1, 4, 16])
def test_full_histogram_path(cluster):
    """The fallback that histograms the data itself (no sampling, no lists) on every config."""
    _native.set_tuning(cluster_ctas=cluster, force_full_histogram=True)
    check(*workloads.c2(L=131072), what=f"full-hist c2 C={cluster}")
    s, ln = workloads.c3(B=4, L=50000)
    check(s, ln, what=f"full-hist ragged C={cluster}")
    s, ln = workloads.c4(B=2, L=100000)
    check(s, ln, what=f"full-hist ties C={cluster}")


@pytest.mark.parametrize("list_cap", [32, 512])
def test_list_overflow_falls_back(list_cap):
    """A candidate list too small for what the filter admits must not lose elements."""
    _native.set_tuning(cluster_ctas=2, list_cap=list_cap)
    check(*workloads.c2(L=262144), what=f"list_cap={list_cap}")
    check(*workloads.c5(B=2, L=300000), what=f"list_cap={list_cap} tail")


def test_position_correlated_rows():
    """Sorted and locally clustered rows: the top k sit in one shard; sampling is by position."""
    L = 400000
    asc = torch.arange(L, dtype=torch.float32).unsqueeze(0) * 1e-3
    desc = asc.flip(1).contiguous()
    g = torch.Generator().manual_seed(21)
    bump = torch.randn(1, L, generator=g)
    bump[0, 123456:123456 + 3000] += 10.0  # all winners inside one 3000-element window
    saw = (torch.arange(L) % 4099).to(torch.float32).unsqueeze(0)
    s = torch.cat([asc, desc, bump, saw], dim=0)
    check(s, torch.full((4,), L, dtype=torch.int32), what="position-correlated")


@pytest.mark.parametrize("offset", [0, 1, 2, 3, 5])
def test_unaligned_rows(offset):
    """Row base addresses that are not 16-byte aligned, via views and row_starts."""
    g = torch.Generator().manual_seed(offset)
    big = torch.randn(3, 40000 + 8, generator=g)
    dev = torch.device("cuda", 0)
    view = big.to(dev)[:, offset:offset + 40000]  # stride 40008, base misaligned by `offset`
    ln = torch.tensor([40000, 39999, 2050], dtype=torch.int32)
    out = fast_topk_v3(view, ln.to(dev), K).cpu().numpy()
    orc.check_result(big[:, offset:offset + 40000].numpy(), ln.numpy(), out, what=f"view offset {offset}")
    rs = torch.tensor([offset, offset + 1, 7], dtype=torch.int32)
    ln2 = torch.tensor([30000, 30001, 30003], dtype=torch.int32)
    check(big, ln2, rs, what=f"row_starts offset {offset}")


def test_short_rows_and_exact_k():
    g = torch.Generator().manual_seed(5)
    s = torch.randn(6, 5000, generator=g)
    ln = torch.tensor([0, 1, 2047, 2048, 2049, 5000], dtype=torch.int32)
    got = check(s, ln, what="short rows")
    assert np.all(got[0] == -1)
    assert np.array_equal(got[3], np.arange(K))  # len == k takes the identity path (radix.cu:864)


def test_lengths_are_clamped_to_the_row():
    g = torch.Generator().manual_seed(6)
    s = torch.randn(2, 6000, generator=g)
    check(s, torch.tensor([9999, 6000], dtype=torch.int32), torch.tensor([100, 5000], dtype=torch.int32),
          what="clamp")


def test_padding_values_are_never_read():
    """Entries beyond lengths[b] must not influence the result, whatever they hold."""
    g = torch.Generator().manual_seed(8)
    s = torch.randn(2, 30000, generator=g)
    ln = torch.tensor([20000, 10001], dtype=torch.int32)
    a = run(s, ln)
    s2 = s.clone()
    s2[0, 20000:] = float("inf")
    s2[1, 10001:] = float("nan")
    b = run(s2, ln)
    assert np.array_equal(np.sort(a, axis=1), np.sort(b, axis=1))
    orc.check_result(s.numpy(), ln.numpy(), a)


def test_all_equal_row_takes_the_first_k():
    s = torch.full((2, 100000), 3.25)
    s[1] = 0.0
    got = check(s, torch.tensor([100000, 77777], dtype=torch.int32), what="all equal")
    assert np.array_equal(np.sort(got[0]), np.arange(K))


def test_two_values_with_ties_across_shards():
    s = torch.zeros(1, 300000)
    s[0, 7::1000] = 1.0  # 300 ones; 1748 zeros must come from the lowest indices
    check(s, torch.tensor([300000], dtype=torch.int32), what="two values")


def test_special_values():
    g = torch.Generator().manual_seed(9)
    s = torch.randn(1, 50000, generator=g)
    s[0, ::3] = 0.0
    s[0, 1::5] = -0.0
    s[0, 11::501] = float("inf")
    s[0, 13::499] = float("-inf")
    s[0, 17::1009] = float("nan")
    check(s, torch.tensor([50000], dtype=torch.int32), what="special")
    neg = -torch.rand(1, 40000, generator=g) * 1e-3 - 1.0  # all negative, narrow range
    check(neg, torch.tensor([40000], dtype=torch.int32), what="negative narrow")


@pytest.mark.parametrize("cap", [32, 256, 2048])
def test_small_candidate_capacity_forces_more_rounds(cap):
    """With a tiny candidate buffer the cluster has to refine on further key digits (and, for
    exact ties, take duplicates in index order) instead of handing survivors to rank 0."""
    _native.set_tuning(cluster_ctas=8, cand_cap=cap)
    check(*workloads.c2(L=262144), what=f"cap={cap} c2")
    s, ln = workloads.c4(B=2, L=131072)
    check(s, ln, what=f"cap={cap} c4")
    q = torch.round(torch.randn(1, 200000, generator=torch.Generator().manual_seed(cap)) * 8) / 8
    check(q, torch.tensor([200000], dtype=torch.int32), what=f"cap={cap} quantised")


def test_low_precision_logits_many_duplicates():
    """bf16-rounded logits: few distinct values, hundreds of ties at the threshold."""
    g = torch.Generator().manual_seed(10)
    s = torch.randn(4, 500000, generator=g).to(torch.bfloat16).to(torch.float32)
    check(s, torch.full((4,), 500000, dtype=torch.int32), what="bf16-rounded")


def test_noncontiguous_row_stride_and_zero_stride():
    g = torch.Generator().manual_seed(11)
    dev = torch.device("cuda", 0)
    big = torch.randn(8, 20000, generator=g)
    view = big.to(dev)[::2]  # stride 40000
    ln = torch.full((4,), 20000, dtype=torch.int32)
    out = fast_topk_v3(view, ln.to(dev), K).cpu().numpy()
    orc.check_result(big[::2].numpy(), ln.numpy(), out, what="stride 2 rows")
    row = torch.randn(1, 9000, generator=g)
    exp_view = row.to(dev).expand(3, 9000)  # stride 0
    out = fast_topk_v3(exp_view, torch.tensor([9000, 5000, 100], dtype=torch.int32, device=dev), K).cpu().numpy()
    orc.check_result(row.expand(3, 9000).numpy(), np.array([9000, 5000, 100]), out, what="stride 0")


def test_keys_output_and_index_offset():
    g = torch.Generator().manual_seed(12)
    dev = torch.device("cuda", 0)
    s = torch.randn(2, 30000, generator=g)
    ln = torch.tensor([30000, 1000], dtype=torch.int32)
    idx = torch.empty(2, K, dtype=torch.int32, device=dev)
    keys = torch.empty(2, K, dtype=torch.int32, device=dev)
    fast_topk(s.to(dev), idx, ln.to(dev), None, keys=keys, idx_offset=1000000)
    idx, keys = idx.cpu().numpy(), keys.cpu().numpy().view(np.uint32)
    all_keys = orc.keys_of(s.numpy().reshape(-1)).reshape(2, -1)
    for b in range(2):
        valid = idx[b] >= 0
        assert np.array_equal(keys[b][valid], all_keys[b][idx[b][valid] - 1000000])
        assert np.all(keys[b][~valid] == 0)
    unshifted = np.where(idx >= 0, idx - 1000000, -1)
    orc.check_result(s.numpy(), ln.numpy(), unshifted, what="offset")


def test_output_needs_no_prefill_and_is_deterministic_as_a_set():
    dev = torch.device("cuda", 0)
    s, ln = workloads.c3(B=16, L=40000)
    sd, ld = s.to(dev), ln.to(dev)
    out = torch.full((16, K), 12345, dtype=torch.int32, device=dev)
    fast_topk(sd, out, ld)
    a = out.cpu().numpy()
    orc.check_result(s.numpy(), ln.numpy(), a, what="prefilled with junk")
    for _ in range(3):
        b = fast_topk_v3(sd, ld, K).cpu().numpy()
        assert np.array_equal(np.sort(a, axis=1), np.sort(b, axis=1))


def test_large_batch_many_rows():
    """B >= number of SMs: the reference's launcher breaks there (split_kv == 1,
    topk_indexer_radix.cu:1081-1083); here it must simply work."""
    s, ln = workloads.c3(seed=3, B=200, L=9000, min_len=100)
    check(s, ln, what="B=200")


def test_cuda_graph_capture_and_replay():
    dev = torch.device("cuda", 0)
    s, ln = workloads.c3(B=8, L=60000)
    sd, ld = s.to(dev), ln.to(dev)
    out = torch.empty(8, K, dtype=torch.int32, device=dev)
    fast_topk(sd, out, ld)  # warm-up outside capture (first call sets function attributes)
    torch.cuda.synchronize()
    out.fill_(-7)
    graph = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        with torch.cuda.graph(graph, stream=side):
            fast_topk(sd, out, ld)
    graph.replay()
    torch.cuda.synchronize()
    orc.check_result(s.numpy(), ln.numpy(), out.cpu().numpy(), what="graph replay")


def _awkward_rows(L, seed):
    """Rows that stress the sampled path of a lone CTA: what the sample sees is not what decides."""
    g = torch.Generator().manual_seed(seed)
    rows = []
    base = torch.randn(L, generator=g)
    # windows of ~1900 winners at several offsets: some fall between the sampled slabs, so the
    # threshold lies above anything the sample suggested (the last bin of the finish's first digit)
    for off in (130, 777, 1500, 2300, 5000, 40001):
        off = min(off, L - 1900)
        r = base.clone()
        r[off:off + 1900] = 100.0 + torch.rand(1900, generator=g)
        rows.append(r)
    # the same with exact duplicates inside the window (ties decided by index)
    r = base.clone()
    r[3000:4900] = 50.0
    rows.append(r)
    # sum of weighted relu heads (one sign), bf16-rounded values (many ties), two values only
    heads = torch.relu(torch.randn(16, L, generator=g)) * torch.rand(16, 1, generator=g)
    rows.append(heads.sum(0))
    rows.append(base.to(torch.bfloat16).to(torch.float32))
    rows.append((torch.rand(L, generator=g) < 0.01).to(torch.float32))
    rows.append(torch.full((L,), 3.0))
    # sorted rows: every winner at one end
    rows.append(torch.arange(L, dtype=torch.float32) * 1e-3)
    rows.append(torch.arange(L, dtype=torch.float32).flip(0) * 1e-3)
    # negative values only, and a row whose winners straddle zero
    rows.append(-torch.rand(L, generator=g) - 1.0)
    r = -torch.rand(L, generator=g)
    r[::97] = torch.rand(r[::97].numel(), generator=g)
    rows.append(r)
    return torch.stack(rows).contiguous()


@pytest.mark.parametrize("L", [9000, 40000, 131072, 250000])
@pytest.mark.parametrize("overlap", [True, False])
def test_awkward_rows_in_both_launch_plans(L, overlap):
    """Throughput plan (one 512-thread CTA per row, finish over the warps' segments with a focused
    first digit) and default plan on rows whose sample is misleading."""
    s = _awkward_rows(L, seed=L)
    ln = torch.full((s.size(0),), L, dtype=torch.int32)
    ln[1] = L - 3
    ln[2] = L // 2 + 1
    pad = 64 - s.size(0) if overlap else 0  # the throughput plan uses one CTA per row from 38 rows on
    if pad:
        s = torch.cat([s, torch.randn(pad, L, generator=torch.Generator().manual_seed(L + 1))])
        ln = torch.cat([ln, torch.randint(2049, L + 1, (pad,), generator=torch.Generator().manual_seed(L + 2), dtype=torch.int32)])
    _native.set_overlap(overlap)
    try:
        if overlap:
            assert _native.plan(s.size(0), L)["cluster_ctas"] == 1
        check(s, ln, what=f"awkward rows L={L} overlap={overlap}")
    finally:
        _native.set_overlap(False)


@pytest.mark.parametrize("list_cap", [2304, 3072])
def test_lone_cta_segment_overflow(list_cap):
    """Warp segments too small for the candidates: the spill area, then the full-histogram path."""
    _native.set_tuning(cluster_ctas=1, threads=512, list_cap=list_cap)
    s, ln = workloads.c3(B=8, L=131072)
    check(s, ln, what=f"lone CTA list_cap={list_cap}")
    check(_awkward_rows(60000, 5), torch.full((15,), 60000, dtype=torch.int32), what=f"lone CTA awkward list_cap={list_cap}")
