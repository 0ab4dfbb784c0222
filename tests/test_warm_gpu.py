"""GPU parity tests of the warm start (fftopk_select2048_warm / fast_topk_v3_warm): whatever the
guess - exact, stale, too high, too low, none - the index set equals the oracle's, ties included,
and the threshold the call hands back is the key of the row's k-th largest element."""
import numpy as np
import pytest
import torch

import workloads
from jit_kernel import _native
from jit_kernel.topk_indexer import _status_word, fast_topk_v3_warm, kernel_status
from oracle import topk_oracle as orc

pytestmark = pytest.mark.gpu
K = 2048
DEV = torch.device("cuda", 0)


@pytest.fixture(autouse=True)
def _reset():
    _native.set_tuning()
    _native.set_overlap(False)
    _status_word(DEV).zero_()
    yield
    _native.set_tuning()
    _status_word(DEV).zero_()


def kth_keys(score, lengths):
    """Key of every row's k-th largest valid element (0 for rows of at most k elements)."""
    out = []
    for b in range(score.size(0)):
        n = int(lengths[b])
        keys = orc.keys_of(score[b, :n].numpy())
        out.append(int(np.sort(keys)[-K]) if n > K else 0)
    return np.array(out, dtype=np.uint32)


def run(score, lengths, thr, margin=0, row_starts=None):
    out = fast_topk_v3_warm(score.to(DEV), lengths.to(DEV), K, thr, margin=margin,
                            row_starts=None if row_starts is None else row_starts.to(DEV))
    torch.cuda.synchronize()
    return out.cpu().numpy()


def as_i32(keys_u32):
    return torch.from_numpy(np.asarray(keys_u32, dtype=np.uint32).view(np.int32).copy()).to(DEV)


@pytest.mark.parametrize("case", ["c2_1m", "c2_128k", "c3", "c5", "c4_ties", "bf16"])
def test_cold_then_warm_matches_oracle_and_returns_the_kth_key(case):
    if case == "c2_1m":
        score, lengths = workloads.c2(L=1 << 20)
    elif case == "c2_128k":
        score, lengths = workloads.c2(L=131072, B=3)
    elif case == "c3":
        score, lengths = workloads.c3(B=24, L=90000, min_len=1000)
    elif case == "c5":
        score, lengths = workloads.c5(B=4, L=1 << 19)
    elif case == "c4_ties":
        score, lengths = workloads.c4(B=4, L=262144)
    else:
        g = torch.Generator().manual_seed(3)
        score = torch.randn(2, 300000, generator=g).to(torch.bfloat16).to(torch.float32)
        lengths = torch.full((2,), 300000, dtype=torch.int32)
    B = score.size(0)
    want = kth_keys(score, lengths)
    thr = torch.zeros(B, dtype=torch.int32, device=DEV)
    got = run(score, lengths, thr)  # no guess: the cold path, which hands back a threshold
    orc.check_result(score.numpy(), lengths.numpy(), got, what=f"{case} cold")
    first = thr.cpu().numpy().view(np.uint32)
    assert np.all(first <= want), "a threshold above the k-th key would lose winners next time"
    for rep in range(3):  # warm: the guess is the previous call's threshold
        got = run(score, lengths, thr)
        orc.check_result(score.numpy(), lengths.numpy(), got, what=f"{case} warm {rep}")
        now = thr.cpu().numpy().view(np.uint32)
        assert np.array_equal(now, want), f"{case}: threshold after a warm call is not the k-th key"
    assert kernel_status(DEV) == 0  # no guess was missed


def test_decode_loop_row_grows_by_one_logit_per_step():
    """The intended use: the same row, one logit appended per step, thresholds carried along."""
    L0, steps = 200000, 12
    g = torch.Generator().manual_seed(11)
    score = torch.randn(2, L0 + steps, generator=g)
    score[0, L0 + 3] = 50.0   # a new maximum arrives
    score[1, L0 + 5] = -50.0  # a new minimum arrives
    sd = score.to(DEV)
    thr = torch.zeros(2, dtype=torch.int32, device=DEV)
    for t in range(steps + 1):
        lengths = torch.full((2,), L0 + t, dtype=torch.int32)
        out = fast_topk_v3_warm(sd, lengths.to(DEV), K, thr)
        torch.cuda.synchronize()
        orc.check_result(score.numpy(), lengths.numpy(), out.cpu().numpy(), what=f"decode step {t}")
        assert np.array_equal(thr.cpu().numpy().view(np.uint32), kth_keys(score, lengths))
    assert kernel_status(DEV) == 0


@pytest.mark.parametrize("how", ["too_high", "too_low", "stale_other_row", "garbage"])
def test_bad_guesses_cost_time_not_correctness(how):
    score, lengths = workloads.c2(L=262144, B=4)
    want = kth_keys(score, lengths)
    if how == "too_high":
        guess = want + np.uint32(1 << 22)          # admits fewer than k
    elif how == "too_low":
        guess = np.full(4, orc.keys_of(np.array([-1.0], np.float32))[0], np.uint32)  # admits everything
    elif how == "stale_other_row":
        other, ol = workloads.c5(B=4, L=262144)    # thresholds of unrelated rows (N(0,1) with a tail)
        guess = kth_keys(other, ol)
    else:
        guess = np.array([1, 0xFFFFFFFF, 0x7F800000, 0x00000002], np.uint32)
    thr = as_i32(guess)
    got = run(score, lengths, thr)
    orc.check_result(score.numpy(), lengths.numpy(), got, what=f"guess {how}")
    after = thr.cpu().numpy().view(np.uint32)
    assert np.all(after <= want) and np.all(after > 0)
    got = run(score, lengths, thr)  # the handed-back thresholds are usable again
    orc.check_result(score.numpy(), lengths.numpy(), got, what=f"guess {how}, next call")
    assert np.array_equal(thr.cpu().numpy().view(np.uint32), want)
    if how in ("too_high", "too_low"):
        assert kernel_status(DEV) & _native.ST_GUESS_MISSED
        _status_word(DEV).zero_()


def test_margin_covers_a_threshold_that_dropped():
    """New logits every step (not an append): the threshold moves a little both ways; a margin of
    2^16 key units keeps the old guess usable."""
    g = torch.Generator().manual_seed(5)
    base = torch.rand(1, 400000, generator=g) * 8 + 1
    thr = torch.zeros(1, dtype=torch.int32, device=DEV)
    lengths = torch.full((1,), 400000, dtype=torch.int32)
    for t in range(6):
        score = base + 0.001 * torch.randn(1, 400000, generator=g)
        got = run(score, lengths, thr, margin=1 << 16)
        orc.check_result(score.numpy(), lengths.numpy(), got, what=f"margin step {t}")
    assert kernel_status(DEV) == 0


def test_short_rows_row_starts_and_mixed_guesses():
    g = torch.Generator().manual_seed(8)
    score = torch.randn(5, 60000, generator=g)
    lengths = torch.tensor([60000 - 9, 2048, 100, 30000, 2049], dtype=torch.int32)
    rs = torch.tensor([9, 0, 5, 1000, 3], dtype=torch.int32)
    thr = torch.zeros(5, dtype=torch.int32, device=DEV)
    for rep in range(3):
        got = run(score, lengths, thr, row_starts=rs)
        orc.check_result(score.numpy(), lengths.numpy(), got, rs.numpy(), K, None, f"row_starts warm {rep}")
    t = thr.cpu().numpy().view(np.uint32)
    assert t[1] == 0 and t[2] == 0 and t[0] != 0 and t[3] != 0


@pytest.mark.parametrize("overlap", [False, True])
def test_both_launch_plans_and_graph_replay(overlap):
    """Throughput plan (one CTA per row) and the default plan, replayed as a CUDA graph with the
    thresholds living on the device between replays."""
    score, lengths = workloads.c3(B=64, L=70000, min_len=1500)
    sd, ld = score.to(DEV), lengths.to(DEV)
    thr = torch.zeros(64, dtype=torch.int32, device=DEV)
    out = torch.empty(64, K, dtype=torch.int32, device=DEV)
    _native.set_overlap(overlap)
    try:
        fast_topk_v3_warm(sd, ld, K, thr, out=out)  # cold, outside the capture
        torch.cuda.synchronize()
        side = torch.cuda.Stream()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.stream(side):
            with torch.cuda.graph(graph, stream=side):
                fast_topk_v3_warm(sd, ld, K, thr, out=out)
        for _ in range(3):
            out.fill_(-3)
            graph.replay()
            torch.cuda.synchronize()
            orc.check_result(score.numpy(), lengths.numpy(), out.cpu().numpy(), what=f"warm replay overlap={overlap}")
    finally:
        _native.set_overlap(False)
    assert np.array_equal(thr.cpu().numpy().view(np.uint32), kth_keys(score, lengths))
    assert kernel_status(DEV) == 0
