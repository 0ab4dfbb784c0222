"""GPU tests of the fused indexer (fftopk_indexer_topk2048 / FusedIndexerTopk): logits computed on
the tensor cores and selected as they are produced.

Floating point: the logits are compared with the same formula in torch (fp32 arithmetic on the
widened bf16 operands) within 2e-5 relative to the row's largest magnitude - the tensor core
accumulates the 128-long dot products in fp32 in its own order. The selection is integer work and
must be bit-exact GIVEN the kernel's logits: the index set equals the oracle's on the logits the
kernel itself wrote, ties to the lower index, whether the row went through the selector (no guess)
or through the candidate filter in the producer's epilogue (guess from the previous call)."""
import numpy as np
import pytest
import torch

from jit_kernel import _native
from jit_kernel.indexer import FusedIndexerTopk, reference_logits
from jit_kernel.topk_indexer import _status_word, kernel_status
from oracle import topk_oracle as orc

pytestmark = pytest.mark.gpu
K = 2048
DEV = torch.device("cuda", 0)
LOGIT_RTOL = 2e-5


@pytest.fixture(autouse=True)
def _clean_status():
    _status_word(DEV).zero_()
    yield
    _status_word(DEV).zero_()


def make(B, L, seed, ties=False):
    g = torch.Generator(device="cpu").manual_seed(seed)
    q = torch.randn(B, 64, 128, generator=g).to(torch.bfloat16)
    k = torch.randn(B, L, 128, generator=g).to(torch.bfloat16)
    if ties:  # repeated keys give exactly equal logits: ties at the threshold are decided by index
        k[:, L // 2:] = k[:, :L - L // 2]
    w = torch.rand(B, 64, generator=g)
    return q.to(DEV), k.to(DEV), w.to(DEV)


def kth_keys(logits, lengths):
    out = []
    for b in range(logits.shape[0]):
        n = int(lengths[b])
        out.append(int(np.sort(orc.keys_of(logits[b, :n]))[-K]) if n > K else 0)
    return np.array(out, dtype=np.uint32)


# (1000 rows of 2200 keys: every producer CTA goes through several whole rows and finishes them;
#  1100 rows: more than the balanced split handles, one CTA per row)
@pytest.mark.parametrize("B,L", [(1, 4096), (3, 50000), (1, 300000), (8, 20000), (1000, 2200), (1100, 2500)])
def test_logits_match_torch_and_selection_is_exact(B, L):
    q, k, w = make(B, L, seed=B * 1000 + L)
    ln = torch.full((B,), L, dtype=torch.int32)
    if B > 1:
        ln[1] = L - 777      # a ragged tail inside the last tiles
        ln[-1] = 1500        # a row of fewer than k keys: -1 padded
    f = FusedIndexerTopk(B, L)
    out = f(q, k, w, ln.to(DEV))  # no guess yet: logits are written, the selector runs
    torch.cuda.synchronize()
    got = f.logits[:B, :L].cpu()
    ref = reference_logits(q, k, w).cpu()
    for b in range(B):
        n = int(ln[b])
        scale = float(ref[b, :n].abs().max())
        assert float((got[b, :n] - ref[b, :n]).abs().max()) <= LOGIT_RTOL * scale, f"row {b}: logits differ from torch"
    logits_np = got.numpy().copy()
    orc.check_result(logits_np, ln.numpy(), out.cpu().numpy(), what="cold")
    want = kth_keys(logits_np, ln.numpy())
    # what the selector hands back is the row's k-th largest key, or - where it could take a whole
    # bin without a finish, as in rows of barely more than k keys - a lower bound of it
    thr = f.thresholds.cpu().numpy().view(np.uint32)[:B]
    assert np.all(thr <= want) and np.array_equal(thr > 0, want > 0)
    if L > 4 * K:
        assert np.array_equal(thr, want)
    # the same inputs again: every row with more than k keys now has a guess and its logits are
    # filtered in the producer's epilogue (they are written all the same, and must be the same bits)
    f.logits.fill_(float("nan"))
    for rep in range(2):
        out = f(q, k, w, ln.to(DEV))
        torch.cuda.synchronize()
        orc.check_result(logits_np, ln.numpy(), out.cpu().numpy(), what=f"warm {rep}")
        assert np.array_equal(f.thresholds.cpu().numpy().view(np.uint32)[:B], want)
    again = f.logits[:B, :L].cpu().numpy()
    for b in range(B):
        n = int(ln[b])
        assert np.array_equal(again[b, :n].view(np.uint32), logits_np[b, :n].view(np.uint32)), f"row {b}: logits changed"
        assert np.isnan(again[b, n:]).all(), f"row {b}: written beyond the row's length"
    assert kernel_status(DEV) == 0


def test_decode_loop_grows_the_key_cache():
    """One key appended per step; thresholds carried along; every step exact on the step's logits."""
    B, L0, steps = 2, 30000, 6
    q, k, w = make(B, L0 + steps, seed=7)
    f = FusedIndexerTopk(B, L0 + steps)
    ref = reference_logits(q, k, w).cpu().numpy()  # close to the kernel's logits; exactness is checked on its own below
    for t in range(steps + 1):
        ln = torch.full((B,), L0 + t, dtype=torch.int32)
        out = f(q, k, w, ln.to(DEV))
        torch.cuda.synchronize()
        got = out.cpu().numpy()
        for b in range(B):
            # the k-th and (k+1)-th logits of these rows are far apart compared with the tolerance,
            # so the torch logits give the same set
            exp = orc.numpy_oracle(ref[b:b + 1, :L0 + t], np.array([L0 + t]), K)[0]
            assert np.array_equal(np.sort(got[b]), np.sort(exp)), f"step {t} row {b}"
    assert kernel_status(DEV) == 0


def test_exact_ties_and_guess_misses():
    B, L = 2, 40000
    q, k, w = make(B, L, seed=11, ties=True)
    ln = torch.full((B,), L, dtype=torch.int32)
    f = FusedIndexerTopk(B, L)
    out = f(q, k, w, ln.to(DEV))
    torch.cuda.synchronize()
    logits_np = f.logits[:B, :L].cpu().numpy().copy()
    assert np.array_equal(logits_np[:, :L // 2], logits_np[:, L // 2:])  # every logit occurs twice
    orc.check_result(logits_np, ln.numpy(), out.cpu().numpy(), what="ties cold")
    out = f(q, k, w, ln.to(DEV))
    torch.cuda.synchronize()
    orc.check_result(logits_np, ln.numpy(), out.cpu().numpy(), what="ties warm")
    assert kernel_status(DEV) == 0
    want = kth_keys(logits_np, ln.numpy())
    # guesses that do not hold: too high (fewer than k admitted) and far too low (the list overflows)
    for bad in (want + np.uint32(1 << 24), np.full(B, orc.keys_of(np.array([-1e30], np.float32))[0], np.uint32)):
        f.thresholds[:B] = torch.from_numpy(bad.view(np.int32).copy()).to(DEV)
        out = f(q, k, w, ln.to(DEV))
        torch.cuda.synchronize()
        orc.check_result(logits_np, ln.numpy(), out.cpu().numpy(), what="missed guess")
        assert kernel_status(DEV) & _native.ST_GUESS_MISSED
        assert np.array_equal(f.thresholds.cpu().numpy().view(np.uint32)[:B], want)
        _status_word(DEV).zero_()


def test_mixed_rows_in_one_call():
    """One call, six kinds of rows: guess holds; guess too high; guess far too low (the candidate list
    overflows); no guess; fewer than k keys; no key at all. Then the same call again (every row of
    more than k keys has an exact guess) and once more with a smaller batch on the same workspace."""
    B, L = 6, 45000
    q, k, w = make(B, L, seed=21)
    ln = torch.tensor([L, L - 5, L, L - 129, 1000, 0], dtype=torch.int32)
    f = FusedIndexerTopk(B, L)
    out = f(q, k, w, ln.to(DEV))
    torch.cuda.synchronize()
    logits_np = f.logits[:B, :L].cpu().numpy().copy()
    want = kth_keys(logits_np, ln.numpy())
    orc.check_result(logits_np, ln.numpy(), out.cpu().numpy(), what="cold")
    guesses = want.copy()
    guesses[1] = want[1] + np.uint32(1 << 24)
    guesses[2] = orc.keys_of(np.array([-1e30], np.float32))[0]
    guesses[3] = 0
    f.thresholds[:B] = torch.from_numpy(guesses.view(np.int32).copy()).to(DEV)
    f.logits.fill_(float("nan"))
    out = f(q, k, w, ln.to(DEV))
    torch.cuda.synchronize()
    orc.check_result(logits_np, ln.numpy(), out.cpu().numpy(), what="mixed")
    assert kernel_status(DEV) == _native.ST_GUESS_MISSED
    assert np.array_equal(f.thresholds.cpu().numpy().view(np.uint32)[:B], want)
    again = f.logits[:B, :L].cpu().numpy()
    for b in range(B):
        n = int(ln[b])
        assert np.array_equal(again[b, :n].view(np.uint32), logits_np[b, :n].view(np.uint32)) and np.isnan(again[b, n:]).all()
    _status_word(DEV).zero_()
    # every call leaves the rows' candidate and arrival counters at zero (the workspace is zero-filled once):
    # [B x 8192 composites][candidate counts][arrival counts][selector marks], each array padded to 256 bytes
    ws = f._ws[f._ws_ptr - f._ws.data_ptr():]
    count_off, pad = B * 8192 * 8, (B * 4 + 255) // 256 * 256
    assert int(ws[count_off:count_off + 2 * pad].to(torch.int32).abs().sum()) == 0
    for nb in (B, 3):
        out = f(q[:nb], k[:nb], w[:nb], ln[:nb].to(DEV))
        torch.cuda.synchronize()
        orc.check_result(logits_np[:nb], ln[:nb].numpy(), out.cpu().numpy(), what=f"again, {nb} rows")
    assert kernel_status(DEV) == 0


def test_random_ragged_batches():
    """Batches of random size and random lengths (empty rows, rows of fewer than k keys, rows that end
    inside a tile), three calls each - cold, warm, warm with some guesses spoilt - every row exact on
    the logits the kernel wrote. The producer's CTAs then cross row boundaries at arbitrary places."""
    rng = np.random.default_rng(5)
    for trial in range(10):
        B = int(rng.integers(1, 40))
        Lmax = int(rng.choice([3000, 9000, 30000]))
        q, k, w = make(B, Lmax, seed=100 + trial)
        kinds = rng.integers(0, 10, size=B)
        ln_np = np.where(kinds == 0, 0, np.where(kinds == 1, rng.integers(1, K + 1, size=B), rng.integers(K + 1, Lmax + 1, size=B)))
        ln = torch.from_numpy(ln_np.astype(np.int32))
        f = FusedIndexerTopk(B, Lmax)
        out = f(q, k, w, ln.to(DEV))
        torch.cuda.synchronize()
        logits_np = f.logits[:B, :Lmax].cpu().numpy().copy()
        orc.check_result(logits_np, ln.numpy(), out.cpu().numpy(), what=f"trial {trial} cold")
        want = kth_keys(logits_np, ln.numpy())
        out = f(q, k, w, ln.to(DEV))
        torch.cuda.synchronize()
        orc.check_result(logits_np, ln.numpy(), out.cpu().numpy(), what=f"trial {trial} warm")
        assert np.array_equal(f.thresholds.cpu().numpy().view(np.uint32)[:B], want)
        assert kernel_status(DEV) == 0
        spoilt = want.copy()
        for b in range(B):
            if want[b] and rng.random() < 0.4:
                spoilt[b] = want[b] + np.uint32(1 << 22) if rng.random() < 0.5 else np.uint32(1)
        f.thresholds[:B] = torch.from_numpy(spoilt.view(np.int32).copy()).to(DEV)
        out = f(q, k, w, ln.to(DEV))
        torch.cuda.synchronize()
        orc.check_result(logits_np, ln.numpy(), out.cpu().numpy(), what=f"trial {trial} spoilt guesses")
        # (rows that went through the selector may hand back a lower bound of their k-th key)
        thr = f.thresholds.cpu().numpy().view(np.uint32)[:B]
        assert np.all(thr <= want) and np.array_equal(thr > 0, want > 0)
        _status_word(DEV).zero_()


def test_graph_replay():
    B, L = 2, 60000
    q, k, w = make(B, L, seed=13)
    ln = torch.full((B,), L, dtype=torch.int32, device=DEV)
    f = FusedIndexerTopk(B, L)
    out = torch.empty(B, K, dtype=torch.int32, device=DEV)
    f(q, k, w, ln, out=out)  # first call outside the capture (kernel attributes), also seeds the thresholds
    torch.cuda.synchronize()
    logits_np = f.logits[:B, :L].cpu().numpy().copy()
    side = torch.cuda.Stream()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        with torch.cuda.graph(graph, stream=side):
            f(q, k, w, ln, out=out)
    for _ in range(3):
        out.fill_(-3)
        graph.replay()
        torch.cuda.synchronize()
        orc.check_result(logits_np, ln.cpu().numpy(), out.cpu().numpy(), what="indexer replay")
    assert kernel_status(DEV) == 0


def make_fp8(B, L, seed):
    g = torch.Generator(device="cpu").manual_seed(seed)
    q = (torch.randn(B, 64, 128, generator=g) * 0.5).to(torch.float8_e4m3fn)
    k = (torch.randn(B, L, 128, generator=g) * 0.5).to(torch.float8_e4m3fn)
    w = torch.rand(B, 64, generator=g)
    scale = torch.rand(B, L, generator=g) * 1.5 + 0.25  # positive per-key scales
    return q.to(DEV), k.to(DEV), w.to(DEV), scale.to(DEV)


@pytest.mark.parametrize("with_scale", [False, True])
# (70001 keys: a scale array whose rows are not 16-byte aligned - the scales are then loaded key by key
#  instead of travelling with the tiles)
@pytest.mark.parametrize("B,L", [(1, 4096), (2, 70000), (2, 70001), (1, 300000)])
def test_fp8_operands(B, L, with_scale):
    """fp8 (e4m3) q and key cache, optional per-key scale: logits against torch on the widened
    operands, selection exact on the kernel's own logits, cold and with a guess."""
    q, k, w, scale = make_fp8(B, L, seed=L + B)
    ks = scale if with_scale else None
    ln = torch.full((B,), L, dtype=torch.int32)
    if B > 1:
        ln[1] = L - 333
    f = FusedIndexerTopk(B, L)
    out = f(q, k, w, ln.to(DEV), k_scale=ks)
    torch.cuda.synchronize()
    got = f.logits[:B, :L].cpu()
    ref = reference_logits(q, k, w, ks).cpu()
    for b in range(B):
        n = int(ln[b])
        assert float((got[b, :n] - ref[b, :n]).abs().max()) <= LOGIT_RTOL * float(ref[b, :n].abs().max()), f"row {b}"
    logits_np = got.numpy().copy()
    orc.check_result(logits_np, ln.numpy(), out.cpu().numpy(), what="fp8 cold")
    for rep in range(2):
        out = f(q, k, w, ln.to(DEV), k_scale=ks)
        torch.cuda.synchronize()
        orc.check_result(logits_np, ln.numpy(), out.cpu().numpy(), what=f"fp8 warm {rep}")
    assert np.array_equal(f.thresholds.cpu().numpy().view(np.uint32)[:B], kth_keys(logits_np, ln.numpy()))
    assert kernel_status(DEV) == 0
