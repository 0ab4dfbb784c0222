"""GPU test of fftopk_topk2048_sliced_noalloc, the entry point for callers that cannot allocate
device memory at call time (a serving process whose HBM is entirely owned by its KV-cache pool, a
loop in which a device-wide blocking cudaMalloc is not acceptable). It keeps its scratch in a
device array built into the library.

The file name sorts last on purpose: if this test fails, a run that stops at the first failure has
already run every other test. It is self-contained (passes alone in a fresh process as well).

What is checked, through the C ABI, on two calls in a row (the second call finds the first call's
leftovers in the shared scratch array): the result equals, as an index set per row, the result of
the existing entry points that do the same work with allocated scratch
(fftopk_select2048_cp per slice + fftopk_merge2048_cp over buffers from fftopk_comm_create), and
both equal the CPU oracle. Sizes beyond the built-in scratch are refused.
"""
import ctypes

import numpy as np
import pytest
import torch

import workloads
from jit_kernel import _native
from jit_kernel.distributed import local_lengths
from oracle import topk_oracle as orc

pytestmark = pytest.mark.gpu
K = 2048


def _with_allocated_scratch(lib, dev, score, lengths, G):
    """The existing path: one comm buffer per slice (cudaMalloc inside fftopk_comm_create)."""
    B, L = score.shape
    Ls = L // G
    comms = []
    for _ in range(G):
        p = ctypes.c_void_p()
        h = ctypes.create_string_buffer(64)
        _native.check(lib.fftopk_comm_create(B, ctypes.byref(p), h), "fftopk_comm_create")
        comms.append(p.value)
    arr = (ctypes.c_void_p * G)(*comms)
    out = torch.empty(B, K, dtype=torch.int32, device=dev)
    keep = []
    for g in range(G):
        shard = score[:, g * Ls:(g + 1) * Ls].contiguous().to(dev)
        lens = local_lengths(lengths, Ls, g).to(dev)
        keep += [shard, lens]
        _native.check(lib.fftopk_select2048_cp(shard.data_ptr(), Ls, B, Ls, lens.data_ptr(), g * Ls, comms[g], B, 1,
                                               None, None), "fftopk_select2048_cp")
    _native.check(lib.fftopk_merge2048_cp(arr, G, 0, B, B, 1, 1000, out.data_ptr(), None, None, None),
                  "fftopk_merge2048_cp")
    torch.cuda.synchronize()
    for c in comms:
        lib.fftopk_comm_destroy(c)
    return out.cpu().numpy()


def _no_alloc(lib, dev, score, lengths, G):
    sd, ld = score.to(dev), lengths.to(dev)
    out = torch.full((score.size(0), K), 7, dtype=torch.int32, device=dev)
    torch.cuda.synchronize()
    rc = lib.fftopk_topk2048_sliced_noalloc(sd.data_ptr(), sd.stride(0), sd.size(0), sd.size(1), ld.data_ptr(), G,
                                            out.data_ptr(), None, None)
    _native.check(rc, "fftopk_topk2048_sliced_noalloc")
    torch.cuda.synchronize()
    return out.cpu().numpy()


def test_no_alloc_entry_point_matches_allocating_path_twice_in_a_row():
    lib = _native.lib()
    dev = torch.device("cuda", 0)
    # call 1: four rows, planted heavy tail, 8 slices; call 2: other data, other shape, ragged
    # lengths with a row shorter than k and exact ties - it runs on top of call 1's leftovers
    s1, l1 = workloads.c5(B=4, L=1 << 18)
    s2, l2 = workloads.c4(B=3, L=98304)
    l2 = torch.tensor([98304, 40000, 1500], dtype=torch.int32)
    for score, lengths, G in ((s1, l1, 8), (s2, l2, 4)):
        got = _no_alloc(lib, dev, score, lengths, G)
        ref = _with_allocated_scratch(lib, dev, score, lengths, G)
        for b in range(score.size(0)):
            assert np.array_equal(np.sort(got[b]), np.sort(ref[b])), f"row {b}: differs from the allocating path"
        exp = orc.numpy_oracle(score.numpy(), lengths.numpy(), K)
        for b in range(score.size(0)):
            n = min(int(lengths[b]), K)
            assert np.array_equal(np.sort(got[b][got[b] >= 0]), np.sort(exp[b][exp[b] >= 0])), f"row {b}: oracle"
            assert int((got[b] >= 0).sum()) == n


@pytest.mark.parametrize("L,G,lens", [
    (100003, 7, [100003, 50001, 14287, 14286, 3000]),  # L not a multiple of the slice count; lengths at slice edges
    (10001, 8, [10001, 9000, 2049, 2048, 100]),        # slices of 1251 columns: every slice is shorter than k
    (5, 8, [5, 3, 0]),                                 # fewer columns than slices: slices of length 0
    (4100, 3, [4100, 4099, 1367, 1366]),               # a row that ends exactly where a slice does
])
def test_no_alloc_entry_point_odd_slicings(L, G, lens):
    """Slices that do not divide the row, slices of 2048 or fewer columns and empty slices, compared
    with the plain entry point (fftopk_select2048) and the oracle."""
    lib = _native.lib()
    dev = torch.device("cuda", 0)
    g = torch.Generator().manual_seed(L + G)
    score = torch.randn(len(lens), L, generator=g)
    score[:, ::7] = 0.5  # exact ties across slice borders
    lengths = torch.tensor(lens, dtype=torch.int32)
    got = _no_alloc(lib, dev, score, lengths, G)
    from jit_kernel.topk_indexer import fast_topk_v3
    plain = fast_topk_v3(score.to(dev), lengths.to(dev), K).cpu().numpy()
    exp = orc.numpy_oracle(score.numpy(), lengths.numpy(), K)
    for b in range(len(lens)):
        assert np.array_equal(np.sort(got[b]), np.sort(plain[b])), f"row {b}: differs from fftopk_select2048"
        assert np.array_equal(np.sort(got[b]), np.sort(exp[b])), f"row {b}: differs from the oracle"


def test_no_alloc_entry_point_refuses_sizes_beyond_its_scratch():
    lib = _native.lib()
    dev = torch.device("cuda", 0)
    s = torch.zeros(9, 4096, device=dev)
    ln = torch.full((9,), 4096, dtype=torch.int32, device=dev)
    out = torch.empty(9, K, dtype=torch.int32, device=dev)
    assert lib.fftopk_topk2048_sliced_noalloc(s.data_ptr(), 4096, 9, 4096, ln.data_ptr(), 2, out.data_ptr(), None, None) == -4
    assert lib.fftopk_topk2048_sliced_noalloc(s.data_ptr(), 4096, 8, 4096, ln.data_ptr(), 9, out.data_ptr(), None, None) == -4
    assert b"range" in lib.fftopk_strerror(-4)
