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


# ----------------------------------------------------------------------------------------------
# fused gather-and-merge (fftopk_select2048_cp / fftopk_merge2048_cp) on one device: the G shards
# publish into G separate comm buffers one after the other (stream order), so the merge kernel's
# waits are already satisfied when it starts - nothing here waits on a concurrently running kernel.
# ----------------------------------------------------------------------------------------------
def _comm_create(b_cap):
    import ctypes
    from jit_kernel import _native
    lib = _native.lib()
    p = ctypes.c_void_p()
    h = ctypes.create_string_buffer(64)
    _native.check(lib.fftopk_comm_create(b_cap, ctypes.byref(p), h), "comm_create")
    return p.value


def _fused_on_one_device(score, lengths, G, epochs=(1,)):
    import ctypes
    from jit_kernel import _native
    lib = _native.lib()
    dev = torch.device("cuda", 0)
    B, L = score.shape
    Ls = L // G
    comms = [_comm_create(B) for _ in range(G)]
    arr = (ctypes.c_void_p * G)(*comms)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    out = torch.empty(B, K, dtype=torch.int32, device=dev)
    shards = [score[:, g * Ls:(g + 1) * Ls].contiguous().to(dev) for g in range(G)]
    lens = [local_lengths(lengths, Ls, g).to(dev) for g in range(G)]
    results = []
    for e in epochs:
        for g in range(G):
            rc = lib.fftopk_select2048_cp(shards[g].data_ptr(), Ls, B, Ls, lens[g].data_ptr(), g * Ls, comms[g], B, e,
                                          status.data_ptr(), None)
            assert rc == 0
        rc = lib.fftopk_merge2048_cp(arr, G, 0, B, B, e, 1000, out.data_ptr(), None, status.data_ptr(), None)
        assert rc == 0
        torch.cuda.synchronize()
        results.append(out.cpu().numpy().copy())
    for c in comms:
        lib.fftopk_comm_destroy(c)
    return results, int(status.item())


@pytest.mark.parametrize("G", [2, 8])
def test_fused_gather_merge_matches_oracle(G):
    score, lengths = workloads.c5(B=2, L=1 << 19)
    results, status = _fused_on_one_device(score, lengths, G, epochs=(1, 2, 3))  # both buffer halves, reused
    assert status == 0
    for got in results:
        orc.check_result(score.numpy(), lengths.numpy(), got, what=f"fused G={G}")


def test_fused_merge_wait_runs_out_without_hanging():
    """A flag that nothing sets: the bounded wait gives up, the row is -1, the status says so and
    the context stays usable."""
    import ctypes
    from jit_kernel import _native
    lib = _native.lib()
    dev = torch.device("cuda", 0)
    comm = _comm_create(2)
    arr = (ctypes.c_void_p * 1)(comm)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    out = torch.zeros(2, K, dtype=torch.int32, device=dev)
    rc = lib.fftopk_merge2048_cp(arr, 1, 0, 2, 2, 5, 20, out.data_ptr(), None, status.data_ptr(), None)  # epoch 5 never published
    assert rc == 0
    torch.cuda.synchronize()
    assert int(status.item()) & _native.ST_PEER_TIMEOUT
    assert bool((out == -1).all())
    # the device still works
    s, ln = workloads.c1()
    from jit_kernel.topk_indexer import fast_topk_v3
    got = fast_topk_v3(s.to(dev), ln.to(dev), K).cpu().numpy()
    orc.check_result(s.numpy(), ln.numpy(), got, what="after timeout")
    lib.fftopk_comm_destroy(comm)


def test_fused_device_side_epochs_and_graph_replay():
    """epoch = 0: the publish kernel counts epochs on the device, so the whole select / publish /
    merge sequence has no per-call host argument and a captured graph can be replayed."""
    import ctypes
    from jit_kernel import _native
    lib = _native.lib()
    dev = torch.device("cuda", 0)
    G = 4
    score, lengths = workloads.c5(B=2, L=1 << 18)
    B, L = score.shape
    Ls = L // G
    comms = [_comm_create(B) for _ in range(G)]
    arr = (ctypes.c_void_p * G)(*comms)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    out = torch.empty(B, K, dtype=torch.int32, device=dev)
    shards = [score[:, g * Ls:(g + 1) * Ls].contiguous().to(dev) for g in range(G)]
    lens = [local_lengths(lengths, Ls, g).to(dev) for g in range(G)]

    def sequence(stream_ptr):
        for g in range(G):
            assert lib.fftopk_select2048_cp(shards[g].data_ptr(), Ls, B, Ls, lens[g].data_ptr(), g * Ls, comms[g], B, 0,
                                            status.data_ptr(), stream_ptr) == 0
        assert lib.fftopk_merge2048_cp(arr, G, 0, B, B, 0, 1000, out.data_ptr(), None, status.data_ptr(), stream_ptr) == 0

    for _ in range(2):  # eager: epochs 1 and 2 (both halves)
        sequence(None)
        torch.cuda.synchronize()
        orc.check_result(score.numpy(), lengths.numpy(), out.cpu().numpy(), what="device epochs eager")
    side = torch.cuda.Stream()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        with torch.cuda.graph(graph, stream=side):
            sequence(side.cuda_stream)
    for _ in range(3):  # epochs 3, 4, 5
        out.fill_(-7)
        graph.replay()
        torch.cuda.synchronize()
        orc.check_result(score.numpy(), lengths.numpy(), out.cpu().numpy(), what="device epochs replay")
    assert int(status.item()) == 0
    for c in comms:
        lib.fftopk_comm_destroy(c)


# ----------------------------------------------------------------------------------------------
# single-launch context-parallel call (fftopk_topk2048_cp) on one device. With one shard (G = 1)
# the kernel selects, publishes the row's flag, "waits" for its own flag and merges its own list;
# real peers are covered by test_multi_gpu.py. Nothing here waits on another kernel.
# ----------------------------------------------------------------------------------------------
def _single_launch(lib, comms_arr, G, own, b_cap, score_dev, lens_dev, epoch, out, status, stream=None, wait_ms=1000):
    return lib.fftopk_topk2048_cp(score_dev.data_ptr(), score_dev.stride(0), score_dev.size(0), score_dev.size(1),
                                  lens_dev.data_ptr(), 0, comms_arr, G, own, b_cap, epoch, wait_ms, out.data_ptr(),
                                  status.data_ptr(), stream)


@pytest.mark.parametrize("case", ["c5", "ragged", "ties", "c2"])
def test_single_launch_one_shard_matches_oracle(case):
    import ctypes
    from jit_kernel import _native
    lib = _native.lib()
    dev = torch.device("cuda", 0)
    if case == "c5":
        score, lengths = workloads.c5(B=4, L=1 << 19)
    elif case == "ragged":
        score, lengths = workloads.c3(B=8, L=70000, min_len=500)
        lengths[0], lengths[1] = 100, 2048
    elif case == "ties":
        score, lengths = workloads.c4(B=3, L=131072)
    else:
        score, lengths = workloads.c2(L=40000, B=20)  # 512-thread plan? no: many rows, fewer CTAs per row
    B = score.size(0)
    comm = _comm_create(B)
    arr = (ctypes.c_void_p * 1)(comm)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    out = torch.empty(B, K, dtype=torch.int32, device=dev)
    sd, ld = score.to(dev), lengths.to(dev)
    for e in (1, 2, 3):  # both halves, reused
        out.fill_(-9)
        assert _single_launch(lib, arr, 1, 0, B, sd, ld, e, out, status) == 0
        torch.cuda.synchronize()
        got = out.cpu().numpy()
        exp = orc.numpy_oracle(score.numpy(), lengths.numpy(), K)
        for b in range(B):
            assert np.array_equal(np.sort(got[b]), np.sort(exp[b])), f"{case} epoch {e} row {b}"
    assert int(status.item()) == 0
    lib.fftopk_comm_destroy(comm)


def test_single_launch_device_side_epochs_and_graph_replay():
    import ctypes
    from jit_kernel import _native
    lib = _native.lib()
    dev = torch.device("cuda", 0)
    score, lengths = workloads.c5(B=2, L=1 << 18)
    comm = _comm_create(2)
    arr = (ctypes.c_void_p * 1)(comm)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    out = torch.empty(2, K, dtype=torch.int32, device=dev)
    sd, ld = score.to(dev), lengths.to(dev)
    for _ in range(2):
        assert _single_launch(lib, arr, 1, 0, 2, sd, ld, 0, out, status) == 0
        torch.cuda.synchronize()
        orc.check_result(score.numpy(), lengths.numpy(), out.cpu().numpy(), what="single launch, device epochs")
    side = torch.cuda.Stream()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        with torch.cuda.graph(graph, stream=side):
            assert _single_launch(lib, arr, 1, 0, 2, sd, ld, 0, out, status, side.cuda_stream) == 0
    for _ in range(3):
        out.fill_(-7)
        graph.replay()
        torch.cuda.synchronize()
        orc.check_result(score.numpy(), lengths.numpy(), out.cpu().numpy(), what="single launch, replay")
    assert int(status.item()) == 0
    lib.fftopk_comm_destroy(comm)


def test_single_launch_wait_runs_out_without_hanging():
    """Two shards, but the second buffer is one that nobody ever publishes into: the bounded wait of
    the CTA that owns that shard gives up, every row is -1, the status says so, the device works."""
    import ctypes
    from jit_kernel import _native
    lib = _native.lib()
    dev = torch.device("cuda", 0)
    score, lengths = workloads.c5(B=2, L=1 << 17)
    own, silent = _comm_create(2), _comm_create(2)
    arr = (ctypes.c_void_p * 2)(own, silent)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    out = torch.zeros(2, K, dtype=torch.int32, device=dev)
    assert _single_launch(lib, arr, 2, 0, 2, score.to(dev), lengths.to(dev), 1, out, status, wait_ms=20) == 0
    torch.cuda.synchronize()
    assert int(status.item()) & _native.ST_PEER_TIMEOUT
    assert bool((out == -1).all())
    s, ln = workloads.c1()
    from jit_kernel.topk_indexer import fast_topk_v3
    got = fast_topk_v3(s.to(dev), ln.to(dev), K).cpu().numpy()
    orc.check_result(s.numpy(), ln.numpy(), got, what="after timeout")
    for c in (own, silent):
        lib.fftopk_comm_destroy(c)


def test_single_launch_refuses_plans_with_fewer_ctas_than_shards():
    import ctypes
    from jit_kernel import _native
    lib = _native.lib()
    dev = torch.device("cuda", 0)
    B = 100  # one CTA per row on a 148-SM device: no room for two shard owners
    a, b = _comm_create(B), _comm_create(B)
    arr = (ctypes.c_void_p * 2)(a, b)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    out = torch.zeros(B, K, dtype=torch.int32, device=dev)
    s = torch.zeros(B, 8192, device=dev)
    ln = torch.full((B,), 8192, dtype=torch.int32, device=dev)
    assert _single_launch(lib, arr, 2, 0, B, s, ln, 1, out, status) == _native.E_RANGE
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    for c in (a, b):
        lib.fftopk_comm_destroy(c)
