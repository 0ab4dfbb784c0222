"""Throughput mode (fftopk_set_overlap(1)) around the entry points that enqueue a producer kernel
of their own before the selection: host buffers (gather kernel -> select), column slices without
allocation (slice lengths -> selects -> merge) and the context-parallel publication (select ->
merge); 16-bit scores, which have no producer any more, run overlapped like plain calls. Their selections must keep plain stream
order whatever the process-wide switch says: a programmatic dependent launch that never waits for
its predecessor would have no guarantee of seeing the producer's writes. Every path runs several
calls back to back on DIFFERENT data through the same staging memory, with the switch on, and is
compared with the oracle; plain overlapped selections run in between."""
import ctypes
import threading

import numpy as np
import pytest
import torch

import workloads
from jit_kernel import _native
from jit_kernel.distributed import local_lengths
from jit_kernel.topk_indexer import fast_topk, fast_topk_general, fast_topk_v3, fast_topk_v3_host, kernel_status
from oracle import topk_oracle as orc

pytestmark = pytest.mark.gpu
K = 2048


@pytest.fixture(autouse=True)
def _overlap_on():
    _native.set_tuning()
    _native.set_overlap(True)
    yield
    _native.set_overlap(False)


def _batches(n, B, L, seed0):
    return [workloads.c3(seed=seed0 + i, B=B, L=L, min_len=1000) for i in range(n)]


def test_host_buffer_entry_with_overlap_on():
    dev = torch.device("cuda", 0)
    batches = _batches(4, 24, 50000, 100)
    outs = []
    filler = workloads.c3(seed=9, B=64, L=30000)
    fs, fl = filler[0].to(dev), filler[1].to(dev)
    fo = torch.empty(64, K, dtype=torch.int32, device=dev)
    pinned = [(s.pin_memory(), ln.pin_memory()) for s, ln in batches]  # alive until the stream has drained:
    for hs, hl in pinned:                                              # the call only enqueues
        fast_topk(fs, fo, fl)  # an overlapped plain call right before the composite one
        outs.append(fast_topk_v3_host(hs, hl, K))
        fast_topk(fs, fo, fl)
    torch.cuda.synchronize()
    for (s, ln), out in zip(batches, outs):
        orc.check_result(s.numpy(), ln.numpy(), out.numpy(), what="host entry, overlap on")
    assert kernel_status(dev) == 0


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_16bit_entry_with_overlap_on(dtype):
    dev = torch.device("cuda", 0)
    batches = [(s.to(dtype), ln) for s, ln in _batches(4, 16, 40000, 200)]
    outs = [fast_topk_general(s.to(dev), ln.to(dev), K) for s, ln in batches]
    torch.cuda.synchronize()
    for (s, ln), out in zip(batches, outs):
        orc.check_result(s.to(torch.float32).numpy(), ln.numpy(), out.cpu().numpy(), what=f"{dtype}, overlap on")
    assert kernel_status(dev) == 0


def test_no_alloc_entry_with_overlap_on():
    lib = _native.lib()
    dev = torch.device("cuda", 0)
    cases = [workloads.c5(seed=3, B=4, L=1 << 17), workloads.c3(seed=4, B=8, L=70001, min_len=1000),
             workloads.c5(seed=5, B=2, L=300000)]
    outs, keep = [], []
    for s, ln in cases:  # enqueued back to back on one stream: they share the built-in scratch
        sd, ld = s.to(dev), ln.to(dev)
        out = torch.empty(s.size(0), K, dtype=torch.int32, device=dev)
        keep += [sd, ld]
        _native.check(lib.fftopk_topk2048_sliced_noalloc(sd.data_ptr(), sd.stride(0), sd.size(0), sd.size(1),
                                                         ld.data_ptr(), 5, out.data_ptr(), None, None), "noalloc")
        outs.append(out)
    torch.cuda.synchronize()
    for (s, ln), out in zip(cases, outs):
        orc.check_result(s.numpy(), ln.numpy(), out.cpu().numpy(), what="no-alloc entry, overlap on")


def test_context_parallel_publication_with_overlap_on():
    """Slices selected into comm buffers, published and merged on ONE device (stream order stands in
    for the peers), several epochs in a row with different data."""
    lib = _native.lib()
    dev = torch.device("cuda", 0)
    G, B = 4, 4
    comms = []
    for _ in range(G):
        p, h = ctypes.c_void_p(), ctypes.create_string_buffer(64)
        _native.check(lib.fftopk_comm_create(B, ctypes.byref(p), h), "fftopk_comm_create")
        comms.append(p.value)
    arr = (ctypes.c_void_p * G)(*comms)
    try:
        keep, results = [], []
        for e in range(1, 5):
            s, ln = workloads.c5(seed=40 + e, B=B, L=1 << 18)
            Ls = s.size(1) // G
            for g in range(G):
                shard = s[:, g * Ls:(g + 1) * Ls].contiguous().to(dev)
                lens = local_lengths(ln, Ls, g).to(dev)
                keep += [shard, lens]
                _native.check(lib.fftopk_select2048_cp(shard.data_ptr(), Ls, B, Ls, lens.data_ptr(), g * Ls, comms[g], B,
                                                       e, None, None), "fftopk_select2048_cp")
            out = torch.empty(B, K, dtype=torch.int32, device=dev)
            _native.check(lib.fftopk_merge2048_cp(arr, G, 0, B, B, e, 1000, out.data_ptr(), None, None, None),
                          "fftopk_merge2048_cp")
            results.append((s, ln, out))
        torch.cuda.synchronize()
        for s, ln, out in results:
            orc.check_result(s.numpy(), ln.numpy(), out.cpu().numpy(), what="cp publication, overlap on")
    finally:
        torch.cuda.synchronize()
        for c in comms:
            lib.fftopk_comm_destroy(c)


def test_concurrent_host_threads():
    """Several host threads, each on its own stream, calling while another thread flips the
    process-wide switches: every launch works on its own snapshot of them."""
    dev = torch.device("cuda", 0)
    s, ln = workloads.c3(seed=77, B=16, L=40000)
    sd, ld = s.to(dev), ln.to(dev)
    expected = np.sort(orc.numpy_oracle(s.numpy(), ln.numpy(), K), axis=1)
    errors = []

    def worker():
        try:
            torch.cuda.set_device(dev)
            st = torch.cuda.Stream(device=dev)
            with torch.cuda.stream(st):
                for _ in range(20):
                    out = fast_topk_v3(sd, ld, K)
                    st.synchronize()
                    if not np.array_equal(np.sort(out.cpu().numpy(), axis=1), expected):
                        errors.append("wrong result")
        except Exception as e:  # pragma: no cover
            errors.append(repr(e))

    def flipper():
        for i in range(200):
            _native.set_overlap(bool(i & 1))
            _native.set_tuning(cluster_ctas=(1, 2, 4, -1)[i & 3])

    threads = [threading.Thread(target=worker) for _ in range(4)] + [threading.Thread(target=flipper)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    _native.set_tuning()
    assert not errors, errors[:3]
