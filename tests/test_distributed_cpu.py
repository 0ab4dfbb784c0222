"""World-size-2 gloo tests of the multi-GPU plumbing on CPU: row sharding arithmetic and the
context-parallel select -> all-gather -> merge flow, with oracle stand-ins for the two kernels
(the kernels themselves are covered by the GPU tests)."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

K = 2048


def _numpy_select(score, lengths, idx_offset):
    """Stand-in for the CUDA select: packed [2, B, K] int32 (global index plane, key plane)."""
    from oracle import topk_oracle as orc
    s = score.numpy()
    B = s.shape[0]
    out = np.zeros((2, B, K), dtype=np.int32)
    idx = orc.numpy_oracle(s, lengths.numpy(), K)
    for b in range(B):
        valid = idx[b] >= 0
        keys = np.zeros(K, dtype=np.uint32)
        keys[valid] = orc.keys_of(s[b, idx[b][valid]])
        out[0, b] = np.where(valid, idx[b] + idx_offset, -1)
        out[1, b] = keys.view(np.int32)
    return torch.from_numpy(out)


def _numpy_merge(cand):
    c = cand.numpy()
    G, _, B, _ = c.shape
    out = np.full((B, K), -1, dtype=np.int32)
    for b in range(B):
        idx = c[:, 0, b].reshape(-1).astype(np.int64)
        key = c[:, 1, b].reshape(-1).view(np.uint32).astype(np.uint64)
        valid = idx >= 0
        comp = (key[valid] << np.uint64(32)) | (np.uint64(0xFFFFFFFF) - idx[valid].astype(np.uint64))
        order = np.argsort(comp)[::-1][:K]
        out[b, :len(order)] = idx[valid][order]
    return torch.from_numpy(out)


def _worker(rank, world, port, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    repo = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    sys.path.insert(0, repo)
    sys.path.insert(0, os.path.join(repo, "flash-float-jit-kernels_b200"))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import workloads
        from jit_kernel.distributed import fast_topk_v3_context_parallel, local_lengths, shard_rows
        from oracle import topk_oracle as orc

        # context parallel: 3 rows, ragged global lengths, one row shorter than k
        score, _ = workloads.c5(B=3, L=16384)
        lengths = torch.tensor([16384, 9000, 1500], dtype=torch.int32)
        Ls = 16384 // world
        shard = score[:, rank * Ls:(rank + 1) * Ls].contiguous()
        got = fast_topk_v3_context_parallel(shard, lengths, K, select_fn=_numpy_select, merge_fn=_numpy_merge)
        exp = orc.numpy_oracle(score.numpy(), lengths.numpy(), K)
        for b in range(3):
            g = np.sort(got[b].numpy())
            e = np.sort(exp[b])
            assert np.array_equal(g, e), f"rank {rank} row {b}"
        assert local_lengths(lengths, Ls, rank).tolist() == [max(0, min(Ls, int(l) - rank * Ls)) for l in lengths]

        # row sharding: every row is owned exactly once
        owned = torch.zeros(7, dtype=torch.int32)
        b0, b1 = shard_rows(7, world, rank)
        owned[b0:b1] = 1
        dist.all_reduce(owned)
        assert owned.tolist() == [1] * 7
        ret[rank] = "ok"
    finally:
        dist.destroy_process_group()


@pytest.mark.timeout(180)
def test_context_parallel_and_row_sharding_world2():
    world = 2
    port = 29500 + (os.getpid() % 2000)
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_worker, args=(world, port, ret), nprocs=world, join=True)
    assert dict(ret) == {0: "ok", 1: "ok"}


def test_shard_rows_partitions():
    from jit_kernel.distributed import shard_rows
    for n in (0, 1, 7, 64, 65):
        for w in (1, 2, 4, 8):
            spans = [shard_rows(n, w, r) for r in range(w)]
            assert spans[0][0] == 0 and spans[-1][1] == n
            assert all(spans[i][1] == spans[i + 1][0] for i in range(w - 1))
            sizes = [b - a for a, b in spans]
            assert max(sizes) - min(sizes) <= 1
