"""Context-parallel mode on real GPUs: one process per GPU, NCCL all-gather, merge kernel.
Needs at least two CUDA devices (skipped otherwise); the single-GPU emulation of the same flow is
in test_merge_gpu.py and the plumbing under gloo in test_distributed_cpu.py."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu
K = 2048


def _worker(rank, world, port, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    repo = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    sys.path.insert(0, repo)
    sys.path.insert(0, os.path.join(repo, "flash-float-jit-kernels_b200"))
    dev = torch.device("cuda", rank)
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        import workloads
        from jit_kernel.distributed import fast_topk_v3_context_parallel, shard_rows
        from jit_kernel.topk_indexer import fast_topk_v3, kernel_status
        from oracle import topk_oracle as orc

        # config 5: B=4, L=1M split evenly, planted heavy tail; bit-exact against the single-device oracle
        score, lengths = workloads.c5()
        Ls = score.size(1) // world
        shard = score[:, rank * Ls:(rank + 1) * Ls].contiguous().to(dev)
        out = fast_topk_v3_context_parallel(shard, lengths, K)
        torch.cuda.synchronize()
        orc.check_result(score.numpy(), lengths.numpy(), out.cpu().numpy(), what=f"cp rank {rank}")
        # the same through the fused paths: IPC-mapped peer buffers, no collective on the data path.
        # `fused` is the single launch per rank (selection, publication, pull and merge in one
        # kernel), `fused2` the two-kernel sequence (selection with publication, merge that pulls)
        from jit_kernel.distributed import FusedContextParallelTopk
        fused = FusedContextParallelTopk(max_rows=8)
        fused2 = FusedContextParallelTopk(max_rows=8, single_launch=False)
        for _ in range(3):
            out = fused(shard, lengths)
            torch.cuda.synchronize()
            orc.check_result(score.numpy(), lengths.numpy(), out.cpu().numpy(), what=f"fused cp rank {rank}")
            out = fused2(shard, lengths)
            torch.cuda.synchronize()
            orc.check_result(score.numpy(), lengths.numpy(), out.cpu().numpy(), what=f"two-kernel cp rank {rank}")
        # ragged global lengths: some slices partly or wholly empty, a row shorter than k
        rs, rl = workloads.c3(seed=5, B=6, L=world * 20000, min_len=1000)
        rl[0], rl[1] = 1500, 20000 + 7
        rshard = rs[:, rank * 20000:(rank + 1) * 20000].contiguous().to(dev)
        for f in (fused, fused2):
            out = f(rshard, rl).cpu().numpy()
            exp = orc.numpy_oracle(rs.numpy(), rl.numpy(), K)
            for b in range(6):
                assert np.array_equal(np.sort(out[b]), np.sort(exp[b])), f"ragged cp row {b} rank {rank}"
        # tie stress across shards
        score, lengths = workloads.c4(B=2, L=131072)
        Ls = score.size(1) // world
        shard = score[:, rank * Ls:(rank + 1) * Ls].contiguous().to(dev)
        out = fast_topk_v3_context_parallel(shard, lengths, K)
        orc.check_result(score.numpy(), lengths.numpy(), out.cpu().numpy(), what=f"cp ties rank {rank}")
        # config 3 row-sharded: every rank its block of rows, no collective on the data path
        score, lengths = workloads.c3(B=16, L=50000)
        b0, b1 = shard_rows(16, world, rank)
        got = fast_topk_v3(score[b0:b1].to(dev), lengths[b0:b1].to(dev), K)
        orc.check_result(score[b0:b1].numpy(), lengths[b0:b1].numpy(), got.cpu().numpy(), what=f"rows rank {rank}")
        s4, l4 = workloads.c4(B=2, L=131072)
        sh4 = s4[:, rank * (131072 // world):(rank + 1) * (131072 // world)].contiguous().to(dev)
        for f in (fused, fused2):
            out = f(sh4, l4)
            orc.check_result(s4.numpy(), l4.numpy(), out.cpu().numpy(), what=f"fused ties rank {rank}")
        fused.close()
        fused2.close()
        assert kernel_status(dev) == 0
        ret[rank] = "ok"
    finally:
        dist.destroy_process_group()


@pytest.mark.timeout(600)
def test_context_parallel_and_row_sharding_on_gpus():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs at least two GPUs")
    world = 2 if torch.cuda.device_count() < 4 else (4 if torch.cuda.device_count() < 8 else 8)
    port = 29600 + (os.getpid() % 2000)
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_worker, args=(world, port, ret), nprocs=world, join=True)
    assert dict(ret) == {r: "ok" for r in range(world)}
