"""Multi-GPU modes of the top-2048 selector (one process per GPU, torch.distributed / NCCL).

The reference has no multi-GPU path; both modes here are additions on top of its single-GPU op.

* Row sharding: rows are independent, so every rank simply runs ``fast_topk_v3`` on its rows.
  ``shard_rows`` gives the row range of a rank; there is no collective on the data path.
* Context parallel: every rank holds a contiguous slice ``score[:, g*Ls:(g+1)*Ls]`` of the
  sequence. The global top-k is contained in the union of the local top-k sets (same total order:
  value descending, global index ascending), so each rank selects locally - emitting the radix
  key and the GLOBAL index of every pick - the picks are all-gathered over NVLink, and one merge
  kernel per rank selects the final 2048 of the G*2048 candidates. Ties resolve to the lower
  global index exactly as on a single device.

``select_fn`` / ``merge_fn`` can be replaced (the CPU tests run the plumbing under gloo with
stand-ins); by default they are the CUDA kernels behind the C ABI.
"""
from __future__ import annotations

from typing import Callable, Optional, Tuple

import torch
import torch.distributed as dist

from . import _native
from .topk_indexer import TOPK, _status_word, fast_topk


def shard_rows(num_rows: int, world_size: int, rank: int) -> Tuple[int, int]:
    """Contiguous block of rows [begin, end) owned by `rank` (sizes differ by at most one)."""
    base, extra = divmod(num_rows, world_size)
    begin = rank * base + min(rank, extra)
    return begin, begin + base + (1 if rank < extra else 0)


def local_lengths(lengths_global: torch.Tensor, shard_len: int, rank: int) -> torch.Tensor:
    """Valid elements of every row that fall into this rank's slice [rank*shard_len, +shard_len)."""
    return torch.clamp(lengths_global.to(torch.int64) - rank * shard_len, 0, shard_len).to(torch.int32)


def _cuda_select(score, lengths, idx_offset):
    B = score.size(0)
    packed = torch.empty((2, B, TOPK), dtype=torch.int32, device=score.device)  # [0]=index, [1]=key
    fast_topk(score, packed[0], lengths, None, keys=packed[1], idx_offset=idx_offset)
    return packed


def merge_candidates(cand: torch.Tensor) -> torch.Tensor:
    """cand: int32 [G, 2, B, 2048] (index plane, key plane per shard) -> int32 [B, 2048]."""
    G, two, B, k = cand.shape
    assert two == 2 and k == TOPK and cand.is_contiguous() and cand.is_cuda
    out = torch.empty((B, TOPK), dtype=torch.int32, device=cand.device)
    if B == 0:
        return out
    # [G, 2, B, 2048]: index plane at the base, key plane B*2048 elements later, shards 2*B*2048 apart
    plane = B * TOPK
    lib = _native.lib()
    with torch.cuda.device(cand.device):
        rc = lib.fftopk_merge2048(cand.data_ptr() + 4 * plane, cand.data_ptr(), 2 * plane, G, B, out.data_ptr(), None,
                                  _status_word(cand.device).data_ptr(),
                                  torch.cuda.current_stream().cuda_stream)
    _native.check(rc, "fftopk_merge2048")
    return out


def fast_topk_v3_context_parallel(
    score_shard: torch.Tensor,
    lengths_global: torch.Tensor,
    topk: int,
    group: Optional[dist.ProcessGroup] = None,
    select_fn: Optional[Callable] = None,
    merge_fn: Optional[Callable] = None,
) -> torch.Tensor:
    """Top-2048 over a sequence that is split evenly across the ranks of `group`.

    score_shard:    [B, Ls] this rank's slice (rank g holds global columns g*Ls .. (g+1)*Ls - 1)
    lengths_global: [B] int32 valid length of every full row (same on all ranks)
    Returns [B, 2048] int32 GLOBAL indices on every rank (unordered; -1 padded if the row has
    fewer than 2048 valid entries).
    """
    assert topk == TOPK, "only topk=2048 is supported"
    assert score_shard.dim() == 2
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    B, Ls = score_shard.shape
    select = select_fn or _cuda_select
    merge = merge_fn or merge_candidates
    lens = local_lengths(lengths_global, Ls, rank).to(score_shard.device)
    mine = select(score_shard, lens, rank * Ls)  # [2, B, 2048]
    gathered = torch.empty((world,) + tuple(mine.shape), dtype=mine.dtype, device=mine.device)
    # concatenation along dim 0 is the layout every backend accepts for all_gather_into_tensor
    dist.all_gather_into_tensor(gathered.view((world * mine.shape[0],) + tuple(mine.shape[1:])),
                                mine.contiguous(), group=group)
    return merge(gathered)


class FusedContextParallelTopk:
    """Context-parallel top-2048 without a collective call on the data path.

    Every rank keeps a "comm" buffer that all peers map through CUDA IPC. A call is ONE kernel per
    rank (fftopk_topk2048_cp): the row's cluster selects the local top 2048, pushes them as
    self-validating packets into every rank's buffer with plain stores over NVLink, polls (bounded,
    `wait_ms`) its own buffer for the packets of the row's other slices and merges. Where the
    launch plan cannot host the merge in the selection kernel (many rows of short slices) the call
    is two kernels instead: selection that publishes an epoch flag (fftopk_select2048_cp) and a
    merge kernel that waits for the peers' flags and pulls their candidates (fftopk_merge2048_cp).
    torch.distributed is used once, at construction, to exchange the IPC handles.

    All ranks of `group` must construct the object and call it the same number of times with the
    same shapes (the epoch counters advance by one per call on every rank).
    """

    def __init__(self, max_rows: int, group: Optional[dist.ProcessGroup] = None, wait_ms: int = 2000,
                 single_launch: bool = True):
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.b_cap = int(max_rows)
        self.wait_ms = int(wait_ms)
        self.single_launch = bool(single_launch)
        self.epoch = 0
        self.device = torch.device("cuda", torch.cuda.current_device())
        # (the single-launch call and the two-call sequence use disjoint regions of the buffers)
        self._sets = [self._exchange_buffers()]
        dist.barrier(group=group)  # every buffer is mapped everywhere before the first call

    def _exchange_buffers(self):
        import ctypes
        lib = _native.lib()
        own = ctypes.c_void_p()
        handle = ctypes.create_string_buffer(64)
        _native.check(lib.fftopk_comm_create(self.b_cap, ctypes.byref(own), handle), "fftopk_comm_create")
        handles = [None] * self.world
        dist.all_gather_object(handles, bytes(handle.raw), group=self.group)
        peers, ptrs = [], []
        for r in range(self.world):
            if r == self.rank:
                ptrs.append(own.value)
                continue
            p = ctypes.c_void_p()
            _native.check(lib.fftopk_comm_open(handles[r], ctypes.byref(p)), "fftopk_comm_open")
            peers.append(p.value)
            ptrs.append(p.value)
        return {"own": own.value, "peers": peers, "comms": (ctypes.c_void_p * self.world)(*ptrs)}

    def __call__(self, score_shard: torch.Tensor, lengths_global: torch.Tensor, topk: int = TOPK) -> torch.Tensor:
        assert topk == TOPK and score_shard.dim() == 2
        B, Ls = score_shard.shape
        if B > self.b_cap:
            raise RuntimeError(f"batch of {B} rows exceeds the comm buffer capacity {self.b_cap}")
        if not score_shard.is_cuda or score_shard.dtype != torch.float32 or (score_shard.stride(1) != 1 and Ls > 1):
            raise RuntimeError("score_shard must be a CUDA float32 tensor with unit inner stride")
        lens = local_lengths(lengths_global, Ls, self.rank).to(score_shard.device)
        out = torch.empty((B, TOPK), dtype=torch.int32, device=score_shard.device)
        self.run_into(score_shard, lens, out)
        return out

    def run_into(self, score_shard: torch.Tensor, local_lens: torch.Tensor, out: torch.Tensor) -> None:
        """The enqueue-only core (no allocation, no host-side state: the epochs live on the device),
        so this sequence can be captured in a CUDA graph and replayed - every rank the same number
        of times. `local_lens` = local_lengths(lengths_global, Ls, rank) on the device."""
        B, Ls = score_shard.shape
        self.epoch += 1
        lib = _native.lib()
        status = _status_word(score_shard.device).data_ptr()
        with torch.cuda.device(score_shard.device):
            stream = torch.cuda.current_stream().cuda_stream
            if self.single_launch:
                one = self._sets[0]
                rc = lib.fftopk_topk2048_cp(score_shard.data_ptr(), score_shard.stride(0), B, Ls, local_lens.data_ptr(),
                                            self.rank * Ls, one["comms"], self.world, self.rank, self.b_cap, 0,
                                            self.wait_ms, out.data_ptr(), status, stream)
                if rc != _native.E_RANGE:
                    _native.check(rc, "fftopk_topk2048_cp")
                    return
                # this shape does not fit the single launch (the same answer on every rank)
            two = self._sets[0]
            rc = lib.fftopk_select2048_cp(score_shard.data_ptr(), score_shard.stride(0), B, Ls, local_lens.data_ptr(),
                                          self.rank * Ls, two["own"], self.b_cap, 0, status, stream)
            _native.check(rc, "fftopk_select2048_cp")
            rc = lib.fftopk_merge2048_cp(two["comms"], self.world, self.rank, B, self.b_cap, 0, self.wait_ms,
                                         out.data_ptr(), None, status, stream)
            _native.check(rc, "fftopk_merge2048_cp")

    def close(self) -> None:
        """Unmap the peers' buffers and free the own ones (all ranks, after a barrier)."""
        if not self._sets:
            return
        torch.cuda.synchronize()
        dist.barrier(group=self.group)
        lib = _native.lib()
        for s in self._sets:
            for p in s["peers"]:
                lib.fftopk_comm_close(p)
        dist.barrier(group=self.group)
        for s in self._sets:
            lib.fftopk_comm_destroy(s["own"])
        self._sets = []
