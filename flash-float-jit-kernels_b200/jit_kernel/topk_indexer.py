"""Top-2048 indexer op: drop-in for the reference's ``jit_kernel.topk_indexer``.

``fast_topk_v3`` keeps the reference's name, module path, signature and assertion behaviour
(jit_kernel/topk_indexer.py:42-75). Underneath, instead of a JIT-compiled pybind11/ATen
module, it calls the C ABI of libfftopk.so (include/fftopk.h): hand-written sm_100a CUDA,
one thread-block cluster per row. There is no Triton, no backend dispatch and no CPU path.
"""
from __future__ import annotations

import os
from typing import Optional

import torch

from . import _native

TOPK = _native.K

#: debugging aid: with FFTOPK_CHECK_STATUS=1 in the environment every op synchronises its stream
#: after the launch and raises if a kernel has reported anything in the device status word (an
#: internal inconsistency, a bounded wait on a peer that ran out). Off by default: the ops are
#: enqueue-only and never synchronise.
CHECK_STATUS = os.environ.get("FFTOPK_CHECK_STATUS", "0") not in ("", "0")

_status_words: dict[int, torch.Tensor] = {}


def _status_word(device: torch.device) -> torch.Tensor:
    idx = device.index if device.index is not None else torch.cuda.current_device()
    t = _status_words.get(idx)
    if t is None:
        t = torch.zeros(1, dtype=torch.int32, device=torch.device("cuda", idx))
        _status_words[idx] = t
    return t


def kernel_status(device=None) -> int:
    """FFTOPK_ST_* bits the kernels have raised on `device` since the process started."""
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    return int(_status_word(dev).item()) & 0xFFFFFFFF


def _after_launch(device: torch.device, what: str) -> None:
    if CHECK_STATUS:
        torch.cuda.current_stream(device).synchronize()
        st = kernel_status(device)
        if st:
            raise _native.FFTopkError(f"{what}: the kernels reported status {st:#x} (FFTOPK_ST_* bits, include/fftopk.h)")


def _check_inputs(score, lengths, row_starts, out=None):
    # reference: CHECK_CUDA + get_params (topk_indexer_radix.cu:997-1027, 1049-1062) raise
    # c10::Error, which Python sees as RuntimeError.
    if not score.is_cuda:
        raise RuntimeError("score must be a CUDA tensor")
    if score.dtype != torch.float32:
        raise RuntimeError("score must be float32")
    if score.stride(1) != 1 and score.size(1) > 1:
        raise RuntimeError("score must have unit inner stride")
    B = score.size(0)
    if not lengths.is_cuda or lengths.dtype != torch.int32:
        raise RuntimeError("lengths must be a CUDA int32 tensor")
    if lengths.dim() != 1 or lengths.size(0) != B or not lengths.is_contiguous():
        raise RuntimeError("lengths must be a contiguous 1-D tensor of size B")
    if row_starts is not None:
        if not row_starts.is_cuda or row_starts.dtype != torch.int32:
            raise RuntimeError("row_starts must be a CUDA int32 tensor")
        if row_starts.dim() != 1 or row_starts.size(0) != B or not row_starts.is_contiguous():
            raise RuntimeError("row_starts must be a contiguous 1-D tensor of size B")
        if row_starts.device != score.device:
            raise RuntimeError("row_starts must be on score's device")
    if lengths.device != score.device:
        raise RuntimeError("lengths must be on score's device")
    if out is not None:
        if out.dtype != torch.int32 or out.dim() != 2 or out.size(0) != B or out.size(1) != TOPK \
                or not out.is_contiguous() or out.device != score.device:
            raise RuntimeError("indices must be a contiguous CUDA int32 tensor of shape [B, 2048]")


def fast_topk(score: torch.Tensor, indices: torch.Tensor, lengths: torch.Tensor,
              row_starts: Optional[torch.Tensor] = None, *, keys: Optional[torch.Tensor] = None,
              idx_offset: int = 0) -> None:
    """In-place form, the call the reference's native module exports
    (``module.fast_topk(score, indices, lengths, row_starts)``, topk_indexer_radix.cu:1252-1254).

    `indices` [B, 2048] int32 is overwritten completely (no -1 pre-fill needed). `keys`, when
    given ([B, 2048] int32/uint32 storage), receives the radix key of every selected element;
    `idx_offset` is added to every index. Both exist for the context-parallel mode.
    """
    assert score.dim() == 2
    _check_inputs(score, lengths, row_starts, indices)
    B, L = score.size(0), score.size(1)
    if B == 0:
        return
    lib = _native.lib()
    with torch.cuda.device(score.device):
        stream = torch.cuda.current_stream().cuda_stream
        rc = lib.fftopk_select2048(
            score.data_ptr(), score.stride(0) if B > 1 else max(score.stride(0), 0), B, L,
            lengths.data_ptr(), row_starts.data_ptr() if row_starts is not None else None,
            indices.data_ptr(), keys.data_ptr() if keys is not None else None, int(idx_offset),
            _status_word(score.device).data_ptr(), stream)
    _native.check(rc, "fftopk_select2048")
    _after_launch(score.device, "fftopk_select2048")


def fast_topk_v3(
    score: torch.Tensor,
    lengths: torch.Tensor,
    topk: int,
    row_starts: Optional[torch.Tensor] = None,
) -> torch.Tensor:
    """
    Get the topk indices of the score tensor.
    Args:
        score: The score tensor of shape (B, L), float32, CUDA, unit inner stride.
        lengths: int32 tensor of shape (B): valid entries per row.
        topk: must be 2048.
        row_starts: optional int32 tensor of shape (B). For row i the selection applies to
            score[i, row_starts[i] : row_starts[i] + lengths[i]] and the returned indices are
            relative to row_starts[i].
    Returns:
        int32 tensor of shape (B, topk): the indices of the 2048 largest valid entries of every
        row, in unspecified order; ties at the threshold go to the lower index. Rows with
        lengths[i] <= 2048 hold 0..lengths[i]-1 followed by -1.
    """
    assert (
        topk == 2048
    ), "fast_topk_v3 only supports topk=2048 (the DeepSeek v3.2 indexer configuration)"
    assert score.dim() == 2
    _check_inputs(score, lengths, row_starts)
    topk_indices = torch.empty((score.size(0), topk), dtype=torch.int32, device=score.device)
    fast_topk(score, topk_indices, lengths, row_starts)
    return topk_indices


def fast_topk_v3_warm(
    score: torch.Tensor,
    lengths: torch.Tensor,
    topk: int,
    thresholds: torch.Tensor,
    row_starts: Optional[torch.Tensor] = None,
    margin: int = 0,
    out: Optional[torch.Tensor] = None,
) -> torch.Tensor:
    """fast_topk_v3 for a decode loop (no counterpart in the reference; README.md:90-98 discusses
    the idea): `thresholds`, an int32 CUDA tensor of shape (B) that starts as zeros, carries every
    row's threshold key from one call to the next and is updated in place. A row with a non-zero
    entry skips sampling and the threshold search and is filtered at once against that key minus
    `margin` (key units; 0 is right when rows only grow between calls). The result is always the
    exact top 2048 - a guess that does not hold only costs time (the row is selected by the
    full-histogram path and FFTOPK_ST_GUESS_MISSED shows up in kernel_status()).
    """
    assert topk == 2048, "fast_topk_v3_warm only supports topk=2048"
    assert score.dim() == 2
    _check_inputs(score, lengths, row_starts, out)
    B = score.size(0)
    if not thresholds.is_cuda or thresholds.dtype != torch.int32 or thresholds.dim() != 1 or thresholds.size(0) != B \
            or not thresholds.is_contiguous() or thresholds.device != score.device:
        raise RuntimeError("thresholds must be a contiguous CUDA int32 tensor of shape (B) on score's device")
    if not (0 <= int(margin) < (1 << 32)):
        raise ValueError("margin must fit 32 bits")
    if out is None:
        out = torch.empty((B, topk), dtype=torch.int32, device=score.device)
    if B == 0:
        return out
    lib = _native.lib()
    with torch.cuda.device(score.device):
        rc = lib.fftopk_select2048_warm(
            score.data_ptr(), score.stride(0) if B > 1 else max(score.stride(0), 0), B, score.size(1),
            lengths.data_ptr(), row_starts.data_ptr() if row_starts is not None else None,
            thresholds.data_ptr(), int(margin), thresholds.data_ptr(), out.data_ptr(),
            _status_word(score.device).data_ptr(), torch.cuda.current_stream().cuda_stream)
    _native.check(rc, "fftopk_select2048_warm")
    _after_launch(score.device, "fftopk_select2048_warm")
    return out


def fast_topk_general(
    score: torch.Tensor,
    lengths: torch.Tensor,
    topk: int,
    row_starts: Optional[torch.Tensor] = None,
) -> torch.Tensor:
    """fast_topk_v3 for any 1 <= topk <= 4096 (the reference's op asserts topk == 2048,
    topk_indexer.py:62-64). Same arguments, same result layout with `topk` columns."""
    if not (1 <= int(topk) <= 4096):
        raise ValueError("topk must be in [1, 4096]")
    assert score.dim() == 2
    if score.is_cuda and score.dtype in (torch.float16, torch.bfloat16):
        return _fast_topk_16bit(score, lengths, int(topk), row_starts)
    _check_inputs(score, lengths, row_starts)
    out = torch.empty((score.size(0), int(topk)), dtype=torch.int32, device=score.device)
    if score.size(0) == 0:
        return out
    lib = _native.lib()
    with torch.cuda.device(score.device):
        stream = torch.cuda.current_stream(score.device)
        rc = lib.fftopk_select_topk(score.data_ptr(), score.stride(0) if score.size(0) > 1 else max(score.stride(0), 0),
                                    score.size(0), score.size(1), lengths.data_ptr(),
                                    None if row_starts is None else row_starts.data_ptr(), int(topk), out.data_ptr(),
                                    None, 0, _status_word(score.device).data_ptr(), stream.cuda_stream)
    _native.check(rc, "fftopk_select_topk")
    _after_launch(score.device, "fftopk_select_topk")
    return out


def _fast_topk_16bit(score, lengths, topk, row_starts):
    """fp16 / bf16 scores (fftopk_select_topk_16bit): the selector instantiated on the 16-bit type;
    rows are read once in their own width and widened to fp32 in registers."""
    if score.stride(1) != 1 and score.size(0) and score.size(1):
        raise RuntimeError("score must have unit inner stride")
    if lengths.dtype != torch.int32 or not lengths.is_cuda or lengths.numel() != score.size(0) or not lengths.is_contiguous():
        raise RuntimeError("lengths must be a contiguous CUDA int32 tensor of shape [B]")
    if row_starts is not None and (row_starts.dtype != torch.int32 or not row_starts.is_cuda
                                   or row_starts.numel() != score.size(0) or not row_starts.is_contiguous()):
        raise RuntimeError("row_starts must be a contiguous CUDA int32 tensor of shape [B]")
    B, L = score.size(0), score.size(1)
    out = torch.empty((B, topk), dtype=torch.int32, device=score.device)
    if B == 0:
        return out
    lib = _native.lib()
    with torch.cuda.device(score.device):
        stream = torch.cuda.current_stream(score.device)
        rc = lib.fftopk_select_topk_16bit(score.data_ptr(), 0 if score.dtype == torch.float16 else 1,
                                          score.stride(0) if B > 1 else max(score.stride(0), 0), B, L, lengths.data_ptr(),
                                          None if row_starts is None else row_starts.data_ptr(), topk, out.data_ptr(),
                                          None, 0, _status_word(score.device).data_ptr(), stream.cuda_stream)
    _native.check(rc, "fftopk_select_topk_16bit")
    _after_launch(score.device, "fftopk_select_topk_16bit")
    return out


_host_workspaces = {}


def fast_topk_v3_host(
    score: torch.Tensor,
    lengths: torch.Tensor,
    topk: int,
    out: Optional[torch.Tensor] = None,
    device=None,
) -> torch.Tensor:
    """fast_topk_v3 for a caller whose tensors are in HOST memory (no counterpart in the reference,
    whose driver does score.cuda() / fast_topk_v3 / .cpu() itself, benchmark/bench_topk.py:90-146).

    score (B, L) float32 and lengths (B) int32 are CPU tensors (pinned memory makes the copies
    asynchronous); the result is an int32 CPU tensor (B, topk) - `out` if given. Only the valid
    prefix of every row is copied to the device, so a ragged batch moves about half the bytes of
    its padded matrix. Everything is enqueued on the current stream of `device`; the call returns
    without synchronising: synchronise that stream before reading the result.
    The device staging area is cached per (device, B, L).
    """
    assert topk == 2048, "fast_topk_v3_host only supports topk=2048"
    if score.is_cuda or lengths.is_cuda:
        raise RuntimeError("score and lengths must be CPU tensors")
    if score.dtype != torch.float32 or lengths.dtype != torch.int32:
        raise RuntimeError("score must be float32 and lengths int32")
    if score.dim() != 2 or lengths.dim() != 1 or lengths.numel() != score.size(0):
        raise RuntimeError("score must be (B, L) and lengths (B)")
    if score.size(0) and score.size(1) and score.stride(1) != 1:
        raise RuntimeError("score must have unit inner stride")
    lengths = lengths.contiguous()
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    B, L = score.size(0), score.size(1)
    if out is None:
        out = torch.empty((B, topk), dtype=torch.int32, pin_memory=True)
    elif out.is_cuda or out.dtype != torch.int32 or tuple(out.shape) != (B, topk) or not out.is_contiguous():
        raise RuntimeError("out must be a contiguous int32 CPU tensor of shape (B, topk)")
    if B == 0:
        return out
    lib = _native.lib()
    nbytes = int(lib.fftopk_host_workspace_bytes(B, L))
    ws = _host_workspaces.get((dev, B, L))
    if ws is None or ws.numel() < nbytes:
        ws = torch.empty(nbytes + 256, dtype=torch.uint8, device=dev)
        _host_workspaces[(dev, B, L)] = ws
    base = (ws.data_ptr() + 255) & ~255
    with torch.cuda.device(dev):
        stream = torch.cuda.current_stream(dev)
        _native.check(
            lib.fftopk_select2048_host(score.data_ptr(), score.stride(0) if B > 1 else L, B, L, lengths.data_ptr(),
                                       out.data_ptr(), base, nbytes, _status_word(dev).data_ptr(), stream.cuda_stream),
            "fftopk_select2048_host")
    _after_launch(dev, "fftopk_select2048_host")
    return out


def fast_topk_transform_fused(
    score: torch.Tensor,
    lengths: torch.Tensor,
    page_table_size_1: torch.Tensor,
    cu_seqlens_q: torch.Tensor,
    topk: int,
    row_starts: Optional[torch.Tensor] = None,
) -> torch.Tensor:
    """Top-2048 selection fused with the page-table gather that follows it.

    Mirrors the reference's exported ``fast_topk_transform_fused``
    (topk_indexer_radix.cu:1160-1214, 1255): ``dst[b, j] = page_table_size_1[i, idx_j]`` where
    ``idx_j`` are the selected indices of row ``b`` and ``i`` is the request that row belongs to
    (``cu_seqlens_q[i] <= b < cu_seqlens_q[i+1]``; with ``row_starts is None`` and one row per
    request - decode - simply ``i = b``). Rows with ``lengths[b] <= 2048`` give the first
    ``lengths[b]`` table entries followed by -1.
    """
    assert topk == TOPK, "only topk=2048 is supported"
    assert score.dim() == 2
    _check_inputs(score, lengths, row_starts)
    B = score.size(0)
    if not page_table_size_1.is_cuda or page_table_size_1.dtype != torch.int32 or page_table_size_1.dim() != 2 \
            or (page_table_size_1.stride(1) != 1 and page_table_size_1.size(1) > 1):
        raise RuntimeError("page_table_size_1 must be a 2-D CUDA int32 tensor with unit inner stride")
    if not cu_seqlens_q.is_cuda or cu_seqlens_q.dtype != torch.int32 or cu_seqlens_q.dim() != 1 \
            or not cu_seqlens_q.is_contiguous():
        raise RuntimeError("cu_seqlens_q must be a contiguous 1-D CUDA int32 tensor")
    prefill_bs = cu_seqlens_q.size(0) - 1
    if page_table_size_1.size(0) != prefill_bs or prefill_bs > B:
        raise RuntimeError("page_table_size_1 must have one row per request and prefill_bs <= B")
    dst = torch.empty((B, TOPK), dtype=torch.int32, device=score.device)
    if B == 0:
        return dst
    is_decode = row_starts is None and prefill_bs == B  # reference: radix.cu:1196
    lib = _native.lib()
    with torch.cuda.device(score.device):
        rc = lib.fftopk_select2048_page_table(
            score.data_ptr(), score.stride(0), B, score.size(1), lengths.data_ptr(),
            row_starts.data_ptr() if row_starts is not None else None, dst.data_ptr(),
            page_table_size_1.data_ptr(), page_table_size_1.stride(0),
            None if is_decode else cu_seqlens_q.data_ptr(), prefill_bs,
            _status_word(score.device).data_ptr(), torch.cuda.current_stream().cuda_stream)
    _native.check(rc, "fftopk_select2048_page_table")
    _after_launch(score.device, "fftopk_select2048_page_table")
    return dst


def fast_topk_transform_ragged_fused(
    score: torch.Tensor,
    lengths: torch.Tensor,
    topk_indices_offset: torch.Tensor,
    topk: int,
    row_starts: Optional[torch.Tensor] = None,
) -> torch.Tensor:
    """Top-2048 selection with a per-row offset added to every index (ragged KV layout).

    Mirrors ``fast_topk_transform_ragged_fused`` (topk_indexer_radix.cu:1216-1250, 1256):
    ``out[b, j] = idx_j + topk_indices_offset[b]``; short rows give ``offset + 0..len-1`` then -1.
    """
    assert topk == TOPK, "only topk=2048 is supported"
    assert score.dim() == 2
    _check_inputs(score, lengths, row_starts)
    B = score.size(0)
    if not topk_indices_offset.is_cuda or topk_indices_offset.dtype != torch.int32 \
            or topk_indices_offset.dim() != 1 or topk_indices_offset.size(0) != B \
            or not topk_indices_offset.is_contiguous():
        raise RuntimeError("topk_indices_offset must be a contiguous CUDA int32 tensor of size B")
    out = torch.empty((B, TOPK), dtype=torch.int32, device=score.device)
    if B == 0:
        return out
    lib = _native.lib()
    with torch.cuda.device(score.device):
        rc = lib.fftopk_select2048_ragged(
            score.data_ptr(), score.stride(0), B, score.size(1), lengths.data_ptr(),
            row_starts.data_ptr() if row_starts is not None else None, out.data_ptr(),
            topk_indices_offset.data_ptr(), _status_word(score.device).data_ptr(),
            torch.cuda.current_stream().cuda_stream)
    _native.check(rc, "fftopk_select2048_ragged")
    _after_launch(score.device, "fftopk_select2048_ragged")
    return out
