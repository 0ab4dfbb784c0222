"""Indexer logits fused with the top-2048 selection (no counterpart in the reference, whose selector
starts from a finished logit matrix; README.md:24 names the step in front of it).

    logit[b, t] = k_scale[b, t] * sum_h w[b, h] * relu(q[b, h, :] . k[b, t, :])
    64 heads, dimension 128; q and k in bf16, or in fp8 (e4m3) with an optional positive scale per key

``FusedIndexerTopk`` keeps what the C entry point ``fftopk_indexer_topk2048`` needs between calls of
a decode loop: the per-row threshold keys, the logit matrix (``.logits``: written by every call,
read again only for rows without a usable guess) and the candidate workspace."""
from __future__ import annotations

import torch

from . import _native
from .topk_indexer import TOPK, _after_launch, _status_word

HEADS, DIM = 64, 128


def reference_logits(q: torch.Tensor, k: torch.Tensor, w: torch.Tensor, k_scale: torch.Tensor | None = None) -> torch.Tensor:
    """The same formula in plain torch, fp32 arithmetic on the widened operands: q [B, 64, 128],
    k [B, L, 128], w [B, 64] (, k_scale [B, L]) -> [B, L]. For tests."""
    s = torch.einsum("bhd,bld->bhl", q.float(), k.float())
    out = (torch.relu(s) * w.float().unsqueeze(-1)).sum(dim=1)
    return out if k_scale is None else out * k_scale.float()


class FusedIndexerTopk:
    def __init__(self, max_rows: int, max_len: int, device=None):
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        self.b_cap, self.l_cap = int(max_rows), int(max_len)
        lib = _native.lib()
        nbytes = int(lib.fftopk_indexer_workspace_bytes(self.b_cap))
        self._ws = torch.zeros(nbytes + 256, dtype=torch.uint8, device=self.device)  # (zero-filled once: the C entry's contract)
        self._ws_ptr = (self._ws.data_ptr() + 255) & ~255
        self._ws_bytes = nbytes
        self.thresholds = torch.zeros(self.b_cap, dtype=torch.int32, device=self.device)
        self.logits = torch.empty(self.b_cap, self.l_cap, dtype=torch.float32, device=self.device)

    def __call__(self, q: torch.Tensor, k_cache: torch.Tensor, w: torch.Tensor, lengths: torch.Tensor,
                 margin: int = 0, out: torch.Tensor | None = None, k_scale: torch.Tensor | None = None) -> torch.Tensor:
        """q [B, 64, 128] and k_cache [B, Lk, 128] (contiguous; both bfloat16, or both float8_e4m3fn
        with an optional fp32 k_scale [B, Lk] of positive per-key scales), w [B, 64] fp32, lengths
        [B] int32, all on the device -> int32 [B, 2048]: the indices of every row's 2048 largest
        logits (unordered, ties to the lower index, -1 padded for rows of fewer than 2048 keys)."""
        B, Lk = k_cache.size(0), k_cache.size(1)
        fp8 = k_cache.dtype == torch.float8_e4m3fn
        if q.dtype != k_cache.dtype or k_cache.dtype not in (torch.bfloat16, torch.float8_e4m3fn) or w.dtype != torch.float32:
            raise RuntimeError("q and k_cache must both be bfloat16 or both float8_e4m3fn, w float32")
        if k_scale is not None and (not fp8 or k_scale.dtype != torch.float32 or tuple(k_scale.shape) != (B, Lk)
                                    or not k_scale.is_contiguous()):
            raise RuntimeError("k_scale goes with fp8 operands: a contiguous float32 tensor of shape [B, L]")
        if tuple(q.shape) != (B, HEADS, DIM) or k_cache.size(2) != DIM or tuple(w.shape) != (B, HEADS):
            raise RuntimeError("expected q [B, 64, 128], k_cache [B, L, 128], w [B, 64]")
        if not (q.is_contiguous() and k_cache.is_contiguous() and w.is_contiguous() and lengths.is_contiguous()):
            raise RuntimeError("q, k_cache, w and lengths must be contiguous")
        if lengths.dtype != torch.int32 or lengths.numel() != B:
            raise RuntimeError("lengths must be int32 of shape [B]")
        if B > self.b_cap or Lk > self.l_cap:
            raise RuntimeError("batch or length beyond what this object was created for")
        if out is None:
            out = torch.empty((B, TOPK), dtype=torch.int32, device=self.device)
        if B == 0:
            return out
        lib = _native.lib()
        with torch.cuda.device(self.device):
            tail = (B, Lk, lengths.data_ptr(), self.thresholds.data_ptr(), int(margin), self.logits.data_ptr(), self.l_cap,
                    out.data_ptr(), self._ws_ptr, self._ws_bytes, _status_word(self.device).data_ptr(),
                    torch.cuda.current_stream().cuda_stream)
            if fp8:
                rc = lib.fftopk_indexer_topk2048_fp8(q.data_ptr(), k_cache.data_ptr(), Lk,
                                                     None if k_scale is None else k_scale.data_ptr(), Lk, w.data_ptr(), *tail)
            else:
                rc = lib.fftopk_indexer_topk2048(q.data_ptr(), k_cache.data_ptr(), Lk, w.data_ptr(), *tail)
        _native.check(rc, "fftopk_indexer_topk2048")
        _after_launch(self.device, "fftopk_indexer_topk2048")
        return out
