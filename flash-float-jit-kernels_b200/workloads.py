"""Seeded synthetic inputs with the shapes and value distributions of the benchmark configs.

The reference measures this path on synthetic ``randn`` only (benchmark/bench_topk.py:97-104,
seed 42 at :14); no dataset is involved.  Every generator draws on the CPU from a
``torch.Generator`` so that host and device sides of a comparison see identical bits.

Configs (k = 2048 everywhere):
  c1  B=1, L=16384, N(0,1)                                   the CPU-runnable case
  c2  B=1, L in {64K..1M}, sum over 64 heads of w_h*relu(N(0,1)), w_h ~ U(0,1)   decode sweep
  c3  B=64, padded L=131072, ragged lengths in [1024, 131072], N(0,1), padding = -inf
  c4  B=8, L=262144, 70% exact zeros, 25% LogNormal(0,1), 5% copies of the row's k-th value
  c5  B=4, L=1M, N(0,1) with a 0.1% planted N(6,1) tail      context-parallel decode
"""
from __future__ import annotations

import torch

SEED = 42
K = 2048


def _gen(seed: int) -> torch.Generator:
    g = torch.Generator(device="cpu")
    g.manual_seed(seed)
    return g


def c1(seed: int = SEED, L: int = 16384):
    g = _gen(seed)
    score = torch.randn(1, L, generator=g, dtype=torch.float32)
    return score, torch.full((1,), L, dtype=torch.int32)


def c2(L: int = 1 << 20, seed: int = SEED, heads: int = 64, B: int = 1):
    g = _gen(seed)
    w = torch.rand(heads, generator=g, dtype=torch.float32)
    score = torch.zeros(B, L, dtype=torch.float32)
    for h in range(heads):
        score += w[h] * torch.relu(torch.randn(B, L, generator=g, dtype=torch.float32))
    return score, torch.full((B,), L, dtype=torch.int32)


def c3(seed: int = SEED, B: int = 64, L: int = 131072, min_len: int = 1024):
    g = _gen(seed)
    score = torch.randn(B, L, generator=g, dtype=torch.float32)
    lengths = torch.randint(min_len, L + 1, (B,), generator=g, dtype=torch.int32)
    col = torch.arange(L).unsqueeze(0)
    score.masked_fill_(col >= lengths.unsqueeze(1).to(torch.int64), float("-inf"))
    return score, lengths


def c4(seed: int = SEED, B: int = 8, L: int = 262144):
    g = _gen(seed)
    u = torch.rand(B, L, generator=g, dtype=torch.float32)
    logn = torch.exp(torch.randn(B, L, generator=g, dtype=torch.float32))
    score = torch.where(u < 0.70, torch.zeros(()), logn)
    dup = u >= 0.95
    base = score.masked_fill(dup, float("-inf"))
    kth = torch.topk(base, K, dim=-1).values[:, K - 1:K]  # the row's current k-th largest value
    score = torch.where(dup, kth.expand(B, L), score)
    return score.contiguous(), torch.full((B,), L, dtype=torch.int32)


def c5(seed: int = SEED, B: int = 4, L: int = 1 << 20):
    g = _gen(seed)
    score = torch.randn(B, L, generator=g, dtype=torch.float32)
    mask = torch.rand(B, L, generator=g, dtype=torch.float32) < 0.001
    tail = 6.0 + torch.randn(B, L, generator=g, dtype=torch.float32)
    score = torch.where(mask, tail, score)
    return score.contiguous(), torch.full((B,), L, dtype=torch.int32)


def algorithmic_bytes(lengths, L: int, k: int = K) -> int:
    """Bytes one call must move: every valid logit read once, lengths read, indices written."""
    ln = torch.clamp(lengths.to(torch.int64), 0, L)
    B = int(lengths.numel())
    return int(4 * ln.sum().item()) + 4 * B + 4 * k * B
