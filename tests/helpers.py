"""Shared helpers for the parity tests."""
from __future__ import annotations

import zlib
from pathlib import Path

import numpy as np
import torch

GOLDEN = Path(__file__).resolve().parent / "golden"


def crc(a: np.ndarray) -> int:
    return zlib.crc32(np.ascontiguousarray(a).view(np.uint8).tobytes()) & 0xFFFFFFFF


def load_golden(name: str):
    """Returns (score [torch, cpu], lengths, row_starts or None, expected [np], value_crc [np])."""
    import workloads

    z = np.load(GOLDEN / f"{name}.npz")
    if "score" in z:
        score = torch.from_numpy(z["score"].copy())
    else:
        score, _ = eval(str(z["gen"]), {"workloads": workloads})
    assert crc(score.numpy()) == int(z["input_crc"]), \
        f"{name}: regenerated input differs from the one the golden vector was made from"
    lengths = torch.from_numpy(z["lengths"].copy())
    rs = torch.from_numpy(z["row_starts"].copy()) if "row_starts" in z else None
    return score, lengths, rs, z["expected"], z["value_crc"]


GOLDEN_NAMES = sorted(p.stem for p in GOLDEN.glob("*.npz"))
