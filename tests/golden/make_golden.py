"""Generate the golden vectors in this directory.

Run from the repository root, in the image the tests run in:
    python tests/golden/make_golden.py

Each ``*.npz`` holds a seeded input (or the generator arguments that rebuild it, plus a checksum
of the generated bits) and the expected result of the reference's own ground truth on it:
``torch.topk(score[:, :len], 2048, sorted=False)`` values (benchmark/bench_topk.py:25-42 of the
reference) and the index set of a stable descending ``torch.sort`` (lower index first among
equal values).  torch is the third-party dependency the reference defines correctness against;
the reference itself ships no golden vectors for this path.
"""
from __future__ import annotations

import sys
import zlib
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
REPO = HERE.parent.parent
sys.path.insert(0, str(REPO / "flash-float-jit-kernels_b200"))
sys.path.insert(0, str(REPO))

import workloads  # noqa: E402
from oracle import topk_oracle  # noqa: E402

K = 2048


def crc(a: np.ndarray) -> int:
    return zlib.crc32(np.ascontiguousarray(a).view(np.uint8).tobytes()) & 0xFFFFFFFF


def save(name, score, lengths, row_starts=None, store_input=False, gen=None):
    idx, vals = topk_oracle.torch_oracle(score, lengths.numpy(), K,
                                         None if row_starts is None else row_starts.numpy())
    # per-row checksum of torch.topk's value multiset (sorted descending)
    vcrc = np.array([0 if v is None else crc(v) for v in vals], dtype=np.uint32)
    payload = dict(
        expected=idx, value_crc=vcrc, lengths=lengths.numpy(),
        input_crc=np.uint32(crc(score.numpy())), shape=np.array(score.shape, dtype=np.int64),
        gen=np.str_(gen or ""), torch_version=np.str_(torch.__version__),
    )
    if row_starts is not None:
        payload["row_starts"] = row_starts.numpy()
    if store_input:
        payload["score"] = score.numpy()
    np.savez_compressed(HERE / f"{name}.npz", **payload)
    print(name, tuple(score.shape), "->", (HERE / f"{name}.npz").stat().st_size, "bytes")


def main():
    # C1: the CPU-runnable case, input stored bit for bit
    s, l = workloads.c1()
    save("c1_b1_l16384", s, l, store_input=True, gen="workloads.c1()")
    # reference benchmark recipe: randn min-max normalised to [0,255), with row_starts
    # (benchmark/bench_topk.py:97-111), B=2, seq_len 16384 inside rows of 20000
    g = torch.Generator().manual_seed(42)
    s = torch.randn(2, 20000, generator=g)
    s = (s - s.min()) / (s.max() - s.min() + 1e-6) * 255
    rs = torch.randint(0, 2048, (2,), generator=g, dtype=torch.int32)
    save("refbench_b2_l16384_rowstarts", s, torch.full((2,), 16384, dtype=torch.int32), rs,
         store_input=True, gen="randn(2,20000) seed 42, min-max to [0,255), row_starts randint(0,2048)")
    # reduced-size instances of the other configs (inputs rebuilt from the generators)
    s, l = workloads.c2(L=65536)
    save("c2_b1_l65536", s, l, gen="workloads.c2(L=65536)")
    s, l = workloads.c3(B=8, L=32768)
    save("c3_b8_l32768_ragged", s, l, gen="workloads.c3(B=8, L=32768)")
    s, l = workloads.c4(B=2, L=65536)
    save("c4_b2_l65536_ties", s, l, gen="workloads.c4(B=2, L=65536)")
    s, l = workloads.c5(B=1, L=262144)
    save("c5_b1_l262144_tail", s, l, gen="workloads.c5(B=1, L=262144)")
    # special values: NaN, +-inf, +-0, denormals, duplicates
    g = torch.Generator().manual_seed(7)
    s = torch.randn(2, 8192, generator=g)
    s[0, ::7] = 0.0
    s[0, 3::11] = -0.0
    s[0, 5::97] = float("inf")
    s[0, 6::89] = float("-inf")
    s[0, 8::301] = float("nan")
    s[1] = torch.round(s[1] * 4) / 4  # heavy duplicates
    s[1, 100:140] = 1e-42  # denormals
    save("special_values_b2_l8192", s, torch.tensor([8192, 8000], dtype=torch.int32),
         store_input=True, gen="see make_golden.py")


if __name__ == "__main__":
    main()
