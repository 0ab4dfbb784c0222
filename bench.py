#!/usr/bin/env python
"""Benchmark of the top-2048 selector (drop-in for fast_topk_v3) on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port P bench.py --gpus N --steps K --warmup W

Prints ONE JSON line (rank 0). A step is one call of the op on one batch of the ragged batched
decode workload (B=64 rows, padded L=131072, valid lengths uniform in [1024, 131072], fp32
N(0,1) logits, -inf padding, k=2048). With N GPUs every rank processes its own 64-row batch
(rows are independent: no collective on the data path), so `value` = 64*N rows per step / time
per step.

Timed region: the K-step sequence is captured in a CUDA graph (several repetitions of it per
graph when K is small, so that a graph holds >= 200 calls) and the graph is replayed until the
region lasts >= 50 ms; `ms_per_step` = region / calls in it, `replays` = how often the K-step
sequence ran, `gpu_launches` = calls in the region. A step is ~5 us, so K steps alone (0.1 ms at
K = 20) would measure the fill and drain of the launch pipeline, not the kernel; that figure is
kept as `cold_start_ms_per_step`.

  value      rows/s with the inputs resident in HBM, eight 32 MiB input buffers rotated so that no
             step finds its input in L2 (256 MiB > 126 MB L2). The steps are independent batches
             and the library's throughput mode is on (fftopk_set_overlap: consecutive calls are
             programmatic dependent launches, so a call starts filling the SMs that the short rows
             of the previous call have already left; every step has its own output buffer)
  serial     the same K steps with the default, strictly serialised launches: us per call
  e2e        the same metric through the host-buffer entry point (fast_topk_v3_host =
             fftopk_select2048_host): pinned-memory H2D copy of every row's valid prefix, the
             kernel, D2H copy of the indices, all inside the timed region
  roofline   algorithmic bytes per launch / measured launch time, against the measured HBM peak
  latency    p50 microseconds per call at B=1 for the decode sweep L = 64K .. 1M (the other half of
             the headline metric), L2-warm (the reference's own method; also as a fraction of the
             L2 read bandwidth measured with the library's probe) and with rotated buffers
  decode_loop  B=1, one logit appended per step: us per step cold and with the warm start that carries
             the previous step's threshold (fast_topk_v3_warm)
  fused_indexer  B=1: indexer logits on the tensor cores fused with the selection
             (fftopk_indexer_topk2048), us per call with and without a threshold guess, GB/s of
             key cache read against the HBM peak
  large_batch  one serialised call at B=256 and B=512 of the same ragged distribution: the rate a
             single call reaches when the batch alone fills the device
  context_parallel  (N > 1) config 5 through the three context-parallel variants: first checked
             bit-exact against single-device torch (every rank, also on the tie-stress config),
             then timed; timings are null when the check fails
  cpu_baseline  torch.topk on the host cores on the same batch (what the reference's benchmark
             uses as ground truth, benchmark/bench_topk.py:25-42)

`--impl reference` times that CPU path alone, in the same JSON shape.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time
from pathlib import Path

REPO = Path(__file__).resolve().parent
sys.path.insert(0, str(REPO / "flash-float-jit-kernels_b200"))
sys.path.insert(0, str(REPO))

import numpy as np  # noqa: E402
import torch  # noqa: E402

import workloads  # noqa: E402

K = 2048
METRIC = "rows/s at B=64 (top-2048 per row, ragged batched decode)"
WORKLOAD = "ragged batched decode: B=64, padded L=131072, lengths U[1024,131072], fp32 N(0,1), k=2048"
N_ROTATE = 8
FALLBACK_HBM_GBS = 6650.0
MIN_REGION_S = 0.05      # a timed region lasts at least this long
MIN_GRAPH_CALLS = 200    # a captured graph holds at least this many calls
# dram__bytes_read.sum + dram__bytes_write.sum of one select2048 launch on this workload, from the
# ncu capture of the throughput plan (profiles/select2048_ragged_b64.md)
NCU_TRAFFIC_BYTES_PER_LAUNCH = 16775253  # throughput plan, mean of 3 captured launches (16.775424, 16.775168, 16.775168 MB read; 0 written)


def bench_config():
    """The `config` object of the JSON line: the workload only, identical in both arms."""
    return {"workload": WORKLOAD, "rows_per_gpu": 64, "padded_L": 131072, "k": K}


def measured_peak_gbs():
    p = REPO / "MEASURED_PEAKS.json"
    try:
        return float(json.loads(p.read_text())["hbm_gbs"]), "measured (MEASURED_PEAKS.json)"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback"


class ClockSampler:
    """Polls NVML (read-only) for SM clock and throttle reasons while a region runs."""

    def __init__(self, index: int, period_s: float = 0.002):
        self.index, self.period = index, period_s
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = int(pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM))
        except Exception:
            self.nv = None

    def _loop(self):
        nv = self.nv
        names = {
            "hw_slowdown": getattr(nv, "nvmlClocksEventReasonHwSlowdown", 0x8),
            "hw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonHwThermalSlowdown", 0x40),
            "sw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonSwThermalSlowdown", 0x20),
            "sw_power_cap": getattr(nv, "nvmlClocksEventReasonSwPowerCap", 0x4),
        }
        get_reasons = getattr(nv, "nvmlDeviceGetCurrentClocksEventReasons", None) or \
            getattr(nv, "nvmlDeviceGetCurrentClocksThrottleReasons", None)
        while not self._stop.is_set():
            try:
                self.samples.append(int(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM)))
                if get_reasons is not None:
                    mask = int(get_reasons(self.h))
                    for name, bit in names.items():
                        if mask & bit:
                            self.reasons.add(name)
            except Exception:
                pass
            time.sleep(self.period)

    def __enter__(self):
        if self.nv is not None:
            self._thread = threading.Thread(target=self._loop, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=1.0)

    def summary(self, note: str = ""):
        return {
            "sm_mhz": float(np.median(self.samples)) if self.samples else None,
            "sm_max_mhz": self.max_mhz,
            "reasons": sorted(self.reasons),
            "samples": len(self.samples),
            "note": note,
        }


def physical_gpu_index(local_rank: int) -> int:
    vis = os.environ.get("CUDA_VISIBLE_DEVICES")
    if vis:
        try:
            return int(vis.split(",")[local_rank])
        except Exception:
            return local_rank
    return local_rank


# ----------------------------------------------------------------------------------------------
# CPU side: the reference's own ground truth on the host cores
# ----------------------------------------------------------------------------------------------
def cpu_topk_batch(score: torch.Tensor, lengths: torch.Tensor) -> None:
    """torch.topk(score[b, :len], 2048, sorted=False) per row (benchmark/bench_topk.py:25-42);
    rows with len <= k have nothing to select."""
    for b in range(score.size(0)):
        n = int(lengths[b])
        if n > K:
            torch.topk(score[b, :n], K, dim=-1, sorted=False)


def time_cpu(score, lengths, steps: int, warmup: int):
    torch.set_num_threads(os.cpu_count() or 1)
    for _ in range(warmup):
        cpu_topk_batch(score, lengths)
    t0 = time.perf_counter()
    for _ in range(steps):
        cpu_topk_batch(score, lengths)
    dt = time.perf_counter() - t0
    return dt / steps


def reference_arm(args, rank: int) -> None:
    """`--impl reference`: the CPU torch.topk path alone, same workload, rank 0 only."""
    if rank != 0:
        return
    score, lengths = workloads.c3()
    rows = score.size(0)
    # bound the run to a few minutes: a 64-row step takes 20-50 ms on 8 cores
    est = 0.05 * (args.steps + args.warmup)
    rows_per_step = rows if est < 150 else max(1, int(rows * 150 / est))
    s, ln = score[:rows_per_step], lengths[:rows_per_step]
    sec = time_cpu(s, ln, args.steps, args.warmup)
    value = rows_per_step / sec
    cores = torch.get_num_threads()
    sample = f"rows 0..{rows_per_step - 1} of the 64-row batch per step, {args.steps} steps"
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": "rows/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": sec * 1e3 * rows / rows_per_step,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic", "config": bench_config(), "run": {"where": "host cores, torch.topk"},
        "cpu_baseline": {"value": value, "unit": "rows/s", "cores": cores, "kind": "port", "sample": sample,
                         "what": "torch.topk(score[b,:len], 2048, sorted=False) per row, the reference "
                                 "benchmark's ground truth"},
        "e2e": {"value": value, "unit": "rows/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ----------------------------------------------------------------------------------------------
# GPU side
# ----------------------------------------------------------------------------------------------
def capture_steps(fn, n: int, stream: torch.cuda.Stream) -> torch.cuda.CUDAGraph:
    """A CUDA graph of n back-to-back calls fn(i): the host cannot enqueue a ~20 us kernel fast
    enough from Python, a graph replays them at device speed (the reference times the same way,
    triton do_bench_cudagraph, benchmark/bench_topk.py:202)."""
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(stream):
        with torch.cuda.graph(graph, stream=stream):
            for i in range(n):
                fn(i)
    return graph


def time_graph(graph, stream, replays: int = 1):
    """Device time of `replays` launches of the graph, CUDA events on the launching stream."""
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with torch.cuda.stream(stream):
        e0.record(stream)
        for _ in range(replays):
            graph.replay()
        e1.record(stream)
    e1.synchronize()
    return e0.elapsed_time(e1) * 1e-3  # seconds


def timed_region(step, steps: int, stream, min_s: float = MIN_REGION_S):
    """Captures the `steps`-step sequence - repeated so that the graph holds >= MIN_GRAPH_CALLS calls
    - and returns (graph, calls per graph, replays needed for a region of >= min_s seconds)."""
    reps_in_graph = max(1, -(-MIN_GRAPH_CALLS // steps))
    calls = reps_in_graph * steps
    graph = capture_steps(step, calls, stream)
    time_graph(graph, stream)  # upload + warm-up
    t1 = min(time_graph(graph, stream) for _ in range(2))
    replays = max(1, int(np.ceil(min_s / max(t1, 1e-7))))
    return graph, calls, reps_in_graph, replays


def measure_l2_read_gbs(dev, stream):
    """Read bandwidth of L2-resident data, all SMs reading (the library's probe): GB/s for a 4 MiB
    and a 32 MiB buffer; the HBM figure from a 1 GiB buffer alongside."""
    import ctypes

    from jit_kernel import _native
    lib = _native.lib()
    sink = torch.zeros(1, dtype=torch.int32, device=dev)
    out = {}
    for name, nbytes, to_read in (("l2_4MiB", 4 << 20, 40 << 30), ("l2_32MiB", 32 << 20, 40 << 30),
                                  ("hbm_1GiB", 1 << 30, 16 << 30)):
        buf = torch.empty(nbytes // 4, dtype=torch.float32, device=dev).normal_()
        got = ctypes.c_size_t()
        best = 0.0
        with torch.cuda.stream(stream):
            for rep in range(4):
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record(stream)
                _native.check(lib.fftopk_probe_read_bandwidth(buf.data_ptr(), nbytes, to_read, sink.data_ptr(),
                                                              ctypes.byref(got), stream.cuda_stream), "probe")
                e1.record(stream)
                e1.synchronize()
                if rep:
                    best = max(best, got.value / (e0.elapsed_time(e1) * 1e-3) / 1e9)
        out[name] = best
        del buf
    return out


def measure_h2d_gbs(dev, stream, nbytes: int = 64 << 20):
    """Pinned host -> device copy bandwidth of this box (one cudaMemcpyAsync of 64 MiB, best of 5)."""
    h = torch.empty(nbytes, dtype=torch.uint8).pin_memory()
    d = torch.empty(nbytes, dtype=torch.uint8, device=dev)
    best = 0.0
    with torch.cuda.stream(stream):
        for rep in range(6):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            d.copy_(h, non_blocking=True)
            e1.record(stream)
            e1.synchronize()
            if rep:
                best = max(best, nbytes / (e0.elapsed_time(e1) * 1e-3) / 1e9)
    return best


def latency_sweep(dev, stream, fast_topk, l2_gbs=None):
    """p50 us per call at B=1 over the decode sweep; warm = same buffer every call (L2-resident,
    the reference's method), cold = buffers rotated over > L2 bytes."""
    out = {}
    idx = torch.empty(1, K, dtype=torch.int32, device=dev)
    for L in (65536, 131072, 262144, 524288, 1048576):
        score, lengths = workloads.c2(L=L)
        ld = lengths.to(dev)
        n_cold = max(2, min(64, (160 << 20) // (4 * L) + 1))
        bufs = [score.to(dev).clone() for _ in range(n_cold)]
        res = {}
        for name, nbuf in (("warm", 1), ("cold", n_cold)):
            reps = max(20, nbuf)
            with torch.cuda.stream(stream):
                for i in range(min(reps, 8)):
                    fast_topk(bufs[i % nbuf], idx, ld)
            stream.synchronize()
            g = capture_steps(lambda i: fast_topk(bufs[i % nbuf], idx, ld), reps, stream)
            ts = sorted(time_graph(g, stream) / reps * 1e6 for _ in range(15))
            res[name] = {"p50_us": ts[len(ts) // 2], "p20_us": ts[len(ts) // 5], "p80_us": ts[(4 * len(ts)) // 5]}
        nbytes = workloads.algorithmic_bytes(lengths, L)
        res["bytes"] = nbytes
        res["cold_gbs"] = nbytes / res["cold"]["p50_us"] / 1e3
        res["warm_gbs"] = nbytes / res["warm"]["p50_us"] / 1e3
        if l2_gbs:
            res["warm_frac_l2"] = res["warm_gbs"] / l2_gbs
        out[str(L)] = res
        del bufs
    return out


def decode_loop_leg(dev, stream):
    """A decode loop at B=1: the same row, one logit appended per step (the decode-sweep
    distribution), selected cold every step (fast_topk_v3's path) and with the warm start that
    carries the previous step's threshold key (fast_topk_v3_warm). 40 steps per CUDA graph; the
    graph's first node restores the threshold of the step before the first, so every replay is the
    same loop. us per step, p50 of 15 replays."""
    from jit_kernel.topk_indexer import fast_topk, fast_topk_v3_warm

    out = {}
    steps = 40
    idx = torch.empty(1, K, dtype=torch.int32, device=dev)
    for L in (131072, 1048576):
        score, _ = workloads.c2(L=L + steps)
        sd = score.to(dev)
        lens = [torch.full((1,), L + t, dtype=torch.int32, device=dev) for t in range(steps + 1)]
        thr = torch.zeros(1, dtype=torch.int32, device=dev)
        with torch.cuda.stream(stream):
            fast_topk_v3_warm(sd, lens[0], K, thr, out=idx)  # the step before the loop: seeds the threshold
            for t in range(1, 4):
                fast_topk(sd, idx, lens[t])
        stream.synchronize()
        seed = thr.clone()

        def warm_steps(_):
            thr.copy_(seed)
            for t in range(1, steps + 1):
                fast_topk_v3_warm(sd, lens[t], K, thr, out=idx)

        def cold_steps(_):
            for t in range(1, steps + 1):
                fast_topk(sd, idx, lens[t])

        res = {}
        for name, fn in (("cold", cold_steps), ("warm", warm_steps)):
            with torch.cuda.stream(stream):
                fn(0)
            stream.synchronize()
            g = capture_steps(fn, 1, stream)
            ts = sorted(time_graph(g, stream) / steps * 1e6 for _ in range(15))
            res[name + "_us_per_step"] = ts[len(ts) // 2]
        out[str(L)] = res
    return out


def indexer_leg(dev, stream, peak_gbs):
    """The step in front of the selector, fused with it (fftopk_indexer_topk2048[_fp8]): B=1 decode
    rows, q [64, 128] and key cache [L, 128] in bf16 and in fp8 (e4m3, one fp32 scale per key). us
    per call with a standing threshold guess (logits filtered in the tensor-core kernel's epilogue,
    never written) and without one (logits written, selector on them), beside torch's own einsum +
    relu + weighted sum for the logits alone (bf16). The roofline of the producer is reading the key
    cache once: 256 B per key in bf16, 128 + 4 B in fp8."""
    from jit_kernel.indexer import FusedIndexerTopk, reference_logits

    out = {}
    for fmt in ("bf16", "fp8"):
        for L in (131072, 1048576):
            g = torch.Generator(device="cpu").manual_seed(L)
            dt = torch.bfloat16 if fmt == "bf16" else torch.float8_e4m3fn
            key_bytes = L * (256 if fmt == "bf16" else 132)
            q = (torch.randn(1, 64, 128, generator=g) * 0.5).to(dt).to(dev)
            nbuf = max(2, (300 << 20) // key_bytes + 1)  # rotate key caches over more than L2
            ks = [(torch.randn(1, L, 128, generator=g) * 0.5).to(dt).to(dev) for _ in range(nbuf)]
            scale = (torch.rand(1, L, generator=g) + 0.5).to(dev) if fmt == "fp8" else None
            w = torch.rand(1, 64, generator=g).to(dev)
            ln = torch.full((1,), L, dtype=torch.int32, device=dev)
            fs = [FusedIndexerTopk(1, L, dev) for _ in range(nbuf)]  # one threshold state per cache
            res = torch.empty(1, K, dtype=torch.int32, device=dev)
            with torch.cuda.stream(stream):
                for f, k in zip(fs, ks):
                    f(q, k, w, ln, out=res, k_scale=scale)  # seeds the thresholds (and sets kernel attributes)
            stream.synchronize()
            n = 2 * nbuf
            r = {"key_cache_bytes": key_bytes, "rotated_caches": nbuf}
            for name in ("warm", "cold"):
                def call(i):
                    f = fs[i % nbuf]
                    if name == "cold":
                        f.thresholds.zero_()
                    f(q, ks[i % nbuf], w, ln, out=res, k_scale=scale)
                with torch.cuda.stream(stream):
                    call(0)
                stream.synchronize()
                gr = capture_steps(call, n, stream)
                ts = sorted(time_graph(gr, stream) / n * 1e6 for _ in range(9))
                r[name + "_us_per_call"] = ts[len(ts) // 2]
                del gr
                if name == "cold":  # leave the states warm again
                    with torch.cuda.stream(stream):
                        for f, k in zip(fs, ks):
                            f(q, k, w, ln, out=res, k_scale=scale)
                    stream.synchronize()
            r["warm_gbs"] = key_bytes / r["warm_us_per_call"] / 1e3
            r["warm_frac_hbm"] = r["warm_gbs"] / peak_gbs
            if fmt == "bf16":
                with torch.cuda.stream(stream):
                    reference_logits(q, ks[0], w)
                stream.synchronize()
                gr = capture_steps(lambda i: reference_logits(q, ks[i % nbuf], w), nbuf, stream)
                ts = sorted(time_graph(gr, stream) / nbuf * 1e6 for _ in range(5))
                r["torch_logits_only_us"] = ts[len(ts) // 2]
                del gr
            out[f"{fmt}_{L}"] = r
            del ks, fs
    # a decode batch: B=64 rows of the bench's ragged lengths, every row with its own key cache
    # (2.1 GB in bf16: nothing stays in L2 from call to call)
    _, lengths = workloads.c3()  # (only the lengths are wanted)
    B, L = int(lengths.numel()), 131072
    ln = lengths.to(dev)
    n_keys = int(lengths.sum())
    for fmt in ("bf16", "fp8"):
        dt = torch.bfloat16 if fmt == "bf16" else torch.float8_e4m3fn
        g = torch.Generator(device=dev).manual_seed(7)
        q = (torch.randn(B, 64, 128, generator=g, device=dev) * 0.5).to(dt)
        k = torch.empty(B, L, 128, dtype=dt, device=dev)
        for b0 in range(0, B, 8):  # (in slices: the fp32 draw of the whole cache would be 4.3 GB)
            k[b0:b0 + 8] = (torch.randn(8, L, 128, generator=g, device=dev) * 0.5).to(dt)
        scale = (torch.rand(B, L, generator=g, device=dev) + 0.5) if fmt == "fp8" else None
        w = torch.rand(B, 64, generator=g, device=dev)
        f = FusedIndexerTopk(B, L, dev)
        res = torch.empty(B, K, dtype=torch.int32, device=dev)
        with torch.cuda.stream(stream):
            f(q, k, w, ln, out=res, k_scale=scale)
        stream.synchronize()
        gr = capture_steps(lambda i: f(q, k, w, ln, out=res, k_scale=scale), 4, stream)
        ts = sorted(time_graph(gr, stream) / 4 * 1e6 for _ in range(7))
        del gr
        key_bytes = n_keys * (256 if fmt == "bf16" else 132)
        us = ts[len(ts) // 2]
        # the selection against torch.topk on the logits the kernel wrote (values: ties may differ in index)
        lg = f.logits[:B, :L].clone()
        lg[torch.arange(L, device=dev).unsqueeze(0) >= ln.unsqueeze(1)] = float("-inf")
        want = torch.topk(lg, K, dim=1).values.sort(dim=1).values
        got = torch.gather(lg, 1, res.long().clamp_min(0)).sort(dim=1).values
        long_rows = ln > K
        same = bool(torch.equal(want[long_rows], got[long_rows]))
        del lg, want, got
        out[f"{fmt}_B{B}_ragged"] = {"keys": n_keys, "key_cache_bytes": key_bytes, "warm_us_per_call": us,
                                     "warm_gbs": key_bytes / us / 1e3, "warm_frac_hbm": key_bytes / us / 1e3 / peak_gbs,
                                     "rows_per_s": B / us * 1e6,
                                     "parity": "values bit-exact vs torch.topk on the written logits" if same else "MISMATCH"}
        del k, f
    return out


def indexer_drift_leg(dev, stream):
    """The fused indexer in a decode loop whose QUERY changes from step to step (q_t = q_{t-1} plus
    noise, at constant norm; bf16, L = 131072 keys plus one per step): how often the threshold carried
    from the previous step still holds (a miss sends the row through the selector in the same call)
    and the mean time per step, for three noise levels and three margins. A margin is subtracted
    from the carried key: 2^18 is about 3 % of the logit's value, 2^20 about 12 %. (One key cache
    of 33 MB, which stays in L2 from step to step - unlike the rotated caches of indexer_leg.)"""
    from jit_kernel import _native
    from jit_kernel.indexer import FusedIndexerTopk
    from jit_kernel.topk_indexer import _status_word

    L0, steps = 131072, 64
    g = torch.Generator(device=dev).manual_seed(11)
    k = (torch.randn(1, L0 + steps, 128, generator=g, device=dev) * 0.5).to(torch.bfloat16)
    w = torch.rand(1, 64, generator=g, device=dev)
    lens = [torch.full((1,), L0 + t, dtype=torch.int32, device=dev) for t in range(steps + 1)]
    res = torch.empty(1, K, dtype=torch.int32, device=dev)
    status = _status_word(dev)
    out = {}
    for noise in (0.0, 0.05, 0.2):
        q = torch.randn(1, 64, 128, generator=g, device=dev) * 0.5
        norm = q.norm()
        qs = [q.to(torch.bfloat16)]
        for _ in range(steps):
            q = q + noise * 0.5 * torch.randn(1, 64, 128, generator=g, device=dev)
            q = q * (norm / q.norm())
            qs.append(q.to(torch.bfloat16))
        row = {}
        for margin in (0, 1 << 18, 1 << 20):
            f = FusedIndexerTopk(1, L0 + steps, dev)
            with torch.cuda.stream(stream):
                f(qs[0], k, w, lens[0], out=res)
            stream.synchronize()
            seed = f.thresholds.clone()
            misses = 0
            for t in range(1, steps + 1):
                status.zero_()
                with torch.cuda.stream(stream):
                    f(qs[t], k, w, lens[t], margin=margin, out=res)
                stream.synchronize()
                misses += 1 if (int(status.item()) & _native.ST_GUESS_MISSED) else 0
            status.zero_()

            def loop(_):
                f.thresholds.copy_(seed)
                for t in range(1, steps + 1):
                    f(qs[t], k, w, lens[t], margin=margin, out=res)

            gr = capture_steps(loop, 1, stream)
            ts = sorted(time_graph(gr, stream) / steps * 1e6 for _ in range(7))
            del gr
            status.zero_()
            row[f"margin_{margin}"] = {"miss_rate": misses / steps, "us_per_step": ts[len(ts) // 2]}
        out[f"noise_{noise}"] = row
    return out


def large_batch_leg(dev, stream, fast_topk, peak_gbs):
    """One serialised call (default launch mode, no overlap between calls) on a batch large enough
    to fill the device by itself: B=256 and B=512 rows of the bench's ragged distribution, inputs
    larger than L2 (two rotated buffers)."""
    L = 131072
    out = []
    for B in (256, 512):
        g = torch.Generator().manual_seed(workloads.SEED + B)
        lengths = torch.randint(1024, L + 1, (B,), generator=g, dtype=torch.int32)
        ld = lengths.to(dev)
        bufs = []
        for i in range(2):
            torch.manual_seed(1234 + i)
            bufs.append(torch.randn(B, L, dtype=torch.float32, device=dev))
        res = torch.empty(B, K, dtype=torch.int32, device=dev)
        with torch.cuda.stream(stream):
            for i in range(3):
                fast_topk(bufs[i % 2], res, ld)
        stream.synchronize()
        n = 20
        gr = capture_steps(lambda i: fast_topk(bufs[i % 2], res, ld), n, stream)
        time_graph(gr, stream)
        sec = min(time_graph(gr, stream) for _ in range(5)) / n
        nbytes = workloads.algorithmic_bytes(lengths, L)
        out.append({"B": B, "us_per_call": sec * 1e6, "rows_per_s": B / sec, "gbs": nbytes / sec / 1e9,
                    "frac": nbytes / sec / 1e9 / peak_gbs, "bytes": nbytes})
        del bufs, gr
    return out


class TorchGroundTruth:
    """Single-device ground truth of a batch, computed here with torch alone: the k largest of every
    full row, equal values resolved to the lower index (stable descending sort), and as a second
    statement the value multiset of torch.topk (north_star: 'bit-exact against single-device
    torch.topk'; the check style of benchmark/bench_topk.py:55-87)."""

    def __init__(self, score: torch.Tensor, lengths: torch.Tensor):
        self.score = score
        self.rows = []
        for b in range(score.size(0)):
            n = int(lengths[b])
            row = score[b, :n]
            want = torch.sort(torch.sort(row, descending=True, stable=True).indices[:K]).values
            vals = torch.sort(torch.topk(row, min(n, K)).values).values
            assert torch.equal(torch.sort(row[want]).values, vals)  # the two statements agree
            self.rows.append((want, vals))

    def matches(self, got: torch.Tensor) -> bool:
        got = got.cpu()
        for b, (want, vals) in enumerate(self.rows):
            have = torch.sort(got[b][got[b] >= 0].to(torch.int64)).values
            if have.numel() != want.numel() or not torch.equal(have, want):
                return False
            if not torch.equal(torch.sort(self.score[b][have]).values, vals):
                return False
        return True


def context_parallel_leg(dev, rank: int, world: int):
    """Config 5: B=4, L=1M split evenly over the ranks; local select, exchange, merge. Variants:
    NCCL all-gather + merge kernel; the fused path over IPC-mapped peer buffers - ONE kernel per
    rank that selects, publishes, pulls the peers' candidates and merges - called eagerly and as a
    replayed CUDA graph; and the two-kernel form of the fused path (selection with publication,
    then a merge kernel that waits and pulls) as a replayed graph. Each variant is first checked on
    every rank against the single-device result (config 5 and the tie-stress config 4 at B=2,
    L=131072), outside every timed region; then timed with CUDA events, max over ranks."""
    import torch.distributed as dist

    from jit_kernel.distributed import FusedContextParallelTopk, fast_topk_v3_context_parallel, local_lengths
    from jit_kernel.topk_indexer import kernel_status

    def all_ok(flag: bool) -> bool:
        t = torch.tensor([1 if flag else 0], dtype=torch.int32, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MIN)
        return bool(t.item())

    score, lengths = workloads.c5()
    B = score.size(0)
    Ls = score.size(1) // world
    shard = score[:, rank * Ls:(rank + 1) * Ls].contiguous().to(dev)
    lens_dev = local_lengths(lengths, Ls, rank).to(dev)
    t_score, t_len = workloads.c4(B=2, L=131072)
    t_Ls = t_score.size(1) // world
    t_shard = t_score[:, rank * t_Ls:(rank + 1) * t_Ls].contiguous().to(dev)
    fused = FusedContextParallelTopk(max_rows=B)
    fused2 = FusedContextParallelTopk(max_rows=B, single_launch=False)
    out = {"workload": f"B=4, L=1048576 over {world} GPUs, k=2048", "parity": {}}
    truth, t_truth = TorchGroundTruth(score, lengths), TorchGroundTruth(t_score, t_len)

    # ---- parity first, outside every timed region ------------------------------------------------
    par = out["parity"]
    got = fast_topk_v3_context_parallel(shard, lengths, K)
    par["nccl"] = "bit-exact" if all_ok(truth.matches(got)) else "MISMATCH"
    ok = True
    for _ in range(3):
        ok = truth.matches(fused(shard, lengths)) and ok
    par["fused"] = "bit-exact" if all_ok(ok) else "MISMATCH"
    ok = t_truth.matches(fast_topk_v3_context_parallel(t_shard, t_len, K))
    ok = t_truth.matches(fused(t_shard, t_len)) and ok
    ok = t_truth.matches(fused2(t_shard, t_len)) and ok
    par["ties"] = "bit-exact" if all_ok(ok) else "MISMATCH"
    # the fused path as a replayed CUDA graph (its epochs live on the device): no Python between the
    # kernels; replayed several times so that both halves of the comm buffer are used
    res = torch.empty(B, K, dtype=torch.int32, device=dev)
    side = torch.cuda.Stream(device=dev)
    graphs = {}
    for name, obj in (("fused_graph", fused), ("two_launch_graph", fused2)):
        obj.run_into(shard, lens_dev, res)  # (first use of this path outside the capture)
        torch.cuda.synchronize()
        dist.barrier()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.stream(side):
            with torch.cuda.graph(graph, stream=side):
                obj.run_into(shard, lens_dev, res)
        dist.barrier()
        ok = True
        for _ in range(4):
            res.fill_(-5)
            graph.replay()
            torch.cuda.synchronize()
            ok = truth.matches(res) and ok
            dist.barrier()
        par[name] = "bit-exact" if all_ok(ok) else "MISMATCH"
        graphs[name] = graph
    all_exact = all(v == "bit-exact" for v in par.values())

    # ---- timing ----------------------------------------------------------------------------------
    reps = 50
    for name, fn in (("nccl_allgather_merge", lambda: fast_topk_v3_context_parallel(shard, lengths, K)),
                     ("fused_peer_merge", lambda: fused(shard, lengths)),
                     ("fused_peer_merge_graph", graphs["fused_graph"].replay),
                     ("fused_two_launch_graph", graphs["two_launch_graph"].replay)):
        for _ in range(5):
            fn()
        torch.cuda.synchronize()
        dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            fn()
        e1.record()
        e1.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) / reps * 1e3], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        out[name + "_us_per_call"] = float(t.item()) if all_exact else None
    torch.cuda.synchronize()
    st = torch.tensor([kernel_status(dev)], dtype=torch.int32, device=dev)
    dist.all_reduce(st, op=dist.ReduceOp.MAX)
    out["kernel_status"] = int(st.item())  # 0: no bounded wait on a peer ran out, no internal error
    if out["kernel_status"] != 0:
        for name in ("nccl_allgather_merge", "fused_peer_merge", "fused_peer_merge_graph", "fused_two_launch_graph"):
            out[name + "_us_per_call"] = None
    out["single_launch"] = bool(fused.single_launch)
    fused.close()
    fused2.close()
    return out


def ours_arm(args, rank: int, local_rank: int, world: int) -> None:
    import torch.distributed as dist

    from jit_kernel import _native
    from jit_kernel.topk_indexer import fast_topk, fast_topk_v3, kernel_status

    if not torch.cuda.is_available():
        raise RuntimeError("bench.py measures the CUDA path and there is no CUDA device; there is no CPU fallback")
    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    stream = torch.cuda.Stream(device=dev)
    steps, warmup = max(1, args.steps), max(args.warmup, 3)

    # ---- workload: every rank its own 64-row batch, N_ROTATE device copies with different data --
    score, lengths = workloads.c3(seed=workloads.SEED + rank)
    B, L = score.shape
    ld = lengths.to(dev)
    bufs = [score.to(dev)]
    for i in range(1, N_ROTATE):  # same lengths, rolled rows: different bytes in every buffer
        bufs.append(torch.roll(bufs[0], shifts=i, dims=0).contiguous())
    lens_rot = [torch.roll(ld, shifts=i, dims=0).contiguous() for i in range(N_ROTATE)]
    outs = [torch.empty(B, K, dtype=torch.int32, device=dev) for _ in range(N_ROTATE)]
    nbytes_rank = workloads.algorithmic_bytes(lengths, L)
    nbytes_total = nbytes_rank
    if world > 1:  # every rank drew its own lengths: the job's bytes are the sum over the ranks
        t = torch.tensor([nbytes_rank], dtype=torch.int64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.SUM)
        nbytes_total = int(t.item())

    def step(i):
        fast_topk(bufs[i % N_ROTATE], outs[i % N_ROTATE], lens_rot[i % N_ROTATE])

    # ---- serialised launches first (the default mode of the library): latency of one call --------
    _native.set_overlap(False)
    plan_serial = _native.plan(B, L)
    with torch.cuda.stream(stream):
        for i in range(warmup):
            step(i)
    stream.synchronize()
    g_serial, calls_s, _, replays_s = timed_region(step, steps, stream, min_s=0.02)
    serial_sec = time_graph(g_serial, stream, replays_s) / (replays_s * calls_s)
    del g_serial

    # ---- throughput mode for the headline -------------------------------------------------------
    _native.set_overlap(True)
    plan = _native.plan(B, L)
    # warm-up (also the first call, which sets kernel attributes, outside any capture)
    with torch.cuda.stream(stream):
        for i in range(warmup):
            step(i)
    stream.synchronize()
    # the K steps alone, once: what a cold start of the launch pipeline costs
    g_cold = capture_steps(step, steps, stream)
    time_graph(g_cold, stream)
    cold_sec_per_step = min(time_graph(g_cold, stream) for _ in range(3)) / steps
    del g_cold
    graph, calls, reps_in_graph, replays = timed_region(step, steps, stream)

    # ---- timed region: barrier + synchronize on both sides, clocks sampled inside ---------------
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
        torch.cuda.synchronize()
    with ClockSampler(physical_gpu_index(local_rank)) as clk:
        sec = time_graph(graph, stream, replays)
        torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
        t = torch.tensor([sec], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        sec = float(t.item())
    launches = replays * calls
    sec_per_step = sec / launches
    value = B * world / sec_per_step
    del graph

    _native.set_overlap(False)
    # ---- end to end through the public op with host buffers ------------------------------------
    e2e_steps = max(3, min(steps, 20))
    # (fast_topk_v3_host = fftopk_select2048_host: H2D of every row's valid prefix from pinned
    # memory, the kernel, D2H of the indices, all on one stream)
    from jit_kernel.topk_indexer import fast_topk_v3_host
    h_score = score.pin_memory()
    h_len = lengths.pin_memory()
    h_out = torch.empty(B, K, dtype=torch.int32).pin_memory()
    h2d_bytes = int(4 * lengths.clamp(0, L).to(torch.int64).sum().item() + 4 * B)

    def e2e_step():
        fast_topk_v3_host(h_score, h_len, K, out=h_out)

    with torch.cuda.stream(stream):
        for _ in range(3):
            e2e_step()
        stream.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(e2e_steps):
            e2e_step()
        e1.record(stream)
    e1.synchronize()
    e2e_sec = e0.elapsed_time(e1) * 1e-3
    if world > 1:
        t = torch.tensor([e2e_sec], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_sec = float(t.item())
    e2e_value = B * world * e2e_steps / e2e_sec

    # ---- context-parallel decode (config 5) when there is more than one GPU -----------------------
    cp = None
    if world > 1 and not args.no_extras:
        try:
            cp = context_parallel_leg(dev, rank, world)
        except Exception as e:  # an extra: never lose the headline over it
            cp = {"error": repr(e)[:300]}

    status = kernel_status(dev)
    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    peak, peak_src = measured_peak_gbs()
    achieved = nbytes_total / world / sec_per_step / 1e9  # per GPU: the job's bytes / N / slowest rank's time
    line = {
        "metric": METRIC, "value": value, "unit": "rows/s", "n_gpus": world, "steps": steps, "warmup": warmup,
        "ms_per_step": sec_per_step * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic", "config": bench_config(),
        "replays": replays * reps_in_graph, "timed_region_ms": sec * 1e3,
        "cold_start_ms_per_step": cold_sec_per_step * 1e3,
        "run": {"l2": f"{N_ROTATE} input buffers of {4 * B * L >> 20} MiB rotated (> 126 MB L2)",
                "timing": f"CUDA graph of {calls} calls ({reps_in_graph} x the {steps}-step sequence) replayed "
                          f"{replays} times, CUDA events on its stream; cold_start_ms_per_step = the {steps} steps "
                          "alone, one replay",
                "mode": "throughput: fftopk_set_overlap(1), consecutive calls are programmatic dependent "
                        "launches and may overlap; one output buffer per rotated input",
                "plan": plan},
        "serial": {"us_per_call": serial_sec * 1e6, "rows_per_s": B * world / serial_sec,
                   "gbs": nbytes_rank / serial_sec / 1e9, "frac": nbytes_rank / serial_sec / 1e9 / peak, "plan": plan_serial,
                   "note": "same steps, default serialised launches (fftopk_set_overlap(0)), this rank"},
        "clocks": clk.summary("sampled during the timed region"),
        "e2e": {"value": e2e_value, "unit": "rows/s", "h2d_bytes_per_step": h2d_bytes,
                "d2h_bytes_per_step": 4 * B * K, "steps": e2e_steps, "ms_per_step": e2e_sec / e2e_steps * 1e3},
        "gpu_launches": launches,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     "traffic": NCU_TRAFFIC_BYTES_PER_LAUNCH, "peak_source": peak_src,
                     "algorithmic_bytes_per_launch": nbytes_total / world, "us_per_launch": sec_per_step * 1e6,
                     "cold_start_frac": nbytes_total / world / cold_sec_per_step / 1e9 / peak,
                     "frac_of_nominal_8TBs": achieved / 8000.0},
        "kernel_status": status,
    }
    if cp is not None:
        line["context_parallel"] = cp
    if not args.no_extras:
        probes = measure_l2_read_gbs(dev, stream)
        h2d_peak = measure_h2d_gbs(dev, stream)
        line["probes"] = {"read_gbs": probes, "pinned_h2d_gbs": h2d_peak,
                          "how": "fftopk_probe_read_bandwidth (128-bit ld.global.cg, all SMs) / one 64 MiB pinned copy"}
        e2e_gbs = (h2d_bytes + 4 * B * K) / (e2e_sec / e2e_steps) / 1e9
        line["e2e"]["roofline"] = {"bound": "pcie", "achieved": e2e_gbs, "peak": h2d_peak, "unit": "GB/s",
                                   "frac": e2e_gbs / h2d_peak if h2d_peak else None,
                                   "note": "bytes copied per step (valid prefixes in, indices out) / step time, per GPU, "
                                           "against this box's measured pinned host-to-device copy rate"}
        line["latency"] = latency_sweep(dev, stream, fast_topk, probes.get("l2_4MiB"))
        line["p50_us_B1_L1M"] = line["latency"]["1048576"]["warm"]["p50_us"]
        line["large_batch"] = large_batch_leg(dev, stream, fast_topk, peak)
        line["decode_loop"] = decode_loop_leg(dev, stream)
        line["fused_indexer"] = indexer_leg(dev, stream, peak)
        line["fused_indexer_drift"] = indexer_drift_leg(dev, stream)
        # CPU baseline on this box's host cores, bounded: the 64-row batch a few times (~20 ms each)
        cpu_reps = 10
        cpu_sec = time_cpu(score, lengths, cpu_reps, 2)
        line["cpu_baseline"] = {"value": B / cpu_sec, "unit": "rows/s", "cores": torch.get_num_threads(), "kind": "port",
                                "sample": f"the full 64-row batch, {cpu_reps} repetitions after 2 warm-ups",
                                "what": "torch.topk(score[b,:len], 2048, sorted=False) per row on the host"}
        s1, l1 = workloads.c2(L=1 << 20)
        line["cpu_baseline"]["B1_L1M_ms"] = time_cpu(s1, l1, 5, 1) * 1e3
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def profile_case(name: str) -> None:
    """Small fixed cases for profiler captures (`--case`): a few launches, one JSON line.
    b1: B=1, L=1M decode call, 40 rotated 4 MiB inputs. warm: the same row through the warm start
    (thresholds carried from call to call). merge: the 8-shard candidate merge of a B=4 batch (shards
    selected one after the other on this device). tp / serial: the bench's ragged B=64 batch in the
    throughput plan / the default plan, 12 launches over 8 rotated inputs. f16: the same batch as
    fp16 scores through the 16-bit instantiation. host: three calls of the host-buffer entry point
    (gather kernel reading pinned memory, selection). probe: the read-bandwidth probe on a 4 MiB and
    a 1 GiB buffer. indexer: eight calls of the fused indexer at B=1, L=1M over two rotated key
    caches (the last six with a threshold guess)."""
    from jit_kernel import _native
    from jit_kernel.distributed import _cuda_select, local_lengths, merge_candidates
    from jit_kernel.topk_indexer import fast_topk, fast_topk_general, fast_topk_v3_host, fast_topk_v3_warm

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    if name in ("b1", "warm"):
        score, lengths = workloads.c2(L=1 << 20)
        bufs = [torch.roll(score, i, 1).contiguous().to(dev) for i in range(40)]  # 160 MiB > L2
        ld = lengths.to(dev)
        out = torch.empty(1, K, dtype=torch.int32, device=dev)
        if name == "b1":
            for i in range(43):
                fast_topk(bufs[i % 40], out, ld)
        else:  # (rolled copies of one row have the same threshold: every call after the first is warm)
            thr = torch.zeros(1, dtype=torch.int32, device=dev)
            for i in range(43):
                fast_topk_v3_warm(bufs[i % 40], ld, K, thr, out=out)
        torch.cuda.synchronize()
        print(json.dumps({"case": name, "launches": 43, "plan": _native.plan(1, 1 << 20)}))
    elif name in ("tp", "serial", "f16"):
        _native.set_overlap(name == "tp")
        score, lengths = workloads.c3()
        dt = torch.float16 if name == "f16" else torch.float32
        bufs = [torch.roll(score, i, 0).to(dt).contiguous().to(dev) for i in range(8)]  # 256 MiB > L2 (fp16: 128 MiB)
        lens = [torch.roll(lengths, i, 0).contiguous().to(dev) for i in range(8)]
        out = torch.empty(score.size(0), K, dtype=torch.int32, device=dev)
        for i in range(12):
            if name == "f16":
                fast_topk_general(bufs[i % 8], lens[i % 8], K)
            else:
                fast_topk(bufs[i % 8], out, lens[i % 8])
        torch.cuda.synchronize()
        print(json.dumps({"case": name, "launches": 12, "plan": _native.plan(score.size(0), score.size(1))}))
        _native.set_overlap(False)
    elif name == "host":
        score, lengths = workloads.c3()
        hs, hl = score.pin_memory(), lengths.pin_memory()
        ho = torch.empty(score.size(0), K, dtype=torch.int32).pin_memory()
        for _ in range(3):
            fast_topk_v3_host(hs, hl, K, out=ho)
        torch.cuda.synchronize()
        print(json.dumps({"case": "host", "launches": 3}))
    elif name in ("indexer", "indexer_fp8"):
        from jit_kernel.indexer import FusedIndexerTopk
        L = 1 << 20
        fp8 = name == "indexer_fp8"
        dt = torch.float8_e4m3fn if fp8 else torch.bfloat16
        g = torch.Generator(device="cpu").manual_seed(L)
        q = (torch.randn(1, 64, 128, generator=g) * 0.5).to(dt).to(dev)
        ks = [(torch.randn(1, L, 128, generator=g) * 0.5).to(dt).to(dev) for _ in range(3 if fp8 else 2)]  # more than L2 together
        scale = (torch.rand(1, L, generator=g) + 0.5).to(dev) if fp8 else None
        w = torch.rand(1, 64, generator=g).to(dev)
        ln = torch.full((1,), L, dtype=torch.int32, device=dev)
        fs = [FusedIndexerTopk(1, L, dev) for _ in ks]
        for i in range(9):  # the first call on every cache seeds its threshold, the rest run with a guess
            fs[i % len(ks)](q, ks[i % len(ks)], w, ln, k_scale=scale)
        torch.cuda.synchronize()
        print(json.dumps({"case": name, "calls": 9, "L": L}))
    elif name == "probe":
        stream = torch.cuda.Stream(device=dev)
        print(json.dumps({"case": "probe", "read_gbs": measure_l2_read_gbs(dev, stream)}))
    else:
        score, lengths = workloads.c5()
        G, Ls = 8, score.size(1) // 8
        parts = [_cuda_select(score[:, g * Ls:(g + 1) * Ls].contiguous().to(dev), local_lengths(lengths, Ls, g).to(dev), g * Ls)
                 for g in range(G)]
        cand = torch.stack(parts).contiguous()
        for _ in range(6):
            merge_candidates(cand)
        torch.cuda.synchronize()
        print(json.dumps({"case": "merge", "launches": 6}))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2000)
    ap.add_argument("--warmup", type=int, default=50)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-extras", action="store_true", help="skip the latency sweep and the CPU baseline")
    ap.add_argument("--case", default=None, choices=["b1", "warm", "merge", "tp", "serial", "f16", "host", "probe", "indexer", "indexer_fp8"], help="run one small fixed case (for profilers)")
    args = ap.parse_args()
    if args.case:
        profile_case(args.case)
        return
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.impl == "reference":
        reference_arm(args, rank)
        return
    if world != args.gpus and world == 1 and args.gpus > 1:
        raise SystemExit("launch with torch.distributed.run --nproc-per-node N for --gpus N")
    ours_arm(args, rank, local_rank, world)


if __name__ == "__main__":
    main()
