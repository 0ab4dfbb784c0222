#!/usr/bin/env python
"""Benchmark of the top-2048 selector (drop-in for fast_topk_v3) on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port P bench.py --gpus N --steps K --warmup W

Prints ONE JSON line (rank 0). A step is one call of the op on one batch of the ragged batched
decode workload (B=64 rows, padded L=131072, valid lengths uniform in [1024, 131072], fp32
N(0,1) logits, -inf padding, k=2048). With N GPUs every rank processes its own 64-row batch
(rows are independent: no collective on the data path), so `value` = 64*N*K rows / time.

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
             the headline metric), L2-warm (the reference's own method) and with rotated buffers
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
# dram__bytes_read.sum + dram__bytes_write.sum of one select2048 launch on this workload, from the
# ncu capture of the throughput plan (None until a capture exists)
NCU_TRAFFIC_BYTES_PER_LAUNCH = 16774315  # throughput plan, mean of 3 captured launches


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
        "data": "synthetic", "config": {"workload": WORKLOAD, "where": "host cores, torch.topk"},
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


def latency_sweep(dev, stream, fast_topk):
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
        out[str(L)] = res
        del bufs
    return out


def context_parallel_leg(dev, rank: int, world: int):
    """Config 5: B=4, L=1M split evenly over the ranks; local select, exchange, merge. Two variants:
    NCCL all-gather + merge kernel, and the fused gather-and-merge over IPC-mapped peer buffers.
    Eager calls, CUDA events, max over ranks."""
    import torch.distributed as dist

    from jit_kernel.distributed import FusedContextParallelTopk, fast_topk_v3_context_parallel

    score, lengths = workloads.c5()
    Ls = score.size(1) // world
    shard = score[:, rank * Ls:(rank + 1) * Ls].contiguous().to(dev)
    fused = FusedContextParallelTopk(max_rows=score.size(0))
    out = {"workload": f"B=4, L=1048576 over {world} GPUs, k=2048"}
    reps = 50
    # the fused path again as a replayed CUDA graph (its epochs live on the device): no Python
    # between the kernels
    from jit_kernel.distributed import local_lengths
    lens_dev = local_lengths(lengths, Ls, rank).to(dev)
    res = torch.empty(score.size(0), K, dtype=torch.int32, device=dev)
    fused.run_into(shard, lens_dev, res)
    torch.cuda.synchronize()
    dist.barrier()
    side = torch.cuda.Stream(device=dev)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        with torch.cuda.graph(graph, stream=side):
            fused.run_into(shard, lens_dev, res)
    dist.barrier()
    for name, fn in (("nccl_allgather_merge", lambda: fast_topk_v3_context_parallel(shard, lengths, K)),
                     ("fused_peer_merge", lambda: fused(shard, lengths)),
                     ("fused_peer_merge_graph", graph.replay)):
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
        out[name + "_us_per_call"] = float(t.item())
    fused.close()
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
    steps, warmup = args.steps, max(args.warmup, 3)

    # ---- workload: every rank its own 64-row batch, N_ROTATE device copies with different data --
    score, lengths = workloads.c3(seed=workloads.SEED + rank)
    B, L = score.shape
    ld = lengths.to(dev)
    bufs = [score.to(dev)]
    for i in range(1, N_ROTATE):  # same lengths, rolled rows: different bytes in every buffer
        bufs.append(torch.roll(bufs[0], shifts=i, dims=0).contiguous())
    lens_rot = [torch.roll(ld, shifts=i, dims=0).contiguous() for i in range(N_ROTATE)]
    outs = [torch.empty(B, K, dtype=torch.int32, device=dev) for _ in range(N_ROTATE)]
    nbytes = workloads.algorithmic_bytes(lengths, L)

    def step(i):
        fast_topk(bufs[i % N_ROTATE], outs[i % N_ROTATE], lens_rot[i % N_ROTATE])

    # ---- serialised launches first (the default mode of the library): latency of one call --------
    _native.set_overlap(False)
    plan_serial = _native.plan(B, L)
    with torch.cuda.stream(stream):
        for i in range(warmup):
            step(i)
    stream.synchronize()
    n_serial = min(steps, 200)
    g_serial = capture_steps(step, n_serial, stream)
    time_graph(g_serial, stream)
    serial_sec = min(time_graph(g_serial, stream) for _ in range(3)) / n_serial
    del g_serial

    # ---- throughput mode for the headline -------------------------------------------------------
    _native.set_overlap(True)
    plan = _native.plan(B, L)

    # ---- warm-up (also the first call, which sets kernel attributes, outside any capture) -------
    with torch.cuda.stream(stream):
        for i in range(warmup):
            step(i)
    stream.synchronize()
    chunk = min(steps, 500)
    n_chunks, rest = divmod(steps, chunk)
    g_chunk = capture_steps(step, chunk, stream)
    g_rest = capture_steps(step, rest, stream) if rest else None
    time_graph(g_chunk, stream)  # graph warm-up (upload)
    if g_rest is not None:
        time_graph(g_rest, stream)

    # ---- timed region: exactly `steps` calls, barrier + synchronize on both sides ---------------
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
        torch.cuda.synchronize()
    with ClockSampler(physical_gpu_index(local_rank)) as clk:
        sec = time_graph(g_chunk, stream, n_chunks)
        if g_rest is not None:
            sec += time_graph(g_rest, stream)
        torch.cuda.synchronize()
        note = "sampled during the timed region"
        if len(clk.samples) < 5:
            # the timed region was shorter than a few NVML polls: keep the same load running
            t_end = time.perf_counter() + 0.06
            while time.perf_counter() < t_end:
                time_graph(g_chunk, stream)
            note = "timed region too short for NVML polling; sampled under the same load right after it"
    if world > 1:
        dist.barrier()
        t = torch.tensor([sec], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        sec = float(t.item())
    sec_per_step = sec / steps
    value = B * world * steps / sec

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
            cp = {"error": repr(e)[:200]}

    status = kernel_status(dev)
    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    peak, peak_src = measured_peak_gbs()
    achieved = nbytes / sec_per_step / 1e9
    line = {
        "metric": METRIC, "value": value, "unit": "rows/s", "n_gpus": world, "steps": steps, "warmup": warmup,
        "ms_per_step": sec_per_step * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD, "rows_per_gpu": B, "l2": f"{N_ROTATE} input buffers of {4 * B * L >> 20} MiB "
                   "rotated (> 126 MB L2)", "timing": "CUDA graph of the steps, CUDA events on its stream",
                   "mode": "throughput: fftopk_set_overlap(1), consecutive calls are programmatic dependent "
                           "launches and may overlap; one output buffer per rotated input",
                   "plan": plan},
        "serial": {"us_per_call": serial_sec * 1e6, "rows_per_s": B * world / serial_sec,
                   "gbs": nbytes / serial_sec / 1e9, "plan": plan_serial,
                   "note": "same steps, default serialised launches (fftopk_set_overlap(0)), this rank"},
        "clocks": clk.summary(note),
        "e2e": {"value": e2e_value, "unit": "rows/s", "h2d_bytes_per_step": h2d_bytes,
                "d2h_bytes_per_step": 4 * B * K, "steps": e2e_steps},
        "gpu_launches": steps,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     "traffic": NCU_TRAFFIC_BYTES_PER_LAUNCH, "peak_source": peak_src,
                     "algorithmic_bytes_per_launch": nbytes, "us_per_launch": sec_per_step * 1e6,
                     "frac_of_nominal_8TBs": achieved / 8000.0},
        "kernel_status": status,
    }
    if cp is not None:
        line["context_parallel"] = cp
    if not args.no_extras:
        line["latency"] = latency_sweep(dev, stream, fast_topk)
        line["p50_us_B1_L1M"] = line["latency"]["1048576"]["warm"]["p50_us"]
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
    b1: B=1, L=1M decode call, eight rotated 4 MiB inputs. merge: the 8-shard candidate merge of a
    B=4 batch (shards selected one after the other on this device). tp / serial: the bench's ragged
    B=64 batch in the throughput plan / the default plan, 12 launches over 8 rotated inputs."""
    from jit_kernel.distributed import _cuda_select, local_lengths, merge_candidates
    from jit_kernel.topk_indexer import fast_topk

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    if name == "b1":
        score, lengths = workloads.c2(L=1 << 20)
        bufs = [torch.roll(score, i, 1).contiguous().to(dev) for i in range(40)]  # 160 MiB > L2
        ld = lengths.to(dev)
        out = torch.empty(1, K, dtype=torch.int32, device=dev)
        for i in range(43):
            fast_topk(bufs[i % 40], out, ld)
        torch.cuda.synchronize()
        print(json.dumps({"case": "b1", "launches": 43, "plan": __import__("jit_kernel._native", fromlist=["x"]).plan(1, 1 << 20)}))
    elif name in ("tp", "serial"):
        from jit_kernel import _native
        _native.set_overlap(name == "tp")
        score, lengths = workloads.c3()
        bufs = [torch.roll(score, i, 0).contiguous().to(dev) for i in range(8)]  # 256 MiB > L2
        lens = [torch.roll(lengths, i, 0).contiguous().to(dev) for i in range(8)]
        out = torch.empty(score.size(0), K, dtype=torch.int32, device=dev)
        for i in range(12):
            fast_topk(bufs[i % 8], out, lens[i % 8])
        torch.cuda.synchronize()
        print(json.dumps({"case": name, "launches": 12, "plan": _native.plan(score.size(0), score.size(1))}))
        _native.set_overlap(False)
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
    ap.add_argument("--case", default=None, choices=["b1", "merge", "tp", "serial"], help="run one small fixed case (for profilers)")
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
