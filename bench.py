#!/usr/bin/env python
"""Benchmark of the hot path: radix sort of uint32 keys (and scan / reduce / histogram
beside it) on 1..8 B200s.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference]

N = 1: one step = one ascending RadixSort of 2^26 uint32 keys (i.i.d. uniform, seeded).
N > 1 (under torchrun, one rank per GPU): one step = one sample sort of N * 2^26 keys,
2^26 per GPU (weak scaling): sampled splitters, a stable partition whose kernel stores every
bucket straight into its owner's receive buffer (peer memory over NVLink), local radix sort.
`--impl reference` times the CPU restatement of the reference's CPUAccelerator sort on the
host cores (the reference is C#; no .NET toolchain exists on these machines).

Prints ONE JSON line (rank 0).
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

KEYS_PER_GPU = 1 << 26
SORT_BYTES_PER_KEY = 36          # 4-byte keys: one histogram read + 4 x (read + write)
SEED = 2
# DRAM traffic of the sort's kernels comes from the ncu summary under profiles/ (written when a
# capture is taken); it is only quoted while the kernel source is the one that was profiled.
TRAFFIC_FILE = os.path.join(ROOT, "profiles", "sort_kernel.md")
KERNEL_SOURCES = [os.path.join(ROOT, "ilgpu_b200", "csrc", f) for f in ("radix_sort.cu", "common.cuh")]


def kernel_source_digest() -> str:
    import hashlib
    h = hashlib.sha256()
    for path in KERNEL_SOURCES:
        with open(path, "rb") as f:
            h.update(f.read())
    return h.hexdigest()[:16]


def profiled_traffic():
    """(bytes per sort call, bytes per digit pass) from the ncu summary, or (None, None) when
    the summary is missing or was taken from other kernel source."""
    import re
    try:
        text = open(TRAFFIC_FILE).read()
    except OSError:
        return None, None
    m = re.search(r"kernel source digest:\s*`?([0-9a-f]{16})", text)
    call = re.search(r"sort call DRAM bytes:\s*`?([0-9.eE+]+)", text)
    one = re.search(r"digit pass DRAM bytes:\s*`?([0-9.eE+]+)", text)
    if not (m and call and one) or m.group(1) != kernel_source_digest():
        return None, None
    return float(call.group(1)), float(one.group(1))


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region is timed."""
    QUERY = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.lines: list[str] = []
        self.first = 0
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "20"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._pump, daemon=True).start()
        except OSError:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def mark(self):
        """Forget the samples taken so far (warm-up)."""
        self.first = len(self.lines)

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines[max(0, self.first - 1):]:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0])); mx.append(float(parts[1]))
            except ValueError:
                continue
            for name, val in zip(names, parts[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def host_cores() -> int:
    try:
        return len(os.sched_getaffinity(0))
    except AttributeError:
        return os.cpu_count() or 1


# ------------------------------------------------------------------------------------------
def cpu_reference_sort(sample_keys, cores: int, repeats: int = 1):
    """Times the literal two-kernel 2-bit CPU sort spread over `cores` threads; returns
    (Gkeys/s, seconds per run)."""
    import numpy as np
    from oracle import cpu_oracle as oracle
    best = None
    for _ in range(repeats):
        t0 = time.perf_counter()
        out = oracle.radix_sort_literal_mt(sample_keys, False, 16 * cores, cores)
        dt = time.perf_counter() - t0
        best = dt if best is None or dt < best else best
    assert np.all(out[1:] >= out[:-1])
    return sample_keys.size / best / 1e9, best


def cpu_default_device_sort(sample_keys):
    """The same sort the way the reference's default CPUDevice runs it: 16 groups of one
    thread on one multiprocessor (Src/ILGPU/Runtime/CPU/CPUDevice.cs:67-77), i.e. one host
    thread.  Returns Gkeys/s."""
    from oracle import cpu_oracle as oracle
    t0 = time.perf_counter()
    oracle.radix_sort_literal_mt(sample_keys, False, 16, 1)
    return sample_keys.size / (time.perf_counter() - t0) / 1e9


def run_reference(args) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from ilgpu_b200 import synthetic
    cores = host_cores()
    n = KEYS_PER_GPU
    keys = synthetic.uniform_uint32(n, SEED)     # the same 2^26 keys the GPU arm sorts at N = 1
    times = []
    for step in range(args.warmup + args.steps):
        _, dt = cpu_reference_sort(keys, cores)
        if step >= args.warmup:
            times.append(dt)
    sec = sum(times) / len(times)
    value = n / sec / 1e9
    single = cpu_default_device_sort(keys[: 1 << 22])
    line = {
        "impl": "reference", "metric": "radix_sort_gkeys_per_s", "value": value, "unit": "Gkeys/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": sec * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "u32", "data": "synthetic",
        "config": {"workload": "RadixSort ascending, 2^26 uint32 keys i.i.d. uniform (seeded)",
                   "keys_per_gpu": KEYS_PER_GPU, "keys_per_step": n},
        "cpu_baseline": {"value": value, "unit": "Gkeys/s", "cores": cores, "kind": "port",
                         "sample": "the full 2^26-key workload per step; C restatement of CPURadixSortKernel1/2 "
                                   "(2 bits per pass), 16 x cores groups spread over all host threads",
                         "default_cpu_device_one_thread": {"value": single, "unit": "Gkeys/s", "cores": 1,
                                                           "sample": "first 2^22 keys, 16 groups run by one thread"}},
        "e2e": {"value": value, "unit": "Gkeys/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------
def time_region(fn, steps: int, stream) -> float:
    """Milliseconds per step of `fn(i)` over `steps` calls, by CUDA events on `stream`."""
    import torch
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    start.record(stream)
    for i in range(steps):
        fn(i)
    end.record(stream)
    torch.cuda.synchronize()
    return start.elapsed_time(end) / steps


def secondary_metrics(acc, peak_gbs: float) -> dict:
    """Scan / reduce / histogram throughput on their own configurations (1 GPU, resident
    inputs larger than L2, CUDA events)."""
    import torch
    import ilgpu_b200 as ib
    from ilgpu_b200 import synthetic
    stream = torch.cuda.current_stream()
    out = {}
    Ops = ib.ScanReduceOperations

    def gbs(nbytes, ms):
        v = nbytes / (ms * 1e-3) / 1e9
        return {"GB/s": round(v, 1), "frac_of_measured_hbm": round(v / peak_gbs, 4), "ms": round(ms, 4)}

    # float32 inclusive scan + sum reduce over 2^30 values (8 B and 4 B per element)
    n = 1 << 30
    x = synthetic.uniform_float32_device(n, 5, "cuda")
    y = torch.empty_like(x)
    temp = acc.Allocate1D(acc.ComputeScanTempStorageSize(torch.float32, n), torch.int32)
    scan = acc.CreateScan(Ops.AddFloat, ib.ScanKind.Inclusive)
    for _ in range(3):
        scan(None, x, y, temp)
    out["scan_f32_inclusive_2^30"] = gbs(8 * n, time_region(lambda i: scan(None, x, y, temp), 5, stream))
    red = acc.CreateReduction(Ops.AddFloat)
    cell = acc.Allocate1D(1, torch.float32)
    for _ in range(3):
        red(None, x, cell)
    out["reduce_f32_sum_2^30"] = gbs(4 * n, time_region(lambda i: red(None, x, cell), 5, stream))
    del x, y, temp
    # int32 reduce + exclusive scan over 2^24 values, rotating over 8 buffers (64 MiB each).  A call
    # is 20 to 40 us of device work, less than what the Python layer needs to enqueue it, so the
    # 16 calls are also captured into a CUDA graph and replayed: that figure is the device's.
    n = 1 << 24
    bufs = [synthetic.uniform_int32_device(n, 1, "cuda", start=i * n) for i in range(8)]
    outs = [torch.empty_like(b) for b in bufs]
    temp = acc.Allocate1D(acc.ComputeScanTempStorageSize(torch.int32, n), torch.int32)
    scan = acc.CreateScan(Ops.AddInt32, ib.ScanKind.Exclusive)
    red = acc.CreateReduction(Ops.AddInt32)
    cell = acc.Allocate1D(1, torch.int32)
    for i in range(8):
        scan(None, bufs[i], outs[i], temp); red(None, bufs[i], cell)

    def replayed(call, reps=5):
        """ms per call of 16 calls captured once and replayed `reps` times; None if capture is refused."""
        try:
            side = torch.cuda.Stream()
            graph = torch.cuda.CUDAGraph()
            torch.cuda.synchronize()
            with torch.cuda.graph(graph, stream=side):
                for i in range(16):
                    call(i)
            graph.replay()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(reps):
                graph.replay()
            e1.record()
            torch.cuda.synchronize()
            return e0.elapsed_time(e1) / (16 * reps)
        except Exception as exc:   # capture of a launch kind the driver refuses: keep the eager figure
            torch.cuda.synchronize()
            return None

    for name, call, nbytes in (("scan_i32_exclusive_2^24", lambda i: scan(None, bufs[i % 8], outs[i % 8], temp), 8 * n),
                               ("reduce_i32_sum_2^24", lambda i: red(None, bufs[i % 8], cell), 4 * n)):
        eager_ms = time_region(call, 16, stream)
        graph_ms = replayed(call)
        entry = gbs(nbytes, graph_ms if graph_ms is not None else eager_ms)
        entry["how"] = "16 calls captured in a CUDA graph and replayed" if graph_ms is not None else "eager calls"
        entry["eager_ms"] = round(eager_ms, 4)
        out[name] = entry
    expect = torch.cumsum(bufs[3].to(torch.int64), 0)
    assert int(outs[3][-1]) == int(((expect[-2] + 2 ** 31) % 2 ** 32) - 2 ** 31) and int(outs[3][0]) == 0, "scan result after replay"
    del bufs, outs
    # histogram of 2^28 float32 N(0,1) into 256 int32 bins
    n = 1 << 28
    f = synthetic.normal_float32_device(n, 3, "cuda")
    bins = torch.zeros(256, dtype=torch.int32, device="cuda")
    ovf = torch.zeros(1, dtype=torch.int32, device="cuda")
    hist = acc.CreateHistogram(ib.EqualWidthClampLocator(-4.0, 4.0))
    for _ in range(3):
        hist(None, f, bins, ovf)
    out["histogram_f32_256bins_2^28"] = gbs(4 * n, time_region(lambda i: hist(None, f, bins, ovf), 5, stream))
    del f
    # stable RadixSortPairs of 2^28 uint64 Zipf(1.1) keys with uint32 payload = index; 104 B/pair
    # (8 + 4 x (16 + 8): the upper four key bytes are constant, so four of eight digit passes run)
    n = 1 << 28
    keys0 = synthetic.zipf_uint64_device(n, 4, "cuda")
    vals0 = torch.arange(n, dtype=torch.int32, device="cuda").view(torch.uint32)
    op = ib.RadixSortOperations.AscendingUInt64
    temp = acc.Allocate1D(acc.ComputeRadixSortPairsTempStorageSize(op, torch.uint32, n), torch.int32)
    sort = acc.CreateRadixSortPairs(op)
    times = []
    for r in range(4):
        k, v = keys0.clone(), vals0.clone()
        ms = time_region(lambda i: sort(None, k, v, temp), 1, stream)
        if r:
            times.append(ms)
    ms = sum(times) / len(times)
    out["sort_pairs_u64_u32_zipf_2^28"] = dict(gbs(104 * n, ms), **{"Gpairs/s": round(n / ms / 1e6, 2)})
    return out


def secondary_metrics_sharded(acc, sharded, world: int, rank: int, peak_gbs: float) -> dict:
    """Scan / reduce / histogram over all GPUs (configs 3 and 5: the totals stay 2^28 and 2^30
    elements, sharded contiguously), timed on the device, max over ranks."""
    import torch
    import torch.distributed as dist
    import ilgpu_b200 as ib
    from ilgpu_b200 import synthetic
    stream = torch.cuda.current_stream()
    Ops = ib.ScanReduceOperations
    out = {}

    def agg(nbytes_total, ms):
        t = torch.tensor([ms], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
        v = nbytes_total / (ms * 1e-3) / 1e9
        return {"GB/s": round(v, 1), "frac_of_measured_hbm_x_gpus": round(v / (peak_gbs * world), 4), "ms": round(ms, 4)}

    import math

    def gathered(value: float):
        t = torch.tensor([value], device="cuda", dtype=torch.float64)
        parts = [torch.zeros_like(t) for _ in range(world)]
        dist.all_gather(parts, t)
        return [float(p.item()) for p in parts]

    n_total = 1 << 30
    n = n_total // world
    x = synthetic.uniform_float32_device(n, 5, "cuda", start=rank * n)
    y = torch.empty_like(x)
    for _ in range(3):
        sharded.Scan(x, y, Ops.AddFloat, ib.ScanKind.Inclusive)
    dist.barrier()
    out["scan_f32_inclusive_2^30_total"] = agg(8 * n_total, time_region(lambda i: sharded.Scan(x, y, Ops.AddFloat, ib.ScanKind.Inclusive), 5, stream))
    # float64 sums of the shards: rank r's last scan element is the total of ranks 0..r; the
    # tolerance is the stated 1e-5 * log2(n) * sum|x| (x >= 0 here)
    shard_sums = gathered(float(x.to(torch.float64).sum().item()))
    total = sum(shard_sums)
    tol = 1e-5 * math.log2(n_total) * total
    assert abs(float(y[-1].item()) - sum(shard_sums[: rank + 1])) <= tol, "sharded scan: last element of the slice is off"
    assert abs(float(y[0].item()) - (sum(shard_sums[:rank]) + float(x[0].item()))) <= tol, "sharded scan: first element of the slice is off"
    for _ in range(3):
        sharded.Reduce(x, Ops.AddFloat)
    dist.barrier()
    out["reduce_f32_sum_2^30_total"] = agg(4 * n_total, time_region(lambda i: sharded.Reduce(x, Ops.AddFloat), 5, stream))
    assert abs(float(sharded.Reduce(x, Ops.AddFloat).item()) - total) <= tol, "sharded reduce is off"
    del x, y
    n_total = 1 << 28
    n = n_total // world
    f = synthetic.normal_float32_device(n, 3, "cuda", start=rank * n)
    bins = torch.zeros(256, dtype=torch.int32, device="cuda")
    ovf = torch.zeros(1, dtype=torch.int32, device="cuda")
    loc = ib.EqualWidthClampLocator(-4.0, 4.0)
    for _ in range(3):
        sharded.Histogram(f, bins, ovf, loc)
    dist.barrier()
    out["histogram_f32_256bins_2^28_total"] = agg(4 * n_total, time_region(lambda i: sharded.Histogram(f, bins, ovf, loc), 5, stream))
    # one more call into fresh bins: they sum to n and equal the bins one GPU computes for the
    # same 2^28 values (rank 0 generates them all)
    del f
    f = synthetic.normal_float32_device(n, 3, "cuda", start=rank * n)
    bins.zero_()
    sharded.Histogram(f, bins, ovf, loc)
    assert int(bins.to(torch.int64).sum().item()) == n_total, "sharded histogram: the bins do not sum to n"
    if rank == 0:
        del f
        whole = synthetic.normal_float32_device(n_total, 3, "cuda")
        single = torch.zeros(256, dtype=torch.int32, device="cuda")
        acc.Histogram(None, whole, single, ovf, loc)
        assert torch.equal(single, bins), "sharded histogram differs from the single-GPU bins"
    out["checked"] = ("scan and reduce against float64 shard sums within 1e-5*log2(n)*sum|x|; histogram bins sum to n "
                      "and equal the single-GPU bins")
    return out


def _gather_variable(t, dist):
    """All ranks' 1-D tensors of different lengths, concatenated in rank order (on every rank)."""
    import torch
    world = dist.get_world_size()
    size = torch.tensor([t.numel()], device=t.device, dtype=torch.int64)
    sizes = [torch.zeros_like(size) for _ in range(world)]
    dist.all_gather(sizes, size)
    sizes = [int(x.item()) for x in sizes]
    cap = max(max(sizes), 1)
    padded = torch.zeros(cap, dtype=t.dtype, device=t.device)
    padded[: t.numel()] = t
    parts = [torch.empty_like(padded) for _ in range(world)]
    dist.all_gather(parts, padded)
    return torch.cat([p[:k] for p, k in zip(parts, sizes)])


def check_sharded_sort(result, checksum_in: int, n_in: int, dist) -> None:
    """Global properties of a sharded sort result (uint32 keys): every rank's slice ascends,
    rank r's last key does not exceed rank r+1's first, and count and key sum of the whole
    equal the input's."""
    import torch
    li = result.view(torch.int32).to(torch.int64) & 0xFFFFFFFF
    assert bool((li[1:] >= li[:-1]).all()), "a rank's slice is not sorted"
    edge = torch.tensor([int(li[0]) if li.numel() else -1, int(li[-1]) if li.numel() else -1, li.numel(), int(li.sum())],
                        device=result.device, dtype=torch.int64)
    edges = [torch.zeros_like(edge) for _ in range(dist.get_world_size())]
    dist.all_gather(edges, edge)
    last = -1
    for e in edges:
        first_key, last_key, count, _ = (int(x) for x in e.tolist())
        if count:
            assert first_key >= last, "rank order broken: a slice starts below the previous slice's last key"
            last = last_key
    assert sum(int(e[2]) for e in edges) == n_in, "keys were lost or duplicated"
    assert sum(int(e[3]) for e in edges) == checksum_in, "key checksum differs from the input's"


def check_small_sorts_against_oracle(sharded, rank: int, world: int, dist) -> None:
    """One untimed SortKeys (uniform uint32) and one SortPairs (Zipf uint64 keys, payload =
    global index) of 2^20 elements in total, gathered and compared bit for bit, payload
    included, with the CPU oracle (rank 0 compares; the oracle is the checker only)."""
    import numpy as np
    import torch
    import ilgpu_b200 as ib
    from ilgpu_b200 import synthetic
    total = 1 << 20
    n = total // world
    keys = synthetic.uniform_uint32_device(n, 11, "cuda", start=rank * n)
    out, _ = sharded.SortKeys(keys, ib.RadixSortOperations.AscendingUInt32)
    got = _gather_variable(out.view(torch.int32), dist)
    pk = synthetic.zipf_uint64_device(n, 12, "cuda", start=rank * n)
    pv = (torch.arange(n, dtype=torch.int32, device="cuda") + rank * n).view(torch.uint32)
    ok, ov = sharded.SortPairs(pk, pv, ib.RadixSortOperations.AscendingUInt64)
    gk = _gather_variable(ok.view(torch.int64), dist)
    gv = _gather_variable(ov.view(torch.int32), dist)
    if rank == 0:
        from oracle import cpu_oracle as oracle
        expect, _ = oracle.radix_sort(synthetic.uniform_uint32(world * n, 11))
        assert np.array_equal(got.cpu().numpy().view(np.uint32), expect), "sharded SortKeys differs from the oracle"
        ek, ev = oracle.radix_sort(synthetic.zipf_uint64(world * n, 12), np.arange(world * n, dtype=np.uint32))
        assert np.array_equal(gk.cpu().numpy().view(np.uint64), ek), "sharded SortPairs keys differ from the oracle"
        assert np.array_equal(gv.cpu().numpy().view(np.uint32), ev), "sharded SortPairs payload differs from the oracle"


def run_profile_case(case: str) -> None:
    """Three launches of one primitive on a case that is larger than L2 but holds at most a
    few GB on the device: what an `ncu` capture is pointed at."""
    import torch
    import ilgpu_b200 as ib
    from ilgpu_b200 import synthetic
    acc = ib.Accelerator(0)
    Ops, Sorts = ib.ScanReduceOperations, ib.RadixSortOperations
    if case == "sort":
        n = 1 << 26
        temp = acc.Allocate1D(acc.ComputeRadixSortTempStorageSize(Sorts.AscendingUInt32, n), torch.int32)
        sort = acc.CreateRadixSort(Sorts.AscendingUInt32)
        for r in range(3):
            keys = synthetic.uniform_uint32_device(n, SEED + r, "cuda")
            sort(None, keys, temp)
    elif case == "sort_pairs":
        n = 1 << 25
        vals = torch.arange(n, dtype=torch.int32, device="cuda").view(torch.uint32)
        temp = acc.Allocate1D(acc.ComputeRadixSortPairsTempStorageSize(Sorts.AscendingUInt64, vals.dtype, n), torch.int32)
        sort = acc.CreateRadixSortPairs(Sorts.AscendingUInt64)
        for r in range(3):
            keys = synthetic.zipf_uint64_device(n, 4 + r, "cuda")
            sort(None, keys, vals.clone(), temp)
    elif case == "partition":
        # the partition + exchange step of the multi-GPU sort on one GPU: eight buckets (equal
        # slices of the key range, as on an 8-GPU box), each stored into a buffer of its own
        from ilgpu_b200.multi_gpu import NativeEngine
        n = 1 << 26
        eng = NativeEngine(acc)
        op = Sorts.AscendingUInt32
        cuts = [(j << 32) // 8 for j in range(1, 8)]
        splitter_keys = torch.tensor([c - (1 << 32) if c >= (1 << 31) else c for c in cuts], dtype=torch.int32,
                                     device="cuda").view(torch.uint32)
        splitter_index = torch.zeros(7, dtype=torch.int64, device="cuda")
        parts = [torch.empty(n // 8 + (1 << 20), dtype=torch.uint32, device="cuda") for _ in range(8)]
        for r in range(3):
            keys = synthetic.uniform_uint32_device(n, SEED + r, "cuda")
            eng.bucket_count(keys, op, splitter_keys, splitter_index, 0)
            eng.bucket_scatter(keys, None, op, splitter_keys, splitter_index, 0, [p.data_ptr() for p in parts], None)
    elif case == "scan":
        n = 1 << 28
        x = synthetic.uniform_float32_device(n, 5, "cuda")
        y = torch.empty_like(x)
        temp = acc.Allocate1D(acc.ComputeScanTempStorageSize(torch.float32, n), torch.int32)
        scan = acc.CreateScan(Ops.AddFloat, ib.ScanKind.Inclusive)
        for _ in range(3):
            scan(None, x, y, temp)
    elif case == "reduce":
        n = 1 << 28
        x = synthetic.uniform_float32_device(n, 5, "cuda")
        cell = acc.Allocate1D(1, torch.float32)
        for _ in range(3):
            acc.CreateReduction(Ops.AddFloat)(None, x, cell)
    else:
        n = 1 << 28
        f = synthetic.normal_float32_device(n, 3, "cuda")
        bins = torch.zeros(256, dtype=torch.int32, device="cuda")
        ovf = torch.zeros(1, dtype=torch.int32, device="cuda")
        for _ in range(3):
            acc.Histogram(None, f, bins, ovf, ib.EqualWidthClampLocator(-4.0, 4.0))
    torch.cuda.synchronize()
    print(json.dumps({"profile_case": case, "ok": True}))


def run_native(args) -> None:
    import numpy as np
    import torch
    import ilgpu_b200 as ib
    from ilgpu_b200 import synthetic

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    acc = ib.Accelerator(local_rank)
    stream = torch.cuda.current_stream()
    peak_gbs, peak_kind = measured_peaks()
    n = KEYS_PER_GPU
    steps, warmup = args.steps, args.warmup
    op = ib.RadixSortOperations.AscendingUInt32

    # One fresh unsorted buffer per step (the sort is in place); 256 MiB each, larger than L2.
    nbuf = steps + warmup
    pristine = synthetic.uniform_uint32_device(n, SEED, "cuda", start=rank * n)
    checksum_in = int((pristine.view(torch.int32).to(torch.int64) & 0xFFFFFFFF).sum().item())

    if world == 1:
        bufs = [pristine.clone() for _ in range(nbuf)]
        temp = acc.Allocate1D(acc.ComputeRadixSortTempStorageSize(op, n), torch.int32)
        sort = acc.CreateRadixSort(op)

        def step_fn(i):
            sort(None, bufs[i], temp)
        launches_per_step = 7   # digit histograms, offsets, 4 digit passes, copy-back (exits at once)
        result_of = lambda i: bufs[i]
    else:
        from ilgpu_b200.multi_gpu import ShardedAlgorithms
        sharded = ShardedAlgorithms(acc, dist.group.WORLD)
        bufs = [pristine.clone() for _ in range(nbuf)]
        last = [None]

        def step_fn(i):
            # enqueued without a host synchronisation; the previous step's output goes back to the allocator
            last[0] = sharded.SortAsync(bufs[i], None, op)
        launches_per_step = sharded.sort_launches_per_step(op)

        def result_of(i):
            out, _, count = last[0]
            sharded.CheckStatus()
            return out[: int(count.item())]

    sampler = ClockSampler(local_rank)
    sampler.start()          # nvidia-smi takes a moment to start: launch it before the warm-up
    for i in range(warmup):
        step_fn(i)
    torch.cuda.synchronize()
    if dist is not None:
        dist.barrier()
    sampler.mark()           # samples from here on belong to the timed region
    torch.cuda.synchronize()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record(stream)
    for i in range(warmup, warmup + steps):
        step_fn(i)
    ev1.record(stream)
    torch.cuda.synchronize()
    ms_total = ev0.elapsed_time(ev1)
    if dist is not None:
        t = torch.tensor([ms_total], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dist.barrier()
        ms_total = float(t.item())
    clocks = sampler.stop()
    ms_per_step = ms_total / steps
    value = world * n / (ms_per_step * 1e-3) / 1e9

    # checks of the timed work, outside the timed region (the parity tests proper live in tests/)
    final = result_of(warmup + steps - 1)
    if world == 1:
        li = final.view(torch.int32).to(torch.int64) & 0xFFFFFFFF
        assert bool((li[1:] >= li[:-1]).all()), "result is not sorted"
        assert int(li.sum().item()) == checksum_in, "keys were lost"
        del li
    else:
        t = torch.tensor([checksum_in], device="cuda", dtype=torch.int64)
        dist.all_reduce(t)
        check_sharded_sort(final, int(t.item()), world * n, dist)
        check_small_sorts_against_oracle(sharded, rank, world, dist)
    parity_checked = True
    del final

    # end to end through the public API with host buffers: H2D of the keys, sort, D2H of the result
    e2e_steps = max(1, min(steps, 8))
    host_in = torch.empty(n, dtype=torch.uint32).pin_memory()
    host_in.copy_(pristine.cpu())
    host_out = torch.empty(n if world == 1 else 2 * n, dtype=torch.uint32).pin_memory()
    dev = bufs[0]
    d2h_bytes = [4 * n]

    def e2e_fn(i):
        dev.copy_(host_in, non_blocking=True)
        if world == 1:
            sort(None, dev, temp)
            host_out.copy_(dev, non_blocking=True)
        else:
            out, count = sharded.SortKeys(dev, op)
            count = min(count, host_out.numel())
            host_out[:count].copy_(out[:count], non_blocking=True)     # this rank's slice of the result
            d2h_bytes[0] = 4 * count
    for i in range(2):
        e2e_fn(i)
    torch.cuda.synchronize()
    if dist is not None:
        dist.barrier()
    e2e_ms = time_region(e2e_fn, e2e_steps, stream)
    e2e_note = "each step: copy-in, sort, copy-out, one after the other on one stream"
    e2e_serial_ms = e2e_ms
    if world == 1:
        # The same calls as a user with a queue of batches would issue them: two device buffers,
        # and the copy-in, the sort and the copy-out of neighbouring steps on three streams, so
        # that both directions of the host link work at once.  Every step still copies its own
        # input in and its own result out inside the timed region.
        s_in, s_sort, s_out = torch.cuda.Stream(), torch.cuda.Stream(), torch.cuda.Stream()
        dev2 = [bufs[0], bufs[1 % len(bufs)]] if len(bufs) > 1 else [bufs[0], torch.empty_like(bufs[0])]
        host_out2 = [host_out, torch.empty(n, dtype=torch.uint32).pin_memory()]
        ev_in = [torch.cuda.Event() for _ in range(2)]
        ev_sorted = [torch.cuda.Event() for _ in range(2)]
        ev_out = [torch.cuda.Event() for _ in range(2)]

        def piped_fn(i):
            b = i & 1
            with torch.cuda.stream(s_in):
                s_in.wait_event(ev_out[b])       # the buffer's previous result has left
                dev2[b].copy_(host_in, non_blocking=True)
                ev_in[b].record(s_in)
            s_sort.wait_event(ev_in[b])
            sort(s_sort, dev2[b], temp)
            ev_sorted[b].record(s_sort)
            with torch.cuda.stream(s_out):
                s_out.wait_event(ev_sorted[b])
                host_out2[b].copy_(dev2[b], non_blocking=True)
                ev_out[b].record(s_out)

        def piped_region(k):
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            start.record(stream)
            for st in (s_in, s_sort, s_out):
                st.wait_stream(stream)
            for i in range(k):
                piped_fn(i)
            for st in (s_in, s_sort, s_out):
                stream.wait_stream(st)
            end.record(stream)
            torch.cuda.synchronize()
            return start.elapsed_time(end) / k
        piped_region(2)
        piped_steps = max(16, 2 * e2e_steps)
        e2e_ms = piped_region(piped_steps)
        for b in range(2):   # both results are complete and sorted
            ho = host_out2[b].view(torch.int32)
            assert int(ho[0]) & 0xFFFFFFFF <= int(ho[n // 2]) & 0xFFFFFFFF <= int(ho[-1]) & 0xFFFFFFFF
        e2e_note = ("double-buffered: copy-in, sort and copy-out of neighbouring steps overlap on three streams; "
                    "ms_per_step_serial is the same work on one stream")
    else:
        # N > 1, the same idea: the copy-in of the next batch and the copy-out of the previous
        # result run on streams of their own beside the sharded sort.  The length of a rank's
        # result slice is only known on the device, so the host reads it (one small copy, once the
        # sort of that step is done) before it sizes that step's copy-out.
        s_in, s_sort, s_out = torch.cuda.Stream(), torch.cuda.Stream(), torch.cuda.Stream()
        dev2 = [bufs[0], bufs[1 % len(bufs)]] if len(bufs) > 1 else [bufs[0], torch.empty_like(bufs[0])]
        host_out2 = [host_out, torch.empty(2 * n, dtype=torch.uint32).pin_memory()]
        ev_in = [torch.cuda.Event() for _ in range(2)]
        ev_sorted = [torch.cuda.Event() for _ in range(2)]
        results = [None, None]
        copied = [0]

        def copy_out(j):
            b = j & 1
            out, count = results[b]
            ev_sorted[b].synchronize()
            m = min(int(count.item()), host_out2[b].numel())
            with torch.cuda.stream(s_out):
                out.record_stream(s_out)
                host_out2[b][:m].copy_(out[:m], non_blocking=True)
            copied[0] = m

        def piped_fn(i):
            b = i & 1
            with torch.cuda.stream(s_in):
                s_in.wait_event(ev_sorted[b])    # the sort that read this buffer before is done
                dev2[b].copy_(host_in, non_blocking=True)
                ev_in[b].record(s_in)
            with torch.cuda.stream(s_sort):
                s_sort.wait_event(ev_in[b])
                out, _, count = sharded.SortAsync(dev2[b], None, op)
                ev_sorted[b].record(s_sort)
            if i > 0:
                copy_out(i - 1)
            results[b] = (out, count)

        def piped_region(k):
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            dist.barrier()
            start.record(stream)
            for st in (s_in, s_sort, s_out):
                st.wait_stream(stream)
            for i in range(k):
                piped_fn(i)
            copy_out(k - 1)
            for st in (s_in, s_sort, s_out):
                stream.wait_stream(st)
            end.record(stream)
            torch.cuda.synchronize()
            return start.elapsed_time(end) / k
        piped_region(2)
        piped_steps = max(8, e2e_steps)
        e2e_ms = piped_region(piped_steps)
        sharded.CheckStatus()
        d2h_bytes[0] = 4 * copied[0]
        ho = host_out2[(piped_steps - 1) & 1][: copied[0]].view(torch.int32).to(torch.int64) & 0xFFFFFFFF
        assert bool((ho[1:] >= ho[:-1]).all()), "end-to-end result is not sorted"
        e2e_note = ("double-buffered: copy-in, sharded sort and copy-out of neighbouring steps overlap on three streams; "
                    "ms_per_step_serial is the same work on one stream")
    e2e_piped_ms = e2e_ms
    if dist is not None:
        t = torch.tensor([e2e_ms, e2e_serial_ms], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_piped_ms, e2e_serial_ms = float(t[0].item()), float(t[1].item())
    # both ways of issuing the same public calls are measured; the figure is the better one (on a
    # host whose memory and PCIe links are shared with other jobs either can come out ahead)
    e2e_ms = min(e2e_piped_ms, e2e_serial_ms)
    if e2e_serial_ms < e2e_piped_ms:
        e2e_note = "each step: copy-in, sort, copy-out, one after the other on one stream (the double-buffered issue was slower in this run)"
    e2e_value = world * n / (e2e_ms * 1e-3) / 1e9

    phases = None
    if world > 1:
        phases = sort_phase_times(sharded, bufs[0], op)   # collective: every rank calls it
    secondary = None
    if world > 1 and not args.no_secondary:
        del bufs
        last[0] = None
        torch.cuda.empty_cache()
        secondary = secondary_metrics_sharded(acc, sharded, world, rank, peak_gbs)
    if rank != 0:
        if dist is not None:
            dist.barrier()
            dist.destroy_process_group()
        return

    achieved = SORT_BYTES_PER_KEY * n / (ms_per_step * 1e-3) / 1e9   # per GPU
    call_traffic, pass_traffic = profiled_traffic()
    pass_ms = None
    if world == 1:
        # one digit pass bracketed by CUDA events inside the library (the measurement hook of
        # include/b200alg_testing.h), on fresh unsorted keys, median of five
        import ctypes
        from ilgpu_b200 import _native as N
        L = N.lib()
        L.b200alg_testing_time_sort_pass.restype = ctypes.c_int
        L.b200alg_testing_time_sort_pass.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64, ctypes.c_int, ctypes.c_int,
                                                     ctypes.c_void_p, ctypes.c_int64, ctypes.c_int, ctypes.POINTER(ctypes.c_float)]
        samples = []
        for r in range(5):
            fresh = pristine.clone()
            ms = ctypes.c_float(0)
            rc = L.b200alg_testing_time_sort_pass(ctypes.c_void_p(stream.cuda_stream), ctypes.c_void_p(fresh.data_ptr()), n, N.U32, 0,
                                                  ctypes.c_void_p(temp.data_ptr()), temp.numel() * 4, 1, ctypes.byref(ms))
            assert rc == 0, rc
            samples.append(float(ms.value))
        samples.sort()
        pass_ms = samples[len(samples) // 2]
    line = {
        "metric": "radix_sort_gkeys_per_s", "value": value, "unit": "Gkeys/s", "n_gpus": world, "steps": steps,
        "warmup": warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "u32", "data": "synthetic",
        "config": {
            "workload": "RadixSort ascending, 2^26 uint32 keys per GPU, i.i.d. uniform over the full range (seeded), "
                        "4 digit passes of 8 bits" + ("" if world == 1 else "; sample sort across GPUs inside the native multi-GPU library, buckets exchanged by peer stores from the partition kernel, no host synchronisation"),
            "keys_per_gpu": n, "total_keys": world * n,
            "l2": "inputs larger than L2: 256 MiB per step, a fresh unsorted buffer each step",
        },
        "roofline": {
            "bound": "hbm", "achieved": achieved, "peak": peak_gbs, "unit": "GB/s", "frac": achieved / peak_gbs,
            "traffic": call_traffic if world == 1 else None, "traffic_unit": "bytes per sort call (ncu summary under profiles/, quoted only for the kernel source it was captured from)",
            "peak_kind": peak_kind,
            "kernel": "whole sort call (digit histograms + 4 onesweep passes); 36 B/key algorithmic",
            "dominant_kernel": (None if world != 1 else {
                "name": "onesweep_kernel (one 8-bit digit pass), 8 B/key algorithmic",
                "ms": pass_ms,
                "achieved": 8 * n / (pass_ms * 1e-3) / 1e9,
                "frac": 8 * n / (pass_ms * 1e-3) / 1e9 / peak_gbs,
                "traffic": pass_traffic,
                "how": "CUDA events around the second digit pass of a sort call, recorded inside the library; median of 5",
            }),
        },
        "e2e": {"value": e2e_value, "unit": "Gkeys/s", "h2d_bytes_per_step": 4 * n, "d2h_bytes_per_step": d2h_bytes[0],
                "ms_per_step": e2e_ms, "ms_per_step_serial": e2e_serial_ms, "ms_per_step_double_buffered": e2e_piped_ms,
                "how": e2e_note},
        "gpu_launches": launches_per_step * steps,
        "clocks": clocks,
        "parity_checked": parity_checked,
    }
    if phases is not None:
        line["sort_phases_ms"] = dict(phases, how="rank 0, CUDA events inside one sort call, median of 5 calls outside the timed region")
    if secondary is not None:
        line["secondary"] = secondary
    if world == 1:
        if not args.no_secondary:
            del bufs
            torch.cuda.empty_cache()
            line["secondary"] = secondary_metrics(acc, peak_gbs)
        cores = host_cores()
        sample = 1 << 24
        cpu_value, cpu_sec = cpu_reference_sort(pristine[:sample].cpu().numpy(), cores)
        line["cpu_baseline"] = {
            "value": cpu_value, "unit": "Gkeys/s", "cores": cores, "kind": "port",
            "sample": f"first 2^24 keys of the workload, one run of {cpu_sec:.2f} s; C restatement of the reference's "
                      "CPURadixSortKernel1/2 (2 bits per pass), groups spread over all host threads",
        }
    print(json.dumps(line), flush=True)
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


def sort_phase_times(sharded, keys, op, reps: int = 5):
    """Device time of the phases of one multi-GPU sort on this rank (the measurement hook of
    include/b200alg_testing.h records CUDA events where the phases meet), median of `reps`
    collective calls."""
    import ctypes
    import torch
    from ilgpu_b200.algorithms import dtype_code
    c = sharded._communicator(sort_elements=keys.numel())
    fn = c.M.b200alg_testing_time_sort_mg
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p] * 4 + [ctypes.c_int64, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_void_p,
                                           ctypes.c_void_p, ctypes.c_int64, ctypes.c_void_p, ctypes.POINTER(ctypes.c_float)]
    cap = c.sort_capacity
    out = torch.empty(cap, dtype=keys.dtype, device=keys.device)
    count = torch.empty(1, dtype=torch.int64, device=keys.device)
    rows = []
    for _ in range(reps):
        ms = (ctypes.c_float * 6)()
        rc = fn(c.handle, ctypes.c_void_p(torch.cuda.current_stream().cuda_stream), ctypes.c_void_p(keys.data_ptr()), None,
                keys.numel(), dtype_code(keys.dtype), 0, 1 if op.descending else 0, ctypes.c_void_p(out.data_ptr()), None, cap,
                ctypes.c_void_p(count.data_ptr()), ms)
        assert rc == 0, rc
        rows.append([float(x) for x in ms])
    names = ["splitters", "bucket_sizes", "barrier_before_exchange", "partition_and_peer_stores",
             "barrier_after_exchange", "local_sort"]
    med = [sorted(r[i] for r in rows)[len(rows) // 2] for i in range(6)]
    return {k: round(v, 4) for k, v in zip(names, med)}


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-secondary", action="store_true", help="skip the scan / reduce / histogram figures")
    ap.add_argument("--profile-case", choices=["sort", "sort_pairs", "partition", "scan", "reduce", "histogram"],
                    help="run a few launches of one primitive on a small case and exit (the target of ncu captures)")
    args = ap.parse_args()
    if args.warmup < 3:
        args.warmup = 3
    if args.profile_case:
        run_profile_case(args.profile_case)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_native(args)


if __name__ == "__main__":
    main()
