#!/usr/bin/env python
"""Benchmark of the segmented-reduction hot path.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference|reference-cuda]

A step is one mgpu segreduce over one batch of synthetic input: fp32 plus over
268,435,456 items uniform in [-1, 1) in 8,388,608 segments with geometric
lengths (mean 32, 5 % empty), init 0 -- per GPU. With N > 1 (launched by
torch.distributed.run, one rank per GPU) every rank holds such a shard of one
N-times larger array, segments straddle the shard boundaries, and each step
also exchanges and folds the boundary partials (weak scaling).

Rank 0 prints ONE JSON line: `value` is whole-job Gitems/s with inputs
resident in HBM (CUDA events on the launching stream, max over ranks), `e2e`
the same metric through the host-buffer entry point of the C ABI (pinned host
inputs, host<->device copies inside the timed region), `roofline` the dominant
kernel against the measured HBM copy bandwidth, `cpu_baseline` the CPU oracle
timed on the host cores, `parity` the check of the last timed step's outputs
against the CPU oracle on every rank (the run exits non-zero when it fails),
and `secondary` the other benchmark configurations: config 5 (fp64 max and
plus over 2^32 items held as 8 shards over the N GPUs, strong scaling), the
headline array cut N ways (strong scaling), and on one GPU configs 1, 3, 4,
lbs_segreduce and a sweep of equal segment lengths, each beside the
reference's own CUDA build where that was built.

--impl reference times the reference's host loop (tests/test_segreduce.cu:
40-49, restated in oracle/oracle.c) on all host cores; --impl reference-cuda
times the reference's own CUDA build (oracle/_ref/libmgpu_ref.so) on the GPU.
"""
import argparse
import ctypes
import json
import os
import statistics
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

COUNT = 1 << 28
NUM_SEGMENTS = 1 << 23
METRIC = "segreduce_throughput_256M_fp32_items"
UNIT = "Gitems/s"
FALLBACK_HBM_GBS = 6650.0
# dram__bytes_read.sum + dram__bytes_write.sum of the reduction kernel from
# one ncu capture of a 2^26-item case of the same workload (profiles/
# segreduce_k_fp32_c2.md: 278.17 MB read + 6.92 MB written for 285.21 MB of
# algorithmic bytes in the capture of the current kernel; 4.5 - 7.6 MB
# written over all captures, since part of the results is still in the L2
# when the kernel ends), divided by that case's algorithmic bytes; DRAM
# traffic grows in proportion to the units processed. To be re-captured
# whenever the kernel's memory behaviour changes.
TRAFFIC_PER_ALGORITHMIC_BYTE = 0.9996
FP32_TOL = 1e-5         # |got - ref| <= tol * max(|ref|, sum |x|), ref in fp64
FP64_TOL = 1e-12        # the same against a long double accumulation


_RESULT_FD = None


def emit(line):
    """Write one JSON line to the process's original stdout."""
    text = (json.dumps(line) + "\n").encode()
    if _RESULT_FD is None:
        sys.stdout.write(text.decode())
        sys.stdout.flush()
    else:
        os.write(_RESULT_FD, text)


def measured_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons while the timed region runs:
    NVML polled every few milliseconds from a thread (read-only queries)."""
    REASONS = {
        "hw_slowdown": 0x8, "hw_thermal_slowdown": 0x40,
        "sw_thermal_slowdown": 0x20, "sw_power_cap": 0x4,
    }

    def __init__(self, uuid, index):
        self.uuid, self.index = uuid, index
        self.samples = []          # (time, sm_mhz, reasons_mask, mem_mhz)
        self.max_mhz = None
        self.stop_flag = threading.Event()
        self.thread = None
        self.window = None

    def start(self):
        try:
            import pynvml
            pynvml.nvmlInit()
            try:
                handle = pynvml.nvmlDeviceGetHandleByUUID(self.uuid)
            except Exception:
                handle = pynvml.nvmlDeviceGetHandleByIndex(self.index)
            self.max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(
                handle, pynvml.NVML_CLOCK_SM))

            def poll():
                while not self.stop_flag.is_set():
                    try:
                        mhz = pynvml.nvmlDeviceGetClockInfo(
                            handle, pynvml.NVML_CLOCK_SM)
                        mask = pynvml.nvmlDeviceGetCurrentClocksThrottleReasons(
                            handle)
                        mem = pynvml.nvmlDeviceGetClockInfo(
                            handle, pynvml.NVML_CLOCK_MEM)
                        self.samples.append((time.perf_counter(), float(mhz),
                                             int(mask), float(mem)))
                    except Exception:
                        pass
                    time.sleep(0.004)
            self.thread = threading.Thread(target=poll, daemon=True)
            self.thread.start()
        except Exception:
            self.thread = None

    def mark(self, t_begin, t_end):
        self.window = (t_begin, t_end)

    def stop(self):
        self.stop_flag.set()
        if self.thread is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [],
                    "note": "NVML unavailable"}
        self.thread.join(timeout=2)
        inside = [s for s in self.samples
                  if self.window and self.window[0] <= s[0] <= self.window[1]]
        note = "sampled inside the timed region"
        if len(inside) < 3:
            inside = self.samples
            note = ("timed region shorter than the sampling period: samples "
                    "cover warm-up, timed steps and the profiling loop")
        mask = 0
        for s in inside:
            mask |= s[2]
        mhz = sorted(s[1] for s in inside)
        mem = sorted(s[3] for s in inside)
        return {"sm_mhz": statistics.median(mhz) if mhz else None,
                "sm_max_mhz": self.max_mhz,
                "mem_mhz": statistics.median(mem) if mem else None,
                "reasons": sorted(k for k, bit in self.REASONS.items()
                                  if mask & bit),
                "samples": len(inside), "note": note}


def host_threads():
    """Host cores this process may run on (a launcher may have pinned
    OMP_NUM_THREADS to 1; the CPU arm asks for its threads explicitly)."""
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except AttributeError:
        return max(1, os.cpu_count() or 1)


class near_gpu:
    """Context manager: restricts this process to the host cores of the NUMA
    node its GPU hangs off (read from sysfs) while the pinned host buffers of
    the end-to-end leg are allocated and used, then restores the affinity.
    Best effort; `note` says what happened."""

    def __init__(self, local_rank):
        self.local_rank = local_rank
        self.saved = None
        self.note = "placement not applied"

    def __enter__(self):
        try:
            import torch
            props = torch.cuda.get_device_properties(self.local_rank)
            bus = "%04x:%02x:%02x.0" % (props.pci_domain_id, props.pci_bus_id,
                                        props.pci_device_id)
            with open("/sys/bus/pci/devices/%s/numa_node" % bus) as f:
                node = int(f.read().strip())
            if node < 0:
                self.note = "host reports one memory node"
                return self
            with open("/sys/devices/system/node/node%d/cpulist" % node) as f:
                text = f.read().strip()
            cpus = set()
            for part in text.split(","):
                lo, _, hi = part.partition("-")
                cpus.update(range(int(lo), int(hi or lo) + 1))
            before = os.sched_getaffinity(0)
            allowed = cpus & set(before)
            if not allowed:
                self.note = "no allowed core on NUMA node %d" % node
                return self
            os.sched_setaffinity(0, allowed)
            self.saved = before
            self.note = "host thread and pinned buffers on NUMA node %d" % node
        except Exception as e:                       # noqa: BLE001
            self.note = "placement not applied (%s)" % type(e).__name__
        return self

    def __exit__(self, *exc):
        if self.saved is not None:
            os.sched_setaffinity(0, self.saved)
        return False


def cpu_workload(count, num_segments, seed=1):
    """The workload of the CPU arm, generated on the host with the same length
    and value distributions as the GPU arm's."""
    from moderngpu_b200 import workloads
    values, seg = workloads.config2(seed=seed, count=count,
                                    num_segments=num_segments, device="cpu")
    return values.numpy(), seg.numpy()


def run_reference_cpu(args, rank, world):
    """The reference's own CPU implementation of the path: the host loop of
    tests/test_segreduce.cu:40-49 (C port, OpenMP over segments) on all host
    cores, on the whole 2^28-item workload of the GPU arm."""
    if rank != 0:
        return
    import oracle
    threads = host_threads()
    values, seg = cpu_workload(COUNT, NUM_SEGMENTS)
    # Pages first touched by the threads that will read them.
    values = oracle.place_by_segments(values, seg, threads)
    for _ in range(max(args.warmup, 1)):
        oracle.segreduce(values, seg, op="plus", init=0.0, threads=threads)
    # Rounds of exactly --steps steps until at least two seconds are timed.
    rounds, dt = 0, 0.0
    while rounds < 1 or (dt < 2.0 and rounds < 1000):
        t0 = time.perf_counter()
        for _ in range(args.steps):
            oracle.segreduce(values, seg, op="plus", init=0.0, threads=threads)
        dt += time.perf_counter() - t0
        rounds += 1
    steps = rounds * args.steps
    value = values.size * steps / dt / 1e9
    sample = ("each step: host loop of tests/test_segreduce.cu:40-49 (C port, "
              "OpenMP over segments, pages placed by the same schedule) on the "
              "whole %d-item / %d-segment workload; %d rounds of %d steps, "
              "%.2f s" % (values.size, seg.size, rounds, args.steps, dt))
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT,
        "n_gpus": args.gpus, "steps": args.steps,
        "warmup": max(args.warmup, 1),
        "ms_per_step": dt / steps * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic",
        "config": workload_config(args.gpus),
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads,
                         "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0,
                "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    emit(line)


def workload_config(n_gpus, exchange="p2p"):
    how = ("stored peer-to-peer over NVLink into the owning GPU's mailbox, "
           "no collective" if exchange == "p2p" else "NCCL all-gather")
    return {
        "workload": "config 2: fp32 plus-segreduce, %d items uniform in "
                    "[-1,1), %d segments, geometric lengths mean 32 with 5%% "
                    "empty, init 0 (per GPU)" % (COUNT, NUM_SEGMENTS),
        "items_per_gpu": COUNT, "segments_per_gpu": NUM_SEGMENTS,
        "sharding": "item range cut evenly over %d GPU(s); one 16-byte "
                    "boundary record per GPU exchanged per step (%s)"
                    % (n_gpus, how if n_gpus > 1 else "none needed"),
        "l2": "inputs are %.2f GB per GPU, larger than the 126 MB L2; no "
              "flush between steps" % ((COUNT * 4 + NUM_SEGMENTS * 8) / 1e9),
    }


# ---------------------------------------------------------------------------
# The reference's own CUDA build (unmodified moderngpu headers compiled for
# sm_100a into oracle/_ref/libmgpu_ref.so), timed on the same device arrays.

_REF = None


def reference_cuda():
    """ctypes handle of the reference's CUDA build, or None when not built."""
    global _REF
    if _REF is None:
        path = os.path.join(ROOT, "oracle", "_ref", "libmgpu_ref.so")
        _REF = ctypes.CDLL(path) if os.path.exists(path) else False
    return _REF or None


def time_reference_cuda(call, steps, units):
    """call(pooled, sync) runs the reference once. Returns its throughput with
    the stock context (cudaMalloc / cudaFree per temporary, as shipped) and
    with a context that recycles temporaries, host-clock timed over `steps`
    back-to-back calls with one device synchronisation at the end."""
    import torch
    out = {}
    for pooled, name in ((0, "stock"), (1, "pooled")):
        for _ in range(3):
            call(pooled, 1)
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(steps):
            call(pooled, 0)
        torch.cuda.synchronize()
        dt = (time.perf_counter() - t0) / steps
        out[name] = {"ms_per_step": dt * 1e3,
                     "gitems_per_s": units / dt / 1e9}
    return out


def run_reference_cuda(args, rank, world):
    if rank != 0:
        return
    import torch
    from moderngpu_b200 import workloads
    ref = reference_cuda()
    if ref is None:
        emit({"impl": "reference-cuda", "unavailable":
              "oracle/_ref/libmgpu_ref.so was not built"})
        return
    torch.cuda.set_device(0)
    if args.config == "c3":
        # The reference's spmv on config 3 (a profiler can be pointed at it).
        m, c, x, r = workloads.config3(seed=2, device="cuda",
                                       rows=1 << (22 if args.small else 24))
        y = torch.empty(r.numel(), dtype=m.dtype, device="cuda")
        p = lambda t: ctypes.c_void_p(t.data_ptr())      # noqa: E731

        def spmv_call(pooled, sync):
            code = ref.ref_spmv_f32(p(m), p(c), p(x), m.numel(), p(r),
                                    r.numel(), p(y), pooled, sync)
            assert code == 0, "reference returned CUDA error %d" % code
        timed = time_reference_cuda(spmv_call, args.steps, m.numel())
        emit({"impl": "reference-cuda", "config": "c3", "rows": r.numel(),
              "nnz": m.numel(), "reference_cuda": timed})
        return
    values, seg = workloads.config2(seed=1, count=COUNT,
                                    num_segments=NUM_SEGMENTS)
    out = torch.empty(NUM_SEGMENTS, dtype=torch.float32, device="cuda")
    torch.cuda.synchronize()

    def call(pooled, sync):
        code = ref.ref_segreduce_f32(
            ctypes.c_void_p(values.data_ptr()), COUNT,
            ctypes.c_void_p(seg.data_ptr()), NUM_SEGMENTS,
            ctypes.c_void_p(out.data_ptr()), ctypes.c_float(0), 0, pooled, sync)
        assert code == 0, "reference returned CUDA error %d" % code

    timed = time_reference_cuda(call, args.steps, COUNT)
    hv = values.cpu().pin_memory()
    hs = seg.cpu().pin_memory()
    ho = torch.empty(NUM_SEGMENTS, dtype=torch.float32).pin_memory()
    e2e_steps = max(2, min(args.steps, 5))
    for _ in range(2):
        ref.ref_segreduce_f32_host(ctypes.c_void_p(hv.data_ptr()), COUNT,
                                   ctypes.c_void_p(hs.data_ptr()), NUM_SEGMENTS,
                                   ctypes.c_void_p(ho.data_ptr()),
                                   ctypes.c_float(0))
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        ref.ref_segreduce_f32_host(ctypes.c_void_p(hv.data_ptr()), COUNT,
                                   ctypes.c_void_p(hs.data_ptr()), NUM_SEGMENTS,
                                   ctypes.c_void_p(ho.data_ptr()),
                                   ctypes.c_float(0))
    e2e_t = (time.perf_counter() - t0) / e2e_steps
    line = {
        "impl": "reference-cuda", "metric": METRIC,
        "value": timed["stock"]["gitems_per_s"], "unit": UNIT, "n_gpus": 1,
        "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": timed["stock"]["ms_per_step"], "higher_is_better": True,
        "dtype": "f32", "data": "synthetic", "config": workload_config(1),
        "note": "unmodified moderngpu headers compiled for sm_100a; value = "
                "stock standard_context_t (cudaMalloc/cudaFree per call), "
                "host-clock timed; pooled_context = same kernels with "
                "recycled temporaries",
        "pooled_context": {"value": timed["pooled"]["gitems_per_s"],
                           "unit": UNIT,
                           "ms_per_step": timed["pooled"]["ms_per_step"]},
        "e2e": {"value": COUNT / e2e_t / 1e9, "unit": UNIT,
                "h2d_bytes_per_step": COUNT * 4 + NUM_SEGMENTS * 4,
                "d2h_bytes_per_step": NUM_SEGMENTS * 4},
    }
    emit(line)


# ---------------------------------------------------------------------------
# Shards and their check against the oracle.

def make_shard(rank, device, count=None, num_segments=None):
    """This rank's shard: values and shard-local start table (entry 0 is the
    virtual start that stands for the segment carried in from the left)."""
    import torch
    from moderngpu_b200 import workloads
    count = COUNT if count is None else count
    num_segments = NUM_SEGMENTS if num_segments is None else num_segments
    values, seg = workloads.config2(seed=1 + rank, count=count,
                                    num_segments=num_segments, device=device)
    if rank > 0:
        # The first real segment starts a little into the shard: the leading
        # items continue the previous rank's last segment.
        lead = 17 + rank
        seg = torch.clamp(seg + lead, max=count)
    table = torch.cat([torch.zeros(1, dtype=torch.int32, device=device), seg])
    return values, seg, table


def chain_expectation(own_last, own_last_mag, records, index, op):
    """What the owner's last output must hold once the following shards'
    boundary partials are folded in. records: per shard of the chain, in
    order, (lead_value, lead_magnitude, flags); `index` is this shard."""
    from moderngpu_b200 import sharded
    flags = [r[2] for r in records]
    value, mag = own_last, own_last_mag
    first = bool(flags[index] & sharded.LAST_EMPTY)
    for k in sharded.fold_plan(flags, index):
        lead, lead_mag = records[k][0], records[k][1]
        if first:
            value = lead
        elif op == "plus":
            value = value + lead
        elif op == "max":
            value = max(value, lead)
        else:
            value = min(value, lead)
        mag += lead_mag
        first = False
    return value, mag


def shard_flags(table, count):
    """The flags of a shard's boundary record, from its host-side table."""
    from moderngpu_b200 import sharded
    real = table.size > 1
    flags = 0
    if (int(table[1]) if real else count) > 0:
        flags |= sharded.HAS_PARTIAL
    if real:
        flags |= sharded.HAS_START
    if real and int(table[-1]) >= count:
        flags |= sharded.LAST_EMPTY
    return flags


def check_headline(values, table, out, rank, world, threads):
    """Every output of this rank's last step against the oracle's fp64 sums of
    its shard (tests/test_segreduce.cu:40-49), the segment that continues on
    later ranks included: its expectation adds those ranks' leading partials
    in rank order. Returns (segments checked, worst error / bound, ok)."""
    import numpy as np
    import torch.distributed as dist
    import oracle
    hv = values.cpu().numpy()
    ht = table.cpu().numpy()
    got = out.cpu().numpy().astype(np.float64)
    sums, mags = oracle.segsum_wide(hv, ht, init=0.0, threads=threads)
    if world > 1:
        record = (float(sums[0]), float(mags[0]), shard_flags(ht, hv.size))
        records = [None] * world
        dist.all_gather_object(records, record)
        if record[2] & 2:
            sums[-1], mags[-1] = chain_expectation(
                float(sums[-1]), float(mags[-1]), records, rank, "plus")
    bound = FP32_TOL * np.maximum(np.abs(sums), mags)
    err = np.abs(got - sums)
    ok = bool(np.all(err <= bound))
    worst = float(np.max(err / np.maximum(bound, 1e-300) * FP32_TOL)) \
        if err.size else 0.0
    return int(sums.size), worst, ok


def check_shard_windows(shards, outs, op, init, chain_first, records,
                        window=1 << 22):
    """Config 5 check: the segments that lie in the first and in the last
    `window` items of every shard this rank holds, against the oracle (max:
    bit for bit; plus: FP64_TOL against a long double sum), and every shard's
    last segment against its own items plus the following shards' leading
    partials. records: (lead, magnitude, flags) of every shard of the chain."""
    import numpy as np
    import oracle
    checked, worst, ok = 0, 0.0, True

    def compare(got, values, table, count):
        nonlocal checked, worst, ok
        if op == "plus":
            want, mags = oracle.segsum_wide(values, table, init=init)
            bound = FP64_TOL * np.maximum(np.abs(want), mags)
            err = np.abs(got - want)
            ok = ok and bool(np.all(err <= bound))
            if err.size:
                worst = max(worst, float(np.max(
                    err / np.maximum(bound, 1e-300) * FP64_TOL)))
        else:
            want = oracle.segreduce(values, table, op=op, init=init)
            ok = ok and bool(np.array_equal(got, want))
        checked += int(got.size)

    for j, ((values, table), out) in enumerate(zip(shards, outs)):
        count = values.numel()
        ht = table.cpu().numpy()
        # Head window: segments that end inside the first `window` items.
        k = int(np.searchsorted(ht, window, side="right")) - 1
        if k >= 1:
            end = int(ht[k])
            compare(out[:k].cpu().numpy(), values[:end].cpu().numpy(),
                    ht[:k], end)
        # Tail window: segments that start inside the last `window` items; the
        # last one continues on the following shards.
        first = int(np.searchsorted(ht, count - window, side="left"))
        first = max(first, 1)
        if first < ht.size:
            base = int(ht[first])
            tail_values = values[base:].cpu().numpy()
            tail_table = (ht[first:] - base).astype(np.int32)
            got = out[first:].cpu().numpy().copy()
            last = got[-1]
            compare(got[:-1], tail_values[:int(tail_table[-1])],
                    tail_table[:-1], int(tail_table[-1]))
            own = tail_values[int(tail_table[-1]):]
            if op == "plus":
                w, m = oracle.segsum_wide(own, np.zeros(1, np.int32), init=init)
                want, mag = chain_expectation(float(w[0]), float(m[0]), records,
                                              chain_first + j, op)
                bound = FP64_TOL * max(abs(want), mag)
                ok = ok and abs(float(last) - want) <= bound
                worst = max(worst, abs(float(last) - want) /
                            max(bound, 1e-300) * FP64_TOL)
            else:
                w = oracle.segreduce(own, np.zeros(1, np.int32), op=op,
                                     init=init)
                want, _ = chain_expectation(float(w[0]), 0.0, records,
                                            chain_first + j, op)
                ok = ok and float(last) == want
            checked += 1
    return checked, worst, ok


def time_steps(fn, steps, warmup, world, device):
    """ms per step of fn(): warm-up, barrier + synchronize, CUDA events on the
    launching stream around `steps` calls, max over ranks."""
    import torch
    import torch.distributed as dist
    for _ in range(max(warmup, 3)):
        fn()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    a = torch.cuda.Event(enable_timing=True)
    b = torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(steps):
        fn()
    b.record()
    torch.cuda.synchronize()
    ms = a.elapsed_time(b) / steps
    if world > 1:
        t = torch.tensor([ms], device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
        dist.barrier()
    return ms


def graph_replay_ms(call, steps, device, calls_per_graph=20):
    """A latency-bound call timed without the host's per-call cost: the call
    (two launches on the caller's stream, nothing else) captured
    `calls_per_graph` times in one CUDA graph, the graph replayed `steps`
    times between CUDA events."""
    import torch
    workspace = torch.empty(4 << 20, dtype=torch.uint8, device=device)
    call(workspace)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for _ in range(calls_per_graph):
            call(workspace)
    for _ in range(3):
        graph.replay()
    torch.cuda.synchronize()
    a = torch.cuda.Event(enable_timing=True)
    b = torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(steps):
        graph.replay()
    b.record()
    torch.cuda.synchronize()
    return {"ms_per_step": a.elapsed_time(b) / (steps * calls_per_graph),
            "calls_per_graph": calls_per_graph,
            "how": "the same call captured in a CUDA graph and replayed: "
                   "device time per call without the host's launch cost"}


def result_row(case, ms, units, nbytes, world, peak, peak_kind, **extra):
    gbs = nbytes / (ms * 1e-3) / 1e9
    row = {"case": case, "ms_per_step": ms,
           "gitems_per_s": world * units / (ms * 1e-3) / 1e9,
           "algorithmic_bytes_per_gpu": nbytes, "hbm_gbs_per_gpu": gbs,
           "frac_of_%s_peak" % peak_kind: gbs / peak}
    row.update(extra)
    return row


# ---------------------------------------------------------------------------
# Secondary configurations.

def config5_legs(args, rank, world, device, steps):
    """fp64 max and plus over the whole 2^32-item array, always as 8 shards of
    2^29 items; each of the N ranks holds 8/N consecutive shards (strong
    scaling). Checked against the oracle on windows at both ends of every
    shard and on every segment that straddles a shard edge."""
    import torch
    import torch.distributed as dist
    import numpy as np
    import moderngpu_b200 as mgpu
    from moderngpu_b200 import sharded, workloads
    import oracle
    peak, peak_kind = measured_peak()
    total_shards, count = 8, 1 << (25 if args.small else 29)
    per_rank = total_shards // world
    shards, nbytes = [], 0
    for j in range(per_rank):
        g = rank * per_rank + j
        v, starts = workloads.config5_shard(4, g, count, device=device)
        table = torch.cat([torch.zeros(1, dtype=torch.int32, device=device),
                           starts])
        shards.append((v, table))
        nbytes += workloads.segreduce_bytes(count, table.numel(), 8)
    outs = [torch.empty(t.numel(), dtype=torch.float64, device=device)
            for _, t in shards]
    box = None
    if args.exchange == "p2p":
        try:
            box = sharded.Mailbox(shards_per_gpu=per_rank)
        except sharded.MailboxError as e:
            print("bench: %s; using --exchange nccl" % e, file=sys.stderr)
    rows = []
    for op, init in (("max", -1e300), ("plus", 0.0)):
        fn = lambda: sharded.sharded_segreduce_multi(       # noqa: E731
            shards, op=op, init=init, outs=outs, mailbox=box)
        ms = time_steps(fn, steps, args.warmup, world, device)
        # Leading partial of every shard of the chain, from the host.
        mine = []
        for v, t in shards:
            ht = t.cpu().numpy()
            lead = int(ht[1]) if ht.size > 1 else count
            hv = v[:lead].cpu().numpy()
            if op == "plus":
                w, m = oracle.segsum_wide(hv, np.zeros(1, np.int32), init=init)
                mine.append((float(w[0]), float(m[0]), shard_flags(ht, count)))
            else:
                w = oracle.segreduce(hv, np.zeros(1, np.int32), op=op, init=init)
                mine.append((float(w[0]), 0.0, shard_flags(ht, count)))
        records = mine
        if world > 1:
            gathered = [None] * world
            dist.all_gather_object(gathered, mine)
            records = [r for part in gathered for r in part]
        checked, worst, ok = check_shard_windows(
            shards, outs, op, init, rank * per_rank, records,
            window=min(1 << 22, count // 4))
        if world > 1:
            t = torch.tensor([float(checked), worst, 0.0 if ok else 1.0],
                             device=device, dtype=torch.float64)
            total = t.clone()
            dist.all_reduce(total, op=dist.ReduceOp.SUM)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            checked, worst, ok = int(total[0].item()), float(t[1].item()), \
                t[2].item() == 0.0
        rows.append(result_row(
            "config 5: fp64 %s, %d items in 8 shards over %d GPU(s), strong "
            "scaling" % (op, total_shards * count, world),
            ms, per_rank * count, nbytes, world, peak, peak_kind,
            parity={"checked": True, "segments": checked,
                    "max_rel_err": worst, "ok": ok,
                    "how": "windows at both ends of every shard and every "
                           "straddling segment against the oracle; max bit "
                           "for bit, plus within 1e-12"}))
    assert mgpu.workspace_status() == 0
    if box is not None:
        assert box.status() == 0
        box.close()
    del shards, outs
    torch.cuda.empty_cache()
    return rows


def config2_strong_leg(args, rank, world, device, steps):
    """The headline's 2^28 items cut N ways: 2^28 / N items per GPU."""
    import torch
    import moderngpu_b200 as mgpu
    from moderngpu_b200 import sharded, workloads
    peak, peak_kind = measured_peak()
    count, segs = COUNT // world, NUM_SEGMENTS // world
    values, seg, table = make_shard(rank, device, count, segs)
    box = sharded.Mailbox() if args.exchange == "p2p" else None
    records = torch.empty(world * sharded.RECORD_BYTES, dtype=torch.uint8,
                          device=device)
    out = [torch.empty(table.numel(), dtype=torch.float32, device=device)]

    def fn():
        out[0] = sharded.sharded_segreduce(values, table, op="plus", init=0.0,
                                           mailbox=box, records=records,
                                           out=out[0])
    ms = time_steps(fn, steps, args.warmup, world, device)
    checked, worst, ok = check_headline(values, table, out[0], rank, world,
                                        max(1, host_threads() // world))
    t = torch.tensor([float(checked), worst, 0.0 if ok else 1.0],
                     device=device, dtype=torch.float64)
    import torch.distributed as dist
    total = t.clone()
    dist.all_reduce(total, op=dist.ReduceOp.SUM)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    if box is not None:
        assert box.status() == 0
        box.close()
    return [result_row(
        "config 2 strong scaling: the 2^28 fp32 items cut %d ways (%d per "
        "GPU); at this size launch and exchange latency, not HBM, set the "
        "floor" % (world, count), ms, count,
        workloads.segreduce_bytes(count, table.numel(), 4), world, peak,
        peak_kind,
        parity={"checked": True, "segments": int(total[0].item()),
                "max_rel_err": float(t[1].item()), "ok": t[2].item() == 0.0})]


def single_gpu_legs(args, device, steps, c2_arrays):
    """Configs 1, 3, 4, lbs_segreduce and the equal-length sweep on one GPU,
    each next to the reference's CUDA build (stock and pooled context) on the
    same device arrays where that build is present."""
    import numpy as np
    import torch
    import moderngpu_b200 as mgpu
    from moderngpu_b200 import workloads
    peak, peak_kind = measured_peak()
    ref = reference_cuda()
    rows = []
    p = lambda t: ctypes.c_void_p(t.data_ptr())          # noqa: E731

    def ours(fn):
        return time_steps(fn, steps, args.warmup, 1, device)

    def theirs(call, units):
        if ref is None:
            return {"unavailable": "oracle/_ref/libmgpu_ref.so was not built"}
        return time_reference_cuda(call, steps, units)

    def checked(code):
        assert code == 0, "reference returned CUDA error %d" % code

    # Config 1: int32 plus, 1,048,576 items, 10,000 segments.
    v_np, s_np = workloads.config1(seed=0)
    v, s = torch.from_numpy(v_np).to(device), torch.from_numpy(s_np).to(device)
    out = torch.empty(s.numel(), dtype=v.dtype, device=device)
    ms = ours(lambda: mgpu.segreduce(v, s, init=0, out=out))
    rows.append(result_row(
        "config 1: int32 plus, 1,048,576 items / 10,000 segments "
        "(latency-bound)", ms, v.numel(),
        workloads.segreduce_bytes(v.numel(), s.numel(), 4), 1, peak, peak_kind,
        cuda_graph=graph_replay_ms(
            lambda ws: mgpu.segreduce(v, s, init=0, out=out, workspace=ws),
            steps, device),
        reference_cuda=theirs(lambda pooled, sync: checked(
            ref.ref_segreduce_i32(p(v), v.numel(), p(s), s.numel(), p(out), 0,
                                  0, pooled, sync)), v.numel())))

    # Config 2 on the reference (ours is the headline).
    values, seg = c2_arrays
    out = torch.empty(seg.numel(), dtype=torch.float32, device=device)
    rows.append({
        "case": "config 2: fp32 plus (this library: the headline value)",
        "reference_cuda": theirs(lambda pooled, sync: checked(
            ref.ref_segreduce_f32(p(values), values.numel(), p(seg),
                                  seg.numel(), p(out), ctypes.c_float(0), 0,
                                  pooled, sync)), values.numel())})

    # lbs_segreduce on config 2's shape: values[index] * weight[seg].
    g = torch.Generator(device=device).manual_seed(11)
    weights = torch.rand(seg.numel(), device=device, generator=g)
    ms = ours(lambda: mgpu.lbs_segreduce_weighted(values, seg, weights, out=out))
    rows.append(result_row(
        "lbs_segreduce fp32 weighted sums, config 2 shape", ms, values.numel(),
        workloads.segreduce_bytes(values.numel(), seg.numel(), 4)
        + 4 * seg.numel(), 1, peak, peak_kind,
        reference_cuda=theirs(lambda pooled, sync: checked(
            ref.ref_lbs_segreduce_weighted_f32(
                p(values), values.numel(), p(seg), seg.numel(), p(weights),
                p(out), pooled, sync)), values.numel())))
    del weights

    # Equal segment lengths (fixed-width rows), 2^28 fp32 items.
    for length in (8, 16, 31, 32, 33, 64, 100, 128):
        n = values.numel() // length
        useg = (torch.arange(n, device=device, dtype=torch.int64) * length
                ).to(torch.int32)
        uout = torch.empty(n, dtype=torch.float32, device=device)
        ms = ours(lambda: mgpu.segreduce(values, useg, init=0.0, out=uout))
        rows.append(result_row(
            "segreduce fp32, every segment exactly %d items" % length, ms,
            values.numel(), workloads.segreduce_bytes(values.numel(), n, 4),
            1, peak, peak_kind))
        del useg, uout

    # Config 3: CSR spmv fp32, 16,777,216 rows.
    m, c, x, r = workloads.config3(seed=2, device=device,
                                   rows=1 << (20 if args.small else 24))
    y = torch.empty(r.numel(), dtype=m.dtype, device=device)
    nbytes = workloads.spmv_bytes(m.numel(), r.numel(), x.numel(), 4)
    ms = ours(lambda: mgpu.spmv(m, c, x, r, out=y))
    # Sector-granular bytes: a 4-byte gather moves a 32-byte sector when it
    # misses, so a kernel that never hits in a cache moves this much.
    sector_bytes = nbytes - 4 * x.numel() + 32 * m.numel()
    rows.append(result_row(
        "config 3: spmv fp32, %d rows, nnz=%d" % (r.numel(), m.numel()), ms,
        m.numel(), nbytes, 1, peak, peak_kind,
        gathers_per_s=m.numel() / (ms * 1e-3),
        sector_granular_bytes=sector_bytes,
        frac_of_sector_granular_roofline=sector_bytes / (ms * 1e-3) / 1e9 / peak,
        reference_cuda=theirs(lambda pooled, sync: checked(
            ref.ref_spmv_f32(p(m), p(c), p(x), m.numel(), p(r), r.numel(),
                             p(y), pooled, sync)), m.numel())))
    mgpu.l2_pin(x)
    ms = ours(lambda: mgpu.spmv(m, c, x, r, out=y))
    mgpu.l2_unpin()
    rows.append(result_row("config 3 with x pinned in the L2 (opt-in)", ms,
                           m.numel(), nbytes, 1, peak, peak_kind))
    del m, c, x, r, y
    torch.cuda.empty_cache()

    # Config 4: load-balancing search, ids and ranks.
    count = values.numel()
    s4 = workloads.config4(seed=3, device=device, count=count,
                           num_segments=1 << (20 if args.small else 22))
    ids = torch.empty(count, dtype=torch.int32, device=device)
    ranks = torch.empty(count, dtype=torch.int32, device=device)
    ms = ours(lambda: mgpu.transform_lbs(count, s4))
    rows.append(result_row(
        "config 4: load-balancing search, segment ids and ranks", ms, count,
        workloads.lbs_bytes(count, s4.numel()), 1, peak, peak_kind,
        reference_cuda=theirs(lambda pooled, sync: checked(
            ref.ref_lbs_seg_rank(count, p(s4), s4.numel(), p(ids), p(ranks),
                                 pooled, sync)), count)))
    ms = ours(lambda: mgpu.load_balance_search(count, s4))
    rows.append(result_row(
        "config 4: load_balance_search (segment ids only)", ms, count,
        workloads.lbs_bytes(count, s4.numel(), False), 1, peak, peak_kind,
        reference_cuda=theirs(lambda pooled, sync: checked(
            ref.ref_load_balance_search(count, p(s4), s4.numel(), p(ids),
                                        pooled, sync)), count)))
    del s4, ids, ranks
    torch.cuda.empty_cache()
    assert mgpu.workspace_status() == 0
    return rows


def run_ours(args, rank, world, local_rank):
    import torch
    import torch.distributed as dist
    import moderngpu_b200 as mgpu
    from moderngpu_b200 import sharded, workloads

    mgpu.load_library()
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)

    sampler = None
    if rank == 0:
        props = torch.cuda.get_device_properties(local_rank)
        sampler = ClockSampler("GPU-" + str(props.uuid), local_rank)
        sampler.start()

    values, seg, table = make_shard(rank, device)
    out = torch.empty(NUM_SEGMENTS, dtype=torch.float32, device=device)
    records = torch.empty(world * sharded.RECORD_BYTES, dtype=torch.uint8,
                          device=device)

    mailbox = None
    if world > 1 and args.exchange == "p2p":
        try:
            mailbox = sharded.Mailbox(side_stream=not args.no_side_stream,
                                      fused=not args.unfused)
        except sharded.MailboxError as e:
            # All ranks fail together; the records then travel by all-gather.
            print("bench: %s; using --exchange nccl" % e, file=sys.stderr)
            args.exchange = "nccl"

    last = [out]
    shard_out = torch.empty(table.numel(), dtype=torch.float32, device=device)

    def step():
        if world == 1:
            mgpu.segreduce(values, seg, op="plus", init=0.0, out=out)
        elif mailbox is not None:
            last[0] = sharded.sharded_segreduce(values, table, op="plus",
                                                init=0.0, mailbox=mailbox,
                                                out=shard_out)
        else:
            last[0] = sharded.sharded_segreduce(values, table, op="plus",
                                                init=0.0, records=records,
                                                out=shard_out)

    for _ in range(max(args.warmup, 3)):
        step()
    torch.cuda.synchronize()
    assert mgpu.workspace_status() == 0, "device-side status reported failure"
    assert mailbox is None or mailbox.status() == 0, "mailbox wait timed out"

    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    start = torch.cuda.Event(enable_timing=True)
    stop = torch.cuda.Event(enable_timing=True)
    t_begin = time.perf_counter()
    start.record()
    for _ in range(args.steps):
        step()
    stop.record()
    torch.cuda.synchronize()
    if sampler:
        sampler.mark(t_begin, time.perf_counter())
    elapsed_ms = start.elapsed_time(stop)
    if world > 1:
        t = torch.tensor([elapsed_ms], device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        elapsed_ms = float(t.item())
        dist.barrier()
    ms_per_step = elapsed_ms / args.steps
    value = world * COUNT / (ms_per_step * 1e-3) / 1e9
    assert mgpu.workspace_status() == 0, "device-side status reported failure"
    assert mailbox is None or mailbox.status() == 0, "mailbox wait timed out"

    # The checker leg: what the last timed step left in `out`, on every rank,
    # against the CPU oracle (the only use of oracle/ on this path).
    threads = max(1, host_threads() // world)
    checked, worst, ok = check_headline(
        values, table if world > 1 else seg, last[0], rank, world, threads)
    if world > 1:
        t = torch.tensor([float(checked), worst, 0.0 if ok else 1.0],
                         device=device, dtype=torch.float64)
        total = t.clone()
        dist.all_reduce(total, op=dist.ReduceOp.SUM)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        checked, worst, ok = int(total[0].item()), float(t[1].item()), \
            t[2].item() == 0.0
    parity = {"checked": True, "segments": checked, "max_rel_err": worst,
              "ok": ok, "tolerance": FP32_TOL,
              "how": "every output of the last timed step on every rank "
                     "against fp64 sums of the CPU oracle, |got - ref| <= "
                     "1e-5 * max(|ref|, sum |x|); a segment that straddles "
                     "ranks is checked on its owner against its own items "
                     "plus the following ranks' leading items"}

    # Dominant kernel alone, timed live with CUDA events between the two
    # launches of a call (rank 0's GPU).
    roofline = None
    if rank == 0:
        reduce_ms, part_ms = [], []
        for _ in range(min(max(args.steps, 3), 10)):
            _, p_ms, r_ms = mgpu.segreduce_profile(values, seg, op="plus",
                                                   init=0.0, out=out)
            part_ms.append(p_ms)
            reduce_ms.append(r_ms)
        kernel_ms = sum(reduce_ms) / len(reduce_ms)
        algorithmic = workloads.segreduce_bytes(COUNT, NUM_SEGMENTS, 4)
        peak, peak_kind = measured_peak()
        achieved = algorithmic / (kernel_ms * 1e-3) / 1e9
        roofline = {
            "bound": "hbm", "kernel": "segreduce_k",
            "achieved": achieved, "peak": peak, "unit": "GB/s",
            "frac": achieved / peak, "peak_source": "of " + peak_kind,
            "algorithmic_bytes": algorithmic,
            "traffic": algorithmic * TRAFFIC_PER_ALGORITHMIC_BYTE,
            "traffic_source": "one ncu capture of a 2^26-item case of this "
                              "workload, scaled by the units processed",
            "kernel_ms": kernel_ms,
            "partition_kernel_ms": sum(part_ms) / len(part_ms),
        }
    clocks = sampler.stop() if sampler else None

    # End to end through the host-buffer entry point of the C ABI.
    with near_gpu(local_rank) as placement:
        hv = values.cpu().pin_memory()
        hs = (table if world > 1 else seg).cpu().pin_memory()
        ho = torch.empty(hs.numel(), dtype=torch.float32).pin_memory()
        e2e_steps = max(2, min(args.steps, 5))
        for _ in range(2):
            mgpu.segreduce_host(hv, hs, op="plus", init=0.0, out=ho)
        if world > 1:
            dist.barrier()
        t0 = time.perf_counter()
        for _ in range(e2e_steps):
            mgpu.segreduce_host(hv, hs, op="plus", init=0.0, out=ho)
            if world > 1:
                # Boundary records cross through a 16-byte device tensor.
                rec = torch.from_numpy(sharded.pack_record_host(
                    int(ho[:1].view(torch.int32).item()) & 0xffffffff,
                    hs.numpy(), COUNT).view("int64").copy()).to(device)
                gathered = torch.empty(world * 2, dtype=torch.int64,
                                       device=device)
                dist.all_gather_into_tensor(gathered, rec)
                recs = gathered.cpu().numpy().view("uint64").reshape(world, 2)
                flags = [int(f) for f in recs[:, 1]]
                for k in sharded.fold_plan(flags, rank):
                    part = float(recs[k, :1].view("float32")[0])
                    ho[-1] = part if flags[rank] & sharded.LAST_EMPTY \
                        else ho[-1] + part
        e2e_s = (time.perf_counter() - t0) / e2e_steps
    if world > 1:
        t = torch.tensor([e2e_s], device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_s = float(t.item())
    e2e = {"value": world * COUNT / e2e_s / 1e9, "unit": UNIT,
           "h2d_bytes_per_step": hv.numel() * 4 + hs.numel() * 4,
           "d2h_bytes_per_step": ho.numel() * 4,
           "ms_per_step": e2e_s * 1e3, "steps": e2e_steps,
           "host_gbs_per_gpu": (hv.numel() * 4 + hs.numel() * 4
                                + ho.numel() * 4) / e2e_s / 1e9,
           "placement": placement.note,
           "api": "mgpu_b200_segreduce_host (pinned host buffers)",
           "note": "bound by the host link: every step moves the arrays "
                   "from host memory to the GPU; with N GPUs the N links "
                   "share the host's memory bandwidth"}
    del hv, hs, ho

    cpu = None
    if rank == 0 and world == 1:
        import oracle
        # A bounded sample: ~10 s of the host loop on the whole workload.
        cv, cs = cpu_workload(COUNT, NUM_SEGMENTS)
        cores = host_threads()
        cv = oracle.place_by_segments(cv, cs, cores)
        oracle.segreduce(cv, cs, op="plus", init=0.0, threads=cores)
        reps, spent = 0, 0.0
        while spent < 10.0 and reps < 100000:
            t0 = time.perf_counter()
            oracle.segreduce(cv, cs, op="plus", init=0.0, threads=cores)
            spent += time.perf_counter() - t0
            reps += 1
        cpu = {"value": cv.size * reps / spent / 1e9, "unit": UNIT,
               "cores": cores, "kind": "port",
               "sample": "%d repetitions (%.1f s) of the host loop of "
                         "tests/test_segreduce.cu:40-49 (C port, OpenMP over "
                         "segments) on the whole %d-item / %d-segment "
                         "workload" % (reps, spent, cv.size, cs.size)}
        del cv, cs

    # Secondary configurations (not part of `value`).
    secondary = []
    if not args.no_secondary:
        side_steps = max(3, min(args.steps, 10))
        if mailbox is not None:
            mailbox.close()
            mailbox = None
        if world == 1:
            secondary += single_gpu_legs(args, device, side_steps,
                                         (values, seg))
        else:
            secondary += config2_strong_leg(args, rank, world, device,
                                            side_steps)
        del values, seg, table, out, records, shard_out
        last[0] = None
        torch.cuda.empty_cache()
        if 8 % world == 0:
            secondary += config5_legs(args, rank, world, device, side_steps)

    if rank == 0:
        launches_per_step = 4 if world > 1 and (
            args.unfused or args.exchange != "p2p") else 2
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3),
            "ms_per_step": ms_per_step, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32",
            "data": "synthetic", "config": workload_config(world, args.exchange),
            "hbm_gbs_per_gpu": workloads.segreduce_bytes(
                COUNT, NUM_SEGMENTS, 4) / (ms_per_step * 1e-3) / 1e9,
            "roofline": roofline, "cpu_baseline": cpu, "e2e": e2e,
            "parity": parity,
            "gpu_launches": launches_per_step * args.steps,
            "clocks": clocks, "secondary": secondary,
        }
        emit(line)
    if mailbox is not None:
        mailbox.close()
    if world > 1:
        dist.destroy_process_group()
    all_ok = ok and all(row.get("parity", {}).get("ok", True)
                        for row in secondary)
    if not all_ok:
        print("bench: outputs differ from the oracle", file=sys.stderr)
        sys.exit(1)


def run_other_config(args, rank, world, local_rank):
    """One secondary configuration alone (--config), e.g. as the small case
    of a profiler capture: device-resident throughput and algorithmic HBM
    GB/s, CUDA events, max over ranks."""
    import torch
    import torch.distributed as dist
    import moderngpu_b200 as mgpu
    from moderngpu_b200 import workloads

    mgpu.load_library()
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    cfg = args.config
    peak, peak_kind = measured_peak()
    results = []
    if cfg == "c5":
        results = config5_legs(args, rank, world, device, args.steps)
    elif cfg == "c2strong":
        results = config2_strong_leg(args, rank, world, device, args.steps)
    elif cfg == "single":
        values, seg = workloads.config2(seed=1, count=COUNT,
                                        num_segments=NUM_SEGMENTS,
                                        device=device)
        results = single_gpu_legs(args, device, args.steps, (values, seg))
    else:
        steps = {}
        if cfg == "c1":
            v, s = workloads.config1(seed=0)
            v, s = torch.from_numpy(v).to(device), torch.from_numpy(s).to(device)
            out = torch.empty(s.numel(), dtype=v.dtype, device=device)
            steps["int32 plus"] = (
                lambda: mgpu.segreduce(v, s, init=0, out=out), v.numel(),
                workloads.segreduce_bytes(v.numel(), s.numel(), 4))
        elif cfg == "c3":
            m, c, x, r = workloads.config3(
                seed=2, device=device, rows=1 << (22 if args.small else 24))
            y = torch.empty(r.numel(), dtype=m.dtype, device=device)
            steps["spmv fp32 rows=%d nnz=%d" % (r.numel(), m.numel())] = (
                lambda: mgpu.spmv(m, c, x, r, out=y), m.numel(),
                workloads.spmv_bytes(m.numel(), r.numel(), x.numel(), 4))
        elif cfg == "c4":
            count = COUNT
            s = workloads.config4(seed=3, device=device, count=count,
                                  num_segments=NUM_SEGMENTS // 2)
            steps["lbs seg+rank"] = (
                lambda: mgpu.transform_lbs(count, s), count,
                workloads.lbs_bytes(count, s.numel()))
            steps["lbs seg only"] = (
                lambda: mgpu.load_balance_search(count, s), count,
                workloads.lbs_bytes(count, s.numel(), False))
        elif cfg == "scan":
            x = torch.randint(0, 64, (COUNT,), device=device, dtype=torch.int32)
            out = torch.empty_like(x)
            steps["exclusive scan int32, %d items" % COUNT] = (
                lambda: mgpu.scan(x, out=out), x.numel(), 8 * x.numel())
        elif cfg == "lbs_segreduce":
            values, seg, _ = make_shard(0, device)
            g = torch.Generator(device=device).manual_seed(11)
            weights = torch.rand(seg.numel(), device=device, generator=g)
            out = torch.empty(seg.numel(), dtype=torch.float32, device=device)
            steps["lbs_segreduce fp32 weighted sums, config 2 shape"] = (
                lambda: mgpu.lbs_segreduce_weighted(values, seg, weights,
                                                    out=out),
                values.numel(),
                workloads.segreduce_bytes(values.numel(), seg.numel(), 4)
                + 4 * seg.numel())
        elif cfg == "uniform":
            values, _, _ = make_shard(0, device)
            length = args.length
            n = values.numel() // length
            useg = (torch.arange(n, device=device, dtype=torch.int64) * length
                    ).to(torch.int32)
            uout = torch.empty(n, dtype=torch.float32, device=device)
            steps["segreduce fp32, every segment exactly %d items" % length] = (
                lambda: mgpu.segreduce(values, useg, init=0.0, out=uout),
                values.numel(),
                workloads.segreduce_bytes(values.numel(), n, 4))
        elif cfg == "search":
            n_keys = COUNT // 2
            g = torch.Generator(device=device).manual_seed(5)
            needles = torch.sort(torch.randint(
                0, 1 << 30, (n_keys,), device=device, dtype=torch.int32,
                generator=g))[0]
            hay = torch.sort(torch.randint(
                0, 1 << 30, (n_keys,), device=device, dtype=torch.int32,
                generator=g))[0]
            found = torch.empty(n_keys, dtype=torch.int32, device=device)
            steps["sorted_search lower bound, %d + %d int32 keys"
                  % (n_keys, n_keys)] = (
                lambda: mgpu.sorted_search(needles, hay, out=found), n_keys,
                12 * n_keys)
        for name, (fn, units, nbytes) in steps.items():
            ms = time_steps(fn, args.steps, args.warmup, world, device)
            results.append(result_row(name, ms, units, nbytes, world, peak,
                                      peak_kind))
        assert mgpu.workspace_status() == 0
    if rank == 0:
        emit({"config": cfg, "n_gpus": world, "steps": args.steps,
              "note": "includes every launch of a step (partitioner + "
                      "kernel, plus the boundary-record kernels of the "
                      "multi-GPU layer)",
              "results": results})
    if world > 1:
        dist.destroy_process_group()


def main():
    # NCCL announces its version on stdout at this debug level, which would
    # put a second line next to the JSON line.
    if os.environ.get("NCCL_DEBUG", "").upper() == "VERSION":
        os.environ["NCCL_DEBUG"] = "WARN"
    # Whatever else a library writes to stdout goes to stderr instead; the
    # JSON line is written to the original stdout by emit().
    global _RESULT_FD
    sys.stdout.flush()
    _RESULT_FD = os.dup(1)
    os.dup2(2, 1)
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=100)
    parser.add_argument("--warmup", type=int, default=3)
    parser.add_argument("--small", action="store_true",
                        help="2^26 items / 2^21 segments per GPU: a case "
                             "small enough for a full ncu capture")
    parser.add_argument("--config", default="c2",
                        choices=["c1", "c2", "c3", "c4", "c5", "c2strong",
                                 "single", "scan", "search", "lbs_segreduce",
                                 "uniform"],
                        help="c2 (default) is the headline line with its "
                             "secondary results; the others run one "
                             "secondary configuration alone")
    parser.add_argument("--length", type=int, default=32,
                        help="--config uniform: the segment length")
    parser.add_argument("--no-secondary", action="store_true",
                        help="headline only: skip the secondary "
                             "configurations")
    parser.add_argument("--exchange", default="p2p", choices=["p2p", "nccl"],
                        help="multi-GPU boundary records: peer-to-peer "
                             "stores into mailboxes (default) or an NCCL "
                             "all-gather")
    parser.add_argument("--no-side-stream", action="store_true",
                        help="multi-GPU, p2p: post the boundary records on "
                             "the main stream, in front of the reduction, "
                             "instead of on a side stream beside it")
    parser.add_argument("--unfused", action="store_true",
                        help="multi-GPU, p2p: post and collect as launches "
                             "of their own (four per step) instead of inside "
                             "the partitioner's and the reduction's")
    parser.add_argument("--impl", default="ours",
                        choices=["ours", "reference", "reference-cuda"])
    args = parser.parse_args()
    if args.small:
        global COUNT, NUM_SEGMENTS
        COUNT, NUM_SEGMENTS = 1 << 26, 1 << 21
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference_cpu(args, rank, world)
    elif args.impl == "reference-cuda":
        run_reference_cuda(args, rank, world)
    elif args.config != "c2":
        run_other_config(args, rank, world, local_rank)
    else:
        run_ours(args, rank, world, local_rank)


if __name__ == "__main__":
    main()
