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
timed on the host cores.

--impl reference times the reference's host loop (tests/test_segreduce.cu:
40-49, restated in oracle/oracle.c) on all host cores; --impl reference-cuda
times the reference's own CUDA build (oracle/_ref/libmgpu_ref.so) on the GPU.
"""
import argparse
import ctypes
import json
import os
import statistics
import subprocess
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
# one ncu capture of a 2^26-item case of the same workload, divided by that
# case's algorithmic bytes; DRAM traffic grows in proportion to the units processed.
TRAFFIC_PER_ALGORITHMIC_BYTE = 0.9988


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
    NVML polled every few milliseconds from a thread (read-only queries), or
    nvidia-smi when the NVML binding is missing."""
    REASONS = {
        "hw_slowdown": 0x8, "hw_thermal_slowdown": 0x40,
        "sw_thermal_slowdown": 0x20, "sw_power_cap": 0x4,
    }

    def __init__(self, uuid, index):
        self.uuid, self.index = uuid, index
        self.samples = []          # (time, sm_mhz, reasons_mask)
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
                        self.samples.append((time.perf_counter(), float(mhz),
                                             int(mask)))
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
        return {"sm_mhz": statistics.median(mhz) if mhz else None,
                "sm_max_mhz": self.max_mhz,
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


def cpu_sample(count=1 << 26, num_segments=1 << 21, seed=1):
    """A bounded sample of the workload for the CPU arm, generated on the host
    with the same length and value distributions."""
    import torch
    from moderngpu_b200 import workloads
    values, seg = workloads.config2(seed=seed, count=count,
                                    num_segments=num_segments, device="cpu")
    return values.numpy(), seg.numpy()


def time_cpu(values, seg, budget_s, threads):
    import oracle
    oracle.segreduce(values[:1 << 20], seg[:1 << 10], threads=threads)
    reps, spent = 0, 0.0
    while spent < budget_s and reps < 100000:
        t0 = time.perf_counter()
        oracle.segreduce(values, seg, op="plus", init=0.0, threads=threads)
        spent += time.perf_counter() - t0
        reps += 1
    return values.size * reps / spent / 1e9, reps, spent


def run_reference_cpu(args, rank, world):
    if rank != 0:
        return
    import oracle
    values, seg = cpu_sample()
    threads = host_threads()
    oracle.segreduce(values, seg, threads=threads)        # warm
    for _ in range(max(args.warmup - 1, 0)):
        oracle.segreduce(values, seg, threads=threads)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        oracle.segreduce(values, seg, op="plus", init=0.0, threads=threads)
    dt = time.perf_counter() - t0
    value = values.size * args.steps / dt / 1e9
    sample = ("each step: host loop of tests/test_segreduce.cu:40-49 (C port, "
              "OpenMP over segments) on a %d-item / %d-segment sample of the "
              "workload" % (values.size, seg.size))
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT,
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": dt / args.steps * 1e3, "higher_is_better": True,
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


def run_reference_cuda(args, rank, world):
    if rank != 0:
        return
    import torch
    from moderngpu_b200 import workloads
    path = os.path.join(ROOT, "oracle", "_ref", "libmgpu_ref.so")
    if not os.path.exists(path):
        emit({"impl": "reference-cuda", "unavailable":
              "oracle/_ref/libmgpu_ref.so was not built"})
        return
    ref = ctypes.CDLL(path)
    torch.cuda.set_device(0)
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

    results = {}
    for pooled in (0, 1):
        for _ in range(max(args.warmup, 3)):
            call(pooled, 1)
        t0 = time.perf_counter()
        for _ in range(args.steps):
            call(pooled, 0)
        torch.cuda.synchronize()
        results[pooled] = (time.perf_counter() - t0) / args.steps
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
        "value": COUNT / results[0] / 1e9, "unit": UNIT, "n_gpus": 1,
        "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": results[0] * 1e3, "higher_is_better": True,
        "dtype": "f32", "data": "synthetic", "config": workload_config(1),
        "note": "unmodified moderngpu headers compiled for sm_100a; value = "
                "stock standard_context_t (cudaMalloc/cudaFree per call), "
                "host-clock timed; pooled_context = same kernels with "
                "recycled temporaries",
        "pooled_context": {"value": COUNT / results[1] / 1e9, "unit": UNIT,
                           "ms_per_step": results[1] * 1e3},
        "e2e": {"value": COUNT / e2e_t / 1e9, "unit": UNIT,
                "h2d_bytes_per_step": COUNT * 4 + NUM_SEGMENTS * 4,
                "d2h_bytes_per_step": NUM_SEGMENTS * 4},
    }
    emit(line)


def make_shard(rank, device):
    """This rank's shard: values and shard-local start table (entry 0 is the
    virtual start that stands for the segment carried in from the left)."""
    import torch
    from moderngpu_b200 import workloads
    values, seg = workloads.config2(seed=1 + rank, count=COUNT,
                                    num_segments=NUM_SEGMENTS, device=device)
    if rank > 0:
        # The first real segment starts a little into the shard: the leading
        # items continue the previous rank's last segment.
        lead = 17 + rank
        seg = torch.clamp(seg + lead, max=COUNT)
    table = torch.cat([torch.zeros(1, dtype=torch.int32, device=device), seg])
    return values, seg, table


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
            mailbox = sharded.Mailbox(side_stream=not args.no_side_stream)
        except sharded.MailboxError as e:
            # All ranks fail together; the records then travel by all-gather.
            print("bench: %s; using --exchange nccl" % e, file=sys.stderr)
            args.exchange = "nccl"

    def step():
        if world == 1:
            mgpu.segreduce(values, seg, op="plus", init=0.0, out=out)
        elif mailbox is not None:
            sharded.sharded_segreduce(values, table, op="plus", init=0.0,
                                      mailbox=mailbox)
        else:
            sharded.sharded_segreduce(values, table, op="plus", init=0.0,
                                      records=records)

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
            "kernel_ms": kernel_ms,
            "partition_kernel_ms": sum(part_ms) / len(part_ms),
        }
    clocks = sampler.stop() if sampler else None

    # End to end through the host-buffer entry point of the C ABI.
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
            gathered = torch.empty(world * 2, dtype=torch.int64, device=device)
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
           "api": "mgpu_b200_segreduce_host (pinned host buffers)"}

    if rank == 0:
        cpu = None
        if world == 1:
            import oracle
            cv, cs = cpu_sample()
            threads = host_threads()
            cpu_value, reps, spent = time_cpu(cv, cs, 10.0, threads)
            cpu = {"value": cpu_value, "unit": UNIT, "cores": threads,
                   "kind": "port",
                   "sample": "%d repetitions (%.1f s) of the host loop of "
                             "tests/test_segreduce.cu:40-49 (C port, OpenMP "
                             "over segments) on a %d-item / %d-segment sample "
                             "of the workload" % (reps, spent, cv.size, cs.size)}
        launches_per_step = 2 if world == 1 else 4
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3),
            "ms_per_step": ms_per_step, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32",
            "data": "synthetic", "config": workload_config(world, args.exchange),
            "hbm_gbs_per_gpu": workloads.segreduce_bytes(
                COUNT, NUM_SEGMENTS, 4) / (ms_per_step * 1e-3) / 1e9,
            "roofline": roofline, "cpu_baseline": cpu, "e2e": e2e,
            "gpu_launches": launches_per_step * args.steps,
            "clocks": clocks,
        }
        emit(line)
    if mailbox is not None:
        mailbox.close()
    if world > 1:
        dist.destroy_process_group()


def run_other_config(args, rank, world, local_rank):
    """Secondary lines for the other benchmark configurations (--config):
    device-resident throughput and algorithmic HBM GB/s, CUDA events, max
    over ranks. c1: int32 plus 1,048,576 items / 10,000 segments; c3: CSR spmv
    fp32, 16,777,216 rows; c4: load-balancing search with ranks, 268,435,456
    items / 4,194,304 segments; c5: fp64 max- and plus-segreduce over 2^32 items of
    log-normal segments held as 8 shards, 8/N per GPU (strong scaling)."""
    import torch
    import torch.distributed as dist
    import moderngpu_b200 as mgpu
    from moderngpu_b200 import sharded, workloads

    mgpu.load_library()
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    cfg = args.config
    steps = {}
    if cfg == "c1":
        v, s = workloads.config1(seed=0)
        v, s = torch.from_numpy(v).to(device), torch.from_numpy(s).to(device)
        out = torch.empty(s.numel(), dtype=v.dtype, device=device)
        steps["int32 plus"] = (lambda: mgpu.segreduce(v, s, init=0, out=out),
                               v.numel(),
                               workloads.segreduce_bytes(v.numel(), s.numel(), 4))
    elif cfg == "c3":
        m, c, x, r = workloads.config3(seed=2, device=device)
        y = torch.empty(r.numel(), dtype=m.dtype, device=device)
        steps["spmv fp32 nnz=%d" % m.numel()] = (
            lambda: mgpu.spmv(m, c, x, r, out=y), m.numel(),
            workloads.spmv_bytes(m.numel(), r.numel(), x.numel(), 4))
        # The same with the x vector pinned in the L2 (mgpu_b200_l2_pin); the
        # pin is taken before this case's warm-up and dropped after the run.
        steps["spmv fp32, x pinned in L2"] = (
            lambda: mgpu.spmv(m, c, x, r, out=y), m.numel(),
            workloads.spmv_bytes(m.numel(), r.numel(), x.numel(), 4))
    elif cfg == "c4":
        count = 1 << 28
        s = workloads.config4(seed=3, device=device)
        steps["lbs seg+rank"] = (lambda: mgpu.transform_lbs(count, s), count,
                                 workloads.lbs_bytes(count, s.numel()))
        steps["lbs seg only"] = (lambda: mgpu.load_balance_search(count, s),
                                 count,
                                 workloads.lbs_bytes(count, s.numel(), False))
    elif cfg == "scan":
        n_scan = 1 << (26 if args.small else 28)
        x = torch.randint(0, 64, (n_scan,), device=device, dtype=torch.int32)
        out = torch.empty_like(x)
        steps["exclusive scan int32, %d items" % n_scan] = (
            lambda: mgpu.scan(x, out=out), x.numel(), 8 * x.numel())
    elif cfg == "lbs_segreduce":
        # Config 2's items and segments through lbs_segreduce: the functor
        # reads values[index] and multiplies by a weight cached per segment.
        values, seg, _ = make_shard(0, device)
        g = torch.Generator(device=device).manual_seed(11)
        weights = torch.rand(seg.numel(), device=device, generator=g)
        out = torch.empty(seg.numel(), dtype=torch.float32, device=device)
        steps["lbs_segreduce fp32 weighted sums, config 2 shape"] = (
            lambda: mgpu.lbs_segreduce_weighted(values, seg, weights, out=out),
            values.numel(),
            workloads.segreduce_bytes(values.numel(), seg.numel(), 4)
            + 4 * seg.numel())
    elif cfg == "search":
        # 2^27 sorted int32 needles into a sorted haystack of 2^27 keys.
        n_keys = 1 << (24 if args.small else 27)
        g = torch.Generator(device=device).manual_seed(5)
        needles = torch.sort(torch.randint(0, 1 << 30, (n_keys,), device=device,
                                           dtype=torch.int32, generator=g))[0]
        hay = torch.sort(torch.randint(0, 1 << 30, (n_keys,), device=device,
                                       dtype=torch.int32, generator=g))[0]
        found = torch.empty(n_keys, dtype=torch.int32, device=device)
        steps["sorted_search lower bound, %d + %d int32 keys" % (n_keys, n_keys)] = (
            lambda: mgpu.sorted_search(needles, hay, out=found), n_keys,
            12 * n_keys)
    elif cfg == "c5":
        # The whole 2^32-item array, always as 8 shards of 2^29 items; each of
        # the N ranks holds 8/N consecutive shards (strong scaling).
        total_shards, count = 8, 1 << 29
        per_rank = total_shards // world
        shards, nbytes = [], 0
        for j in range(per_rank):
            g = rank * per_rank + j
            v, starts = workloads.config5_shard(4, g, count, device=device)
            table = torch.cat([torch.zeros(1, dtype=torch.int32,
                                           device=device), starts])
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
        for op, init in (("max", -1e300), ("plus", 0.0)):
            steps["fp64 %s, 2^32 items in 8 shards" % op] = (
                lambda op=op, init=init: sharded.sharded_segreduce_multi(
                    shards, op=op, init=init, outs=outs, mailbox=box),
                per_rank * count, nbytes)
    peak, peak_kind = measured_peak()
    results = []
    for name, (fn, units, nbytes) in steps.items():
        if "pinned" in name:
            mgpu.l2_pin(x)
        for _ in range(max(args.warmup, 3)):
            fn()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        a = torch.cuda.Event(enable_timing=True)
        b = torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(args.steps):
            fn()
        b.record()
        torch.cuda.synchronize()
        ms = a.elapsed_time(b) / args.steps
        if world > 1:
            t = torch.tensor([ms], device=device)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        if "pinned" in name:
            mgpu.l2_unpin()
        gbs = nbytes / (ms * 1e-3) / 1e9
        results.append({"case": name, "ms_per_step": ms,
                        "gitems_per_s": world * units / (ms * 1e-3) / 1e9,
                        "algorithmic_bytes_per_gpu": nbytes,
                        "hbm_gbs_per_gpu": gbs,
                        "frac_of_%s_peak" % peak_kind: gbs / peak})
    assert mgpu.workspace_status() == 0
    if cfg == "c5" and box is not None:
        assert box.status() == 0
        box.close()
    if rank == 0:
        emit({"config": cfg, "n_gpus": world, "steps": args.steps,
              "note": "includes every launch of a step (partitioner + "
                      "kernel, plus the boundary-record post / collect "
                      "kernels of the multi-GPU layer)",
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
    parser.add_argument("--steps", type=int, default=200)
    parser.add_argument("--warmup", type=int, default=3)
    parser.add_argument("--small", action="store_true",
                        help="2^26 items / 2^21 segments per GPU: a case "
                             "small enough for a full ncu capture")
    parser.add_argument("--config", default="c2",
                        choices=["c1", "c2", "c3", "c4", "c5", "scan", "search",
                                 "lbs_segreduce"],
                        help="c2 (default) is the headline line; the others "
                             "print a shorter secondary line")
    parser.add_argument("--exchange", default="p2p", choices=["p2p", "nccl"],
                        help="multi-GPU boundary records: peer-to-peer "
                             "stores into mailboxes (default) or an NCCL "
                             "all-gather")
    parser.add_argument("--no-side-stream", action="store_true",
                        help="multi-GPU, p2p: post the boundary records on "
                             "the main stream, in front of the reduction, "
                             "instead of on a side stream beside it")
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
