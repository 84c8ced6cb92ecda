"""Multi-GPU segmented reduction on real GPUs (needs at least 2): one process
per GPU over NCCL, shard-local reduction by the library's kernels, boundary
records all-gathered, owner-side fold by mgpu_b200_shard_fold. The assembled
result must equal the oracle's reduction of the whole array."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from moderngpu_b200 import sharded

pytestmark = pytest.mark.gpu


def free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def make_problem(kind, dtype):
    rng = np.random.default_rng(77)
    count = 4_000_000
    if kind == "lognormal":      # config-5 shape: many straddling segments
        lengths = np.floor(np.exp(3 + 1.5 * rng.standard_normal(80_000))).astype(np.int64)
        seg = np.minimum(np.cumsum(lengths) - lengths, count)
    elif kind == "few_long":
        seg = np.array([0, 10, 3_900_000], dtype=np.int64)
    else:
        seg = np.array([0], dtype=np.int64)
    if np.issubdtype(dtype, np.integer):
        values = rng.integers(-1000, 1000, size=count).astype(dtype)
    else:
        values = ((rng.random(count) * 2 - 1) * 1e6).astype(dtype)
    return values, seg


def worker(rank, world, port, kind, dtype_name, op, queue):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world,
                            device_id=torch.device("cuda", rank))
    try:
        dtype = np.dtype(dtype_name).type
        values, seg = make_problem(kind, dtype)
        begin, end, first, table = sharded.shard_table(seg, values.size, rank, world)
        out = sharded.sharded_segreduce(
            torch.from_numpy(values[begin:end].copy()).cuda(),
            torch.from_numpy(table).cuda(), op=op, init=-7)
        torch.cuda.synchronize()
        pieces = [None] * world
        dist.all_gather_object(pieces, (first, out.cpu().numpy()[1:].tolist()))
        if rank == 0:
            queue.put(pieces)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("kind,dtype,op", [
    ("lognormal", "float64", "max"), ("lognormal", "int64", "plus"),
    ("few_long", "int32", "plus"), ("one", "float64", "min"),
    ("lognormal", "float64", "plus"),
])
def test_sharded_matches_oracle(oracle, kind, dtype, op):
    world = min(torch.cuda.device_count(), 4)
    if world < 2:
        pytest.skip("needs at least two GPUs")
    ctx = mp.get_context("spawn")
    queue = ctx.Queue()
    port = free_port()
    procs = [ctx.Process(target=worker, args=(r, world, port, kind, dtype, op, queue))
             for r in range(world)]
    for p in procs:
        p.start()
    pieces = queue.get(timeout=300)
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    values, seg = make_problem(kind, np.dtype(dtype).type)
    got = np.zeros(seg.size, dtype=np.float64)
    for first, vals in pieces:
        got[first:first + len(vals)] = vals
    seg32 = seg.astype(np.int32)
    if op == "plus" and dtype == "float64":
        want, mags = oracle.segsum_wide(values, seg32, init=-7)
        assert np.all(np.abs(got - want) <= 1e-12 * np.maximum(np.abs(want), mags))
    else:
        want = oracle.segreduce(values, seg32, op=op, init=-7).astype(np.float64)
        assert np.array_equal(got, want)


@pytest.mark.parametrize("kind,dtype,op", [
    ("lognormal", "float64", "max"), ("few_long", "int64", "plus"),
    ("one", "int32", "plus"),
])
def test_several_shards_on_one_gpu(mgpu, oracle, kind, dtype, op):
    """The array cut into 5 shards that one GPU reduces one after the other
    (how an array beyond the 2^31 index limit of a single call is handled);
    the chain of boundary records is folded exactly as across GPUs."""
    values, seg = make_problem(kind, np.dtype(dtype).type)
    pieces = 5
    shards, firsts = [], []
    for r in range(pieces):
        begin, end, first, table = sharded.shard_table(seg, values.size, r, pieces)
        shards.append((torch.from_numpy(values[begin:end].copy()).cuda(),
                       torch.from_numpy(table).cuda()))
        firsts.append(first)
    outs = sharded.sharded_segreduce_multi(shards, op=op, init=-7)
    got = np.zeros(seg.size, dtype=np.float64)
    for first, out in zip(firsts, outs):
        vals = out.cpu().numpy()[1:]
        got[first:first + vals.size] = vals
    want = oracle.segreduce(values, seg.astype(np.int32), op=op, init=-7)
    assert np.array_equal(got, want.astype(np.float64))
