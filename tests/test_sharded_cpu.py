"""Host logic of the multi-GPU layer on CPU ranks (gloo, world_size 2 and 3):
shard tables, boundary records, ownership and fold order. The per-shard
reduction is done by the CPU oracle inside this test (the library itself has
no CPU path); on GPUs it is the library's kernel (tests/test_sharded_gpu.py)."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from moderngpu_b200 import sharded


def free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def make_problem(kind, dtype):
    rng = np.random.default_rng(101)
    count = 30_000
    if kind == "many_short":
        seg = np.zeros(2500, dtype=np.int64)
        seg[1:] = np.sort(rng.integers(0, count + 1, size=seg.size - 1))
    elif kind == "few_long":         # segments far longer than a shard
        seg = np.array([0, 100, 29_000], dtype=np.int64)
    elif kind == "one":              # a single segment spanning every shard
        seg = np.array([0], dtype=np.int64)
    elif kind == "aligned":          # starts exactly on shard boundaries
        seg = np.array([0, 10_000, 10_000, 15_000, 20_000, 30_000, 30_000],
                       dtype=np.int64)
    else:
        raise ValueError(kind)
    if np.issubdtype(dtype, np.integer):
        values = rng.integers(-1000, 1000, size=count).astype(dtype)
    else:
        values = rng.integers(-1000, 1000, size=count).astype(dtype) / 8
    return values, seg


def worker(rank, world, port, kind, dtype_name, op, result_queue):
    import oracle
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        dtype = np.dtype(dtype_name).type
        values, seg = make_problem(kind, dtype)
        begin, end, first, table = sharded.shard_table(seg, values.size, rank,
                                                       world)

        # The per-shard reduction is the oracle's here (a stand-in that lives
        # in this test only); everything after it is the host logic under
        # test: record flags, exchange, who folds what and in which order.
        local = values[begin:end]
        out = oracle.segreduce(local, table, op=op, init=-7)
        bits = np.zeros(1, dtype=np.uint64)
        bits.view(np.uint8)[:out.itemsize] = out[:1].view(np.uint8)
        rec = sharded.pack_record_host(bits[0], table, local.size)
        gathered = [torch.zeros(2, dtype=torch.int64) for _ in range(world)]
        dist.all_gather(gathered, torch.from_numpy(rec.view(np.int64).copy()))
        recs = np.stack([g.numpy().view(np.uint64) for g in gathered])
        flags = [int(f) for f in recs[:, 1]]
        fold = {"plus": lambda a, b: a + b, "max": max, "min": min}[op]
        acc = None
        for k in sharded.fold_plan(flags, rank):
            val = recs[k, :1].view(np.uint8)[:out.itemsize].view(out.dtype)[0]
            acc = val if acc is None else fold(acc, val)
        if acc is not None:
            out[-1] = acc if flags[rank] & sharded.LAST_EMPTY \
                else fold(out[-1], acc)
        pieces = [None] * world
        dist.all_gather_object(pieces, (first, out[1:].tolist()))
        if rank == 0:
            got = np.full(seg.size, -12345, dtype=np.float64)
            for f, vals in pieces:
                got[f:f + len(vals)] = vals
            want = oracle.segreduce(values, seg.astype(np.int32), op=op,
                                    init=-7).astype(np.float64)
            result_queue.put((got.tolist(), want.tolist()))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
@pytest.mark.parametrize("kind,dtype,op", [
    ("many_short", "int32", "plus"),
    ("few_long", "int64", "plus"),
    ("one", "int32", "max"),
    ("aligned", "float64", "plus"),
    ("few_long", "float64", "min"),
])
def test_sharded_equals_global(world, kind, dtype, op):
    ctx = mp.get_context("spawn")
    queue = ctx.Queue()
    port = free_port()
    procs = [ctx.Process(target=worker,
                         args=(r, world, port, kind, dtype, op, queue))
             for r in range(world)]
    for p in procs:
        p.start()
    got, want = queue.get(timeout=120)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert got == want


def test_shard_table_covers_every_segment_once():
    rng = np.random.default_rng(5)
    count = 1000
    seg = np.zeros(300, dtype=np.int64)
    seg[1:] = np.sort(rng.integers(0, count + 1, size=seg.size - 1))
    seg[-3:] = count                      # trailing empty segments
    for world in (1, 2, 4, 8):
        seen = []
        for rank in range(world):
            begin, end, first, table = sharded.shard_table(seg, count, rank, world)
            assert table[0] == 0
            local = table[1:].astype(np.int64) + begin
            assert np.array_equal(local, seg[first:first + local.size])
            seen.extend(range(first, first + local.size))
        assert seen == list(range(seg.size))


def test_fold_plan():
    P, S = sharded.HAS_PARTIAL, sharded.HAS_START
    # rank 0 owns a segment that runs through ranks 1 and 2 and ends in 3.
    flags = [S, P, P, P | S, S]
    assert sharded.fold_plan(flags, 0) == [1, 2, 3]
    assert sharded.fold_plan(flags, 1) == []
    assert sharded.fold_plan(flags, 3) == []       # rank 4 has no partial
    assert sharded.fold_plan([S, S | P, P], 1) == [2]
