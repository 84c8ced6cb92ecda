"""Multi-GPU segmented reduction on real GPUs (needs at least 2): one process
per GPU over NCCL, shard-local reduction by the library's kernels, boundary
records (from the shard's leading items, exchanged while the reduction runs;
or from the reduction's first output) all-gathered, owner-side fold by
mgpu_b200_shard_fold. The assembled
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


def worker(rank, world, port, kind, dtype_name, op, overlap, queue):
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
        v = torch.from_numpy(values[begin:end].copy()).cuda()
        t = torch.from_numpy(table).cuda()
        if overlap in ("mailbox", "mailbox4"):
            # Peer-to-peer records, no collective in the data path; 70 steps
            # so that the 64-slot ring wraps and the acks are exercised.
            # "mailbox": the fused step (two launches); "mailbox4": post,
            # reduction and collect as launches of their own.
            box = sharded.Mailbox(fused=overlap == "mailbox")
            for _ in range(70):
                out = sharded.sharded_segreduce(v, t, op=op, init=-7, mailbox=box)
            assert box.status() == 0
            box.close()
        else:
            out = sharded.sharded_segreduce(v, t, op=op, init=-7, overlap=overlap)
        torch.cuda.synchronize()
        pieces = [None] * world
        dist.all_gather_object(pieces, (first, out.cpu().numpy()[1:].tolist()))
        if rank == 0:
            queue.put(pieces)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("kind,dtype,op,overlap", [
    ("lognormal", "float64", "max", True), ("lognormal", "int64", "plus", True),
    ("few_long", "int32", "plus", True), ("one", "float64", "min", True),
    ("lognormal", "float64", "plus", True), ("lognormal", "int64", "plus", False),
    ("few_long", "int32", "plus", False),
    ("lognormal", "float64", "max", "mailbox"), ("lognormal", "int64", "plus", "mailbox"),
    ("few_long", "int32", "plus", "mailbox"), ("one", "float64", "min", "mailbox"),
    ("lognormal", "float64", "plus", "mailbox"),
    ("lognormal", "float64", "max", "mailbox4"), ("few_long", "int32", "plus", "mailbox4"),
    ("one", "float64", "min", "mailbox4"),
])
def test_sharded_matches_oracle(oracle, kind, dtype, op, overlap):
    world = min(torch.cuda.device_count(), 4)
    if world < 2:
        pytest.skip("needs at least two GPUs")
    ctx = mp.get_context("spawn")
    queue = ctx.Queue()
    port = free_port()
    procs = [ctx.Process(target=worker, args=(r, world, port, kind, dtype, op, overlap, queue))
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


@pytest.mark.parametrize("overlap", [True, False, "mailbox", "mailbox4"])
@pytest.mark.parametrize("kind,dtype,op", [
    ("lognormal", "float64", "max"), ("few_long", "int64", "plus"),
    ("one", "int32", "plus"),
])
def test_several_shards_on_one_gpu(mgpu, oracle, kind, dtype, op, overlap):
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
    if overlap in ("mailbox", "mailbox4"):
        box = sharded.Mailbox(shards_per_gpu=pieces, fused=overlap == "mailbox")
        for _ in range(3):
            outs = sharded.sharded_segreduce_multi(shards, op=op, init=-7,
                                                   mailbox=box)
        assert box.status() == 0
        box.close()
    else:
        outs = sharded.sharded_segreduce_multi(shards, op=op, init=-7,
                                               overlap=overlap)
    got = np.zeros(seg.size, dtype=np.float64)
    for first, out in zip(firsts, outs):
        vals = out.cpu().numpy()[1:]
        got[first:first + vals.size] = vals
    want = oracle.segreduce(values, seg.astype(np.int32), op=op, init=-7)
    assert np.array_equal(got, want.astype(np.float64))


@pytest.mark.parametrize("dtype,op", [("int32", "plus"), ("int64", "min"),
                                      ("float32", "max"), ("float64", "min")])
@pytest.mark.parametrize("lead", [0, 1, 63, 64, 65, 1000, 8192, 8193, 300_001, 1_000_000])
def test_lead_record_equals_pack_record(mgpu, dtype, op, lead):
    """mgpu_b200_shard_lead (from the items) and mgpu_b200_shard_pack (from the
    reduction's first output) write the same record; called twice to check
    that the scratch is left ready."""
    import ctypes
    from moderngpu_b200 import binding
    lib = binding.load_library()
    rng = np.random.default_rng(lead + 5)
    count = 1_000_000
    values = rng.integers(-10**6, 10**6, size=count).astype(dtype)
    if lead < count:
        table = np.array([0, lead, min(lead + 17, count), count], dtype=np.int32)
    else:
        table = np.array([0], dtype=np.int32)
    v = torch.from_numpy(values).cuda()
    t = torch.from_numpy(table).cuda()
    out = mgpu.segreduce(v, t, op=op, init=3)
    recs = torch.zeros(3, 2, dtype=torch.int64, device="cuda")
    stream = binding._stream(v.device)
    code = binding._DTYPES[v.dtype]
    binding._check(lib.mgpu_b200_shard_pack(
        code, out.data_ptr(), t.data_ptr(), t.numel(), count,
        recs[0].data_ptr(), stream))
    for k in (1, 2):
        binding._check(lib.mgpu_b200_shard_lead(
            code, binding._OPS[op], v.data_ptr(), count, t.data_ptr(),
            t.numel(), recs[k].data_ptr(),
            sharded.lead_scratch(v.device).data_ptr(), stream))
    got = recs.cpu().numpy()
    assert got[0, 1] == got[1, 1] == got[2, 1]            # flags
    if lead > 0:
        assert got[0, 0] == got[1, 0] == got[2, 0]        # the partial's bits


def _post(lib, box, v, t, shard, num_shards, step, timeout_ns):
    from moderngpu_b200 import binding
    binding._check(lib.mgpu_b200_shard_post(
        binding._DTYPES[v.dtype], binding._OPS["plus"], v.data_ptr(), v.numel(),
        t.data_ptr(), t.numel(), box.own, box.peers.data_ptr(), shard,
        num_shards, num_shards, step, timeout_ns, binding._stream(v.device)))


def test_mailbox_waits_are_bounded(mgpu):
    """A record that nobody posts and a ring slot that nobody releases: the
    waiting kernel gives up after its time limit, reports it through the
    mailbox's status word, leaves the output alone, and the context stays
    usable. One GPU, two shards of a chain, both held here."""
    import ctypes
    from moderngpu_b200 import binding
    lib = binding.load_library()
    v = torch.arange(1000, dtype=torch.int32, device="cuda")
    t = torch.tensor([0, 10, 500], dtype=torch.int32, device="cuda")
    out = mgpu.segreduce(v, t, op="plus", init=0)
    before = out.clone()
    limit = 3_000_000                       # 3 ms

    # (a) shard 0 collects, shard 1 never posted.
    box = sharded.Mailbox(shards_per_gpu=2)
    _post(lib, box, v, t, 0, 2, 1, limit)
    init = ctypes.c_int(0)
    binding._check(lib.mgpu_b200_shard_collect(
        binding._DTYPES[v.dtype], binding._OPS["plus"], box.own,
        box.peers.data_ptr(), 0, 2, 2, 1, out.data_ptr(), t.numel(),
        ctypes.byref(init), limit, binding._stream(v.device)))
    assert box.status() == 3
    assert torch.equal(out, before)
    box.close()

    # (b) 65 posts and no collect: the 65th finds its ring slot still taken.
    box = sharded.Mailbox(shards_per_gpu=1)
    for step in range(1, 65):
        _post(lib, box, v, t, 0, 1, step, limit)
    assert box.status() == 0
    _post(lib, box, v, t, 0, 1, 65, limit)
    assert box.status() == 4
    box.close()

    # (c) the fused step: shard 0's reduction ends with the collect, and the
    # record of shard 1 never comes. The reduction's own outputs stand.
    box = sharded.Mailbox(shards_per_gpu=2)
    dtype = binding._DTYPES[v.dtype]
    need = lib.mgpu_b200_segreduce_workspace_bytes(dtype, v.numel(), t.numel())
    space = torch.empty(max(need, 1 << 20), dtype=torch.uint8, device="cuda")
    fused_out = torch.full_like(before, -1)
    binding._check(lib.mgpu_b200_shard_begin(
        dtype, binding._OPS["plus"], v.data_ptr(), v.numel(), t.data_ptr(),
        t.numel(), space.data_ptr(), space.numel(), box.own,
        box.peers.data_ptr(), 0, 2, 2, 1, limit, binding._stream(v.device)))
    binding._check(lib.mgpu_b200_shard_finish(
        dtype, binding._OPS["plus"], v.data_ptr(), v.numel(), t.data_ptr(),
        t.numel(), fused_out.data_ptr(), ctypes.byref(init), space.data_ptr(),
        space.numel(), box.own, box.peers.data_ptr(), 0, 2, 2, 1, limit,
        binding._stream(v.device)))
    assert box.status() == 3
    assert torch.equal(fused_out, before)
    box.clear_status()
    assert box.status() == 0
    box.close()

    # The context still works.
    again = mgpu.segreduce(v, t, op="plus", init=0)
    assert torch.equal(again, before)


def stall_worker(rank, world, port, queue):
    """Step 1: every rank takes part. Step 2: the last rank stalls (posts
    nothing, collects nothing, stays alive). Step 3: every rank again."""
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world,
                            device_id=torch.device("cuda", rank))
    try:
        values, seg = make_problem("few_long", np.int64)
        begin, end, first, table = sharded.shard_table(seg, values.size, rank, world)
        v = torch.from_numpy(values[begin:end].copy()).cuda()
        t = torch.from_numpy(table).cuda()
        box = sharded.Mailbox(timeout_ns=20_000_000)          # 20 ms
        report = {}
        for step in (1, 2, 3):
            if step == 2 and rank == world - 1:
                box.next_step()                 # the stalled rank skips the step
                out = None
            else:
                out = sharded.sharded_segreduce(v, t, op="plus", init=-7, mailbox=box)
            torch.cuda.synchronize()
            report[step] = (box.status(),
                            None if out is None else out.cpu().numpy().tolist())
            box.clear_status()      # so that step 3 shows its own status
            dist.barrier()
        box.close()
        pieces = [None] * world
        dist.all_gather_object(pieces, (first, report))
        if rank == 0:
            queue.put(pieces)
    finally:
        dist.destroy_process_group()


def test_a_stalled_rank_is_detected_not_waited_for(oracle):
    """Failure detection without a GPU fault: when a rank posts no record for
    a step, the rank that owns the straddling segment gives up after its time
    limit, reports status 3 through its mailbox, leaves its own result
    unfolded, and the next step works again. Plain peer stores, NVLS off; no
    process exits while another may still write to it."""
    world = 2
    if torch.cuda.device_count() < world:
        pytest.skip("needs two GPUs")
    ctx = mp.get_context("spawn")
    queue = ctx.Queue()
    port = free_port()
    procs = [ctx.Process(target=stall_worker, args=(r, world, port, queue))
             for r in range(world)]
    for p in procs:
        p.start()
    pieces = queue.get(timeout=300)
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    values, seg = make_problem("few_long", np.int64)
    want = oracle.segreduce(values, seg.astype(np.int32), op="plus", init=-7)
    (first0, rep0), (first1, rep1) = pieces
    # Steps 1 and 3: the assembled result is the whole array's reduction.
    for step in (1, 3):
        got = np.zeros(seg.size, dtype=np.int64)
        for first, rep in pieces:
            vals = rep[step][1][1:]
            got[first:first + len(vals)] = vals
        assert np.array_equal(got, want)
    assert rep0[1][0] == 0 and rep1[1][0] == 0
    assert rep0[3][0] == 0 and rep1[3][0] == 0    # one stall, one report
    # Step 2 on rank 0: timed out waiting for rank 1's record, said so, and
    # kept the reduction of its own items in the straddling segment.
    assert rep0[2][0] == 3
    half = values.size // 2
    last_start = int(seg[seg < half][-1])      # rank 0's straddling segment
    own_part = int(values[last_start:half].sum())
    assert rep0[2][1][-1] == own_part
    assert rep1[2][1] is None
