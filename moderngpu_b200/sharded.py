"""Multi-GPU segmented reduction: one process per GPU, the item range cut
evenly across ranks, one 16-byte boundary record exchanged per shard and step.

The reference is single-device (src/moderngpu/context.hxx:85,109-110 knows one
stream on the current device); this layer is new. It binds the C ABI's shard
entry points for the one-process-per-GPU case; a C++ program that drives
several GPUs from one process uses mgpu::sharded_segreduce
(include/moderngpu/kernel_sharded.hxx), which runs the same kernels.

Default data path (with a `Mailbox`; no collective anywhere in it), two
launches per shard and step:

  1. mgpu_b200_shard_begin: the partitioner of the shard's reduction; a few
     extra CTAs of the same launch fold the shard's leading items (those
     before its first segment start) and store the record straight into the
     memory of the GPUs that hold earlier shards -- peer-to-peer stores over
     NVLink into memory mapped with CUDA IPC;
  2. mgpu_b200_shard_finish: the reduction kernel on (items, shard-local
     start table); the thread that stores the shard's last output first
     waits -- in its own GPU's memory, for a bounded time -- for the
     following shards' records and folds them in, in shard order.

`Mailbox(fused=False)` runs the same exchange as four launches
(mgpu_b200_shard_post, the reduction's two, mgpu_b200_shard_collect).

Without a mailbox the records travel by one torch.distributed all_gather of
16 bytes per rank: mgpu_b200_shard_lead (record from the leading items, the
all-gather overlapping the reduction) or, with overlap=False,
mgpu_b200_shard_pack (record from the reduction's first output), then
mgpu_b200_shard_fold on the owner.

Shard-local start table: entry 0 is always 0 and stands for the segment
carried in from the previous rank; the remaining entries are the local offsets
of the segments that START inside the shard. `shard_table` derives it from a
global start table on the host; mgpu::sharded_partition does it on the
devices.
"""
import ctypes

import numpy as np
import torch
import torch.distributed as dist

from . import binding

RECORD_BYTES = 16
HAS_PARTIAL, HAS_START, LAST_EMPTY = 1, 2, 4


def shard_bounds(count, world):
    """Item range [begin, end) of every rank: an even cut of [0, count)."""
    edges = [(count * r) // world for r in range(world + 1)]
    return [(edges[r], edges[r + 1]) for r in range(world)]


def shard_table(segments, count, rank, world):
    """Shard-local start table of `rank` for a global problem.

    segments: global int64/int32 start offsets (numpy, sorted, segments[0]==0).
    Returns (item_begin, item_end, first_segment, table) where `table` is an
    int32 array [0, local starts...] and `first_segment` is the global index
    of the first segment that starts inside the shard. A segment that starts
    exactly at item_end belongs to the next rank, except on the last rank,
    which also takes the trailing (empty) segments that start at count."""
    segments = np.asarray(segments)
    begin, end = shard_bounds(count, world)[rank]
    first = int(np.searchsorted(segments, begin, side="left"))
    if rank == world - 1:
        last = segments.size
    else:
        last = int(np.searchsorted(segments, end, side="left"))
    local = (segments[first:last].astype(np.int64) - begin).astype(np.int32)
    table = np.concatenate([np.zeros(1, dtype=np.int32), local])
    return begin, end, first, table


def pack_record_host(out0_bits, table, count):
    """The boundary record of a shard whose outputs are already on the host
    (the host-buffer path): same flags as mgpu_b200_shard_pack."""
    flags = 0
    real = table.size > 1
    first = int(table[1]) if real else count
    if first > 0:
        flags |= HAS_PARTIAL
    if real:
        flags |= HAS_START
    if real and int(table[-1]) >= count:
        flags |= LAST_EMPTY
    rec = np.zeros(2, dtype=np.uint64)
    rec[0] = out0_bits
    rec[1] = flags
    return rec


def fold_plan(flags, rank):
    """Ranks whose boundary partial the rank `rank` must fold into its last
    segment, in order: every later rank with a partial, up to and including
    the first later rank that holds a segment start of its own. Empty when
    `rank` holds no segment start (it owns nothing)."""
    if not flags[rank] & HAS_START:
        return []
    take = []
    for k in range(rank + 1, len(flags)):
        if flags[k] & HAS_PARTIAL:
            take.append(k)
        if flags[k] & HAS_START:
            break
    return take


class MailboxError(RuntimeError):
    """The peer-to-peer mailboxes could not be set up on every rank."""


class Mailbox:
    """This rank's mailbox and its mapping of every other rank's mailbox.

    Collective over `group`: every rank constructs one at the same time (the
    64-byte handles travel through the process group once, at set-up; no
    collective runs in the data path afterwards). shards_per_gpu: how many
    consecutive shards of the chain each rank holds. side_stream: post the
    records on a stream of the mailbox's own, forked from and joined to the
    caller's stream by events. Use one Mailbox per stream, call `close()`
    (collective) when done."""

    def __init__(self, group=None, shards_per_gpu=1, device=None,
                 timeout_ns=0, side_stream=True, fused=True):
        lib = binding.load_library()
        self.lib = lib
        # fused: two launches per shard and step (post and collect ride in the
        # partitioner's and the reduction's launches); otherwise four.
        self.fused = fused
        self._spaces = []
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.per_gpu = shards_per_gpu
        self.num_shards = self.world * shards_per_gpu
        self.timeout_ns = timeout_ns
        self.step = 0
        if device is None:
            device = torch.device("cuda", torch.cuda.current_device())
        self.device = device
        # Set-up is all-or-nothing across the group: a rank on which a step
        # fails keeps taking part in the collectives below, and every rank
        # learns of the failure from the final vote.
        failure = None
        self.own = None
        self.opened = []
        handle = (ctypes.c_ubyte * 64)()
        try:
            own = ctypes.c_void_p()
            with torch.cuda.device(device):
                binding._check(lib.mgpu_b200_mailbox_create(ctypes.byref(own),
                                                            handle))
            self.own = own.value
        except Exception as e:                      # noqa: BLE001
            failure = e
        handles = [bytes(handle)]
        if self.world > 1:
            handles = [None] * self.world
            dist.all_gather_object(
                handles, bytes(handle) if failure is None else None,
                group=group)
        pointers = []
        if failure is None and all(h is not None for h in handles):
            try:
                with torch.cuda.device(device):
                    for k in range(self.world):
                        if k == self.rank:
                            pointers.append(self.own)
                            continue
                        peer = ctypes.c_void_p()
                        raw = (ctypes.c_ubyte * 64).from_buffer_copy(handles[k])
                        binding._check(lib.mgpu_b200_mailbox_open(
                            raw, ctypes.byref(peer)))
                        self.opened.append(peer.value)
                        pointers.append(peer.value)
            except Exception as e:                  # noqa: BLE001
                failure = e
        elif failure is None:
            failure = MailboxError("another rank could not create its mailbox")
        if self.world > 1:
            vote = torch.tensor([0 if failure is None else 1], device=device,
                                dtype=torch.int32)
            dist.all_reduce(vote, op=dist.ReduceOp.MAX, group=group)
            if int(vote.item()) and failure is None:
                failure = MailboxError("another rank could not map the mailboxes")
        if failure is not None:
            self._release()
            raise MailboxError("peer-to-peer mailbox set-up failed: %s"
                               % failure)
        self.peers = torch.tensor(pointers, dtype=torch.int64, device=device)
        self.side = self.fork = self.join = None
        if side_stream:
            self.side = torch.cuda.Stream(device=device)
            self.fork = torch.cuda.Event()
            self.join = torch.cuda.Event()
        torch.cuda.synchronize(device)

    def _release(self):
        with torch.cuda.device(self.device):
            for peer in self.opened:
                self.lib.mgpu_b200_mailbox_close(peer)
            if self.own is not None:
                self.lib.mgpu_b200_mailbox_destroy(self.own)
        self.own, self.opened = None, []

    def next_step(self):
        self.step += 1
        return self.step

    def workspaces(self, sizes):
        """One scratch buffer per shard of this rank (the fused step keeps
        every shard's partition table until its reduction has run)."""
        while len(self._spaces) < len(sizes):
            self._spaces.append(None)
        for j, need in enumerate(sizes):
            buf = self._spaces[j]
            if buf is None or buf.numel() < need:
                self._spaces[j] = torch.empty(max(need, 1 << 20),
                                              dtype=torch.uint8,
                                              device=self.device)
        return self._spaces[:len(sizes)]

    def clear_status(self):
        """Status word back to 0 (enqueued on the current stream), so that
        a later wait that runs out can be told from an earlier one."""
        with torch.cuda.device(self.device):
            binding._check(self.lib.mgpu_b200_mailbox_clear_status(
                self.own, binding._stream(self.device)))

    def status(self):
        """0, or the code of the first bounded wait that ran out (3: a record
        did not arrive, 4: a ring slot was not released). Synchronises."""
        out = ctypes.c_int(0)
        with torch.cuda.device(self.device):
            binding._check(self.lib.mgpu_b200_mailbox_status(
                self.own, binding._stream(self.device), ctypes.byref(out)))
        return out.value

    def close(self):
        if self.own is None:
            return
        torch.cuda.synchronize(self.device)
        if self.world > 1:
            dist.barrier(group=self.group)     # nobody still writes to anybody
        with torch.cuda.device(self.device):
            for peer in self.opened:
                binding._check(self.lib.mgpu_b200_mailbox_close(peer))
            if self.world > 1:
                dist.barrier(group=self.group)  # every mapping is gone
            binding._check(self.lib.mgpu_b200_mailbox_destroy(self.own))
        self.own, self.opened = None, []


_lead_scratch = {}


def lead_scratch(dev):
    """Zeroed scratch of mgpu_b200_shard_lead, one per device (calls on one
    stream follow one another, and every call leaves it zeroed)."""
    key = (dev.type, dev.index)
    if key not in _lead_scratch:
        lib = binding.load_library()
        size = lib.mgpu_b200_shard_lead_scratch_bytes()
        _lead_scratch[key] = torch.zeros((size + 7) // 8, dtype=torch.int64,
                                         device=dev)
    return _lead_scratch[key]


def sharded_segreduce(values, table, op="plus", init=0, group=None,
                      records=None, overlap=True, mailbox=None, out=None):
    """Reduce this rank's shard and fold boundary partials across ranks.

    values: this rank's items (CUDA tensor); table: its shard-local start
    table (see module docstring). Returns the local outputs (table.numel()
    entries; entry 0 is this rank's boundary partial, owned by an earlier
    rank). Every step runs in the library's kernels and the exchange is one
    all_gather of 16 bytes per rank. There is no CPU path."""
    if not values.is_cuda:
        raise binding.LibraryMissing(
            "sharded_segreduce runs on CUDA tensors only (no CPU fallback)")
    if mailbox is not None:
        return sharded_segreduce_multi(
            [(values, table)], op=op, init=init, mailbox=mailbox,
            outs=None if out is None else [out])[0]
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    return _sharded_cuda(values, table, op, init, group, rank, world, records,
                         overlap, out)


def _sharded_cuda(values, table, op, init, group, rank, world, records,
                  overlap, out=None):
    lib = binding.load_library()
    dev = values.device
    dtype = binding._DTYPES[values.dtype]
    stream = binding._stream(dev)
    mine = torch.empty(RECORD_BYTES, dtype=torch.uint8, device=dev)
    if records is None:
        records = torch.empty(world * RECORD_BYTES, dtype=torch.uint8,
                              device=dev)
    with torch.cuda.device(dev):
        pending = None
        if overlap:
            binding._check(lib.mgpu_b200_shard_lead(
                dtype, binding._OPS[op], values.data_ptr(), values.numel(),
                table.data_ptr(), table.numel(), mine.data_ptr(),
                lead_scratch(dev).data_ptr(), stream))
            if world > 1:
                pending = dist.all_gather_into_tensor(records, mine,
                                                      group=group,
                                                      async_op=True)
        out = binding.segreduce(values, table, op=op, init=init, out=out)
        if not overlap:
            binding._check(lib.mgpu_b200_shard_pack(
                dtype, out.data_ptr(), table.data_ptr(), table.numel(),
                values.numel(), mine.data_ptr(), stream))
            if world > 1:
                dist.all_gather_into_tensor(records, mine, group=group)
        if pending is not None:
            pending.wait()
        if world == 1:
            records[:RECORD_BYTES].copy_(mine)
        init_c = binding._CTYPES[values.dtype](init)
        binding._check(lib.mgpu_b200_shard_fold(
            dtype, binding._OPS[op], records.data_ptr(), rank, world,
            out.data_ptr(), table.numel(), ctypes.byref(init_c), stream))
    return out


def _sharded_mailbox(shards, op, init, outs, workspace, mailbox):
    """The fused step: every shard's partitioner (its launch also posts the
    shard's boundary record), then every shard's reduction (the thread that
    stores the last output collects the following shards' records first): two launches per shard."""
    lib = mailbox.lib
    k = len(shards)
    if k != mailbox.per_gpu:
        raise ValueError("the mailbox was set up for %d shards per GPU" %
                         mailbox.per_gpu)
    dev = shards[0][0].device
    dtype = binding._DTYPES[shards[0][0].dtype]
    stream = binding._stream(dev)
    step = mailbox.next_step()
    first = mailbox.rank * k
    init_c = binding._CTYPES[shards[0][0].dtype](init)
    results = []
    with torch.cuda.device(dev):
        spaces = mailbox.workspaces(
            [lib.mgpu_b200_segreduce_workspace_bytes(
                dtype, values.numel(), table.numel())
             for values, table in shards])
        for j, (values, table) in enumerate(shards):
            binding._check(lib.mgpu_b200_shard_begin(
                dtype, binding._OPS[op], values.data_ptr(), values.numel(),
                table.data_ptr(), table.numel(), spaces[j].data_ptr(),
                spaces[j].numel(), mailbox.own, mailbox.peers.data_ptr(),
                first + j, mailbox.num_shards, k, step, mailbox.timeout_ns,
                stream))
        for j, (values, table) in enumerate(shards):
            out = None if outs is None else outs[j]
            if out is None:
                out = torch.empty(table.numel(), dtype=values.dtype,
                                  device=dev)
            binding._check(lib.mgpu_b200_shard_finish(
                dtype, binding._OPS[op], values.data_ptr(), values.numel(),
                table.data_ptr(), table.numel(), out.data_ptr(),
                ctypes.byref(init_c), spaces[j].data_ptr(), spaces[j].numel(),
                mailbox.own, mailbox.peers.data_ptr(), first + j,
                mailbox.num_shards, k, step, mailbox.timeout_ns, stream))
            results.append(out)
    return results


def _sharded_mailbox_unfused(shards, op, init, outs, workspace, mailbox):
    """The same exchange as four launches per shard (post, partitioner,
    reduction, collect): kept for comparison and for callers that drive the
    three entry points themselves."""
    lib = mailbox.lib
    k = len(shards)
    if k != mailbox.per_gpu:
        raise ValueError("the mailbox was set up for %d shards per GPU" %
                         mailbox.per_gpu)
    dev = shards[0][0].device
    dtype = binding._DTYPES[shards[0][0].dtype]
    stream = binding._stream(dev)
    step = mailbox.next_step()
    first = mailbox.rank * k
    init_c = binding._CTYPES[shards[0][0].dtype](init)
    results = []
    with torch.cuda.device(dev):
        # The posts depend on nothing the reductions produce: on the mailbox's
        # side stream they run beside the partitioner and the first tiles
        # instead of in front of them.
        side = mailbox.side
        post_stream = stream
        if side is not None:
            mailbox.fork.record(torch.cuda.current_stream(dev))
            side.wait_event(mailbox.fork)
            post_stream = ctypes.c_void_p(side.cuda_stream)
        for j, (values, table) in enumerate(shards):
            binding._check(lib.mgpu_b200_shard_post(
                dtype, binding._OPS[op], values.data_ptr(), values.numel(),
                table.data_ptr(), table.numel(), mailbox.own,
                mailbox.peers.data_ptr(), first + j, mailbox.num_shards, k,
                step, mailbox.timeout_ns, post_stream))
        if side is not None:
            mailbox.join.record(side)
        for j, (values, table) in enumerate(shards):
            results.append(binding.segreduce(
                values, table, op=op, init=init,
                out=None if outs is None else outs[j], workspace=workspace))
        if side is not None:
            # The collects read this GPU's own records too.
            torch.cuda.current_stream(dev).wait_event(mailbox.join)
        for j, (values, table) in enumerate(shards):
            binding._check(lib.mgpu_b200_shard_collect(
                dtype, binding._OPS[op], mailbox.own,
                mailbox.peers.data_ptr(), first + j, mailbox.num_shards, k,
                step, results[j].data_ptr(), table.numel(),
                ctypes.byref(init_c), mailbox.timeout_ns, stream))
    return results


def sharded_segreduce_multi(shards, op="plus", init=0, group=None, outs=None,
                            workspace=None, overlap=True, mailbox=None):
    """Several consecutive shards per rank (CUDA tensors only).

    shards: list of (values, table) pairs held by this rank, in array order;
    every rank holds the same number k of shards, and rank r's shards are
    shards r*k .. r*k+k-1 of the whole array. Used when one GPU's share of the
    array exceeds what a single call can index (count + segments < 2^31), for
    instance the whole 2^32-item array on one GPU as 8 shards. One all-gather
    of k records per rank; the fold treats the world*k shards as one chain.
    Returns the list of per-shard outputs. With `mailbox` the records travel
    by peer-to-peer stores and no collective runs."""
    if mailbox is not None:
        if mailbox.fused:
            return _sharded_mailbox(shards, op, init, outs, workspace, mailbox)
        return _sharded_mailbox_unfused(shards, op, init, outs, workspace,
                                        mailbox)
    lib = binding.load_library()
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    rank = dist.get_rank(group) if dist.is_initialized() else 0
    k = len(shards)
    dev = shards[0][0].device
    dtype = binding._DTYPES[shards[0][0].dtype]
    stream = binding._stream(dev)
    mine = torch.empty(k * RECORD_BYTES, dtype=torch.uint8, device=dev)
    records = torch.empty(world * k * RECORD_BYTES, dtype=torch.uint8,
                          device=dev)
    results = []
    with torch.cuda.device(dev):
        pending = None
        if overlap:
            for j, (values, table) in enumerate(shards):
                binding._check(lib.mgpu_b200_shard_lead(
                    dtype, binding._OPS[op], values.data_ptr(),
                    values.numel(), table.data_ptr(), table.numel(),
                    mine.data_ptr() + j * RECORD_BYTES,
                    lead_scratch(dev).data_ptr(), stream))
            if world > 1:
                pending = dist.all_gather_into_tensor(records, mine,
                                                      group=group,
                                                      async_op=True)
        for j, (values, table) in enumerate(shards):
            out = binding.segreduce(values, table, op=op, init=init,
                                    out=None if outs is None else outs[j],
                                    workspace=workspace)
            if not overlap:
                binding._check(lib.mgpu_b200_shard_pack(
                    dtype, out.data_ptr(), table.data_ptr(), table.numel(),
                    values.numel(), mine.data_ptr() + j * RECORD_BYTES,
                    stream))
            results.append(out)
        if world > 1 and not overlap:
            dist.all_gather_into_tensor(records, mine, group=group)
        if pending is not None:
            pending.wait()
        if world == 1:
            records.copy_(mine)
        init_c = binding._CTYPES[shards[0][0].dtype](init)
        for j, (values, table) in enumerate(shards):
            binding._check(lib.mgpu_b200_shard_fold(
                dtype, binding._OPS[op], records.data_ptr(), rank * k + j,
                world * k, results[j].data_ptr(), table.numel(),
                ctypes.byref(init_c), stream))
    return results
