"""Parity of the CUDA segreduce (through the C ABI) with the CPU oracle:
bit-exact for integer types and for max/min, tolerance for floating-point
sums (|got - ref| <= tol * max(|ref|, sum |x|), tol = 1e-5 for fp32 and 1e-12
for fp64 against a wider host accumulation)."""
import numpy as np
import pytest
import torch

from moderngpu_b200 import workloads

pytestmark = pytest.mark.gpu

FP32_TOL = 1e-5
FP64_TOL = 1e-12


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def random_segments(rng, count, num_segments):
    seg = np.zeros(num_segments, dtype=np.int32)
    if num_segments > 1:
        seg[1:] = np.sort(rng.integers(0, count + 1, size=num_segments - 1))
    return seg


def check_exact(mgpu, oracle, values, seg, op, init):
    got = mgpu.segreduce(dev(values), dev(seg), op=op, init=init).cpu().numpy()
    want = oracle.segreduce(values, seg, op=op, init=init)
    assert mgpu.workspace_status() == 0
    bad = np.nonzero(got != want)[0]
    assert bad.size == 0, "first mismatch at segment %d: got %r want %r" % (
        bad[0], got[bad[0]], want[bad[0]])


def check_sum(mgpu, oracle, values, seg, init, tol):
    got = mgpu.segreduce(dev(values), dev(seg), op="plus", init=init)
    got = got.cpu().numpy().astype(np.float64)
    want, mags = oracle.segsum_wide(values, seg, init=init)
    assert mgpu.workspace_status() == 0
    bound = tol * np.maximum(np.abs(want), mags)
    err = np.abs(got - want)
    worst = int(np.argmax(err - bound))
    assert np.all(err <= bound), "segment %d: got %r want %r" % (
        worst, got[worst], want[worst])


@pytest.mark.parametrize("seed", range(8))
def test_config1_int32_plus_bit_exact(mgpu, oracle, seed):
    values, seg = workloads.config1(seed=seed)
    check_exact(mgpu, oracle, values, seg, "plus", 0)


@pytest.mark.parametrize("count,segs", [
    (0, [0]), (0, [0, 0, 0]), (1, [0]), (1, [0, 0, 1]), (10, [0, 3, 3, 7]),
    (100, [0, 50, 100, 100]), (7159, [0]), (7160, [0, 7160]), (7161, [0, 1]),
    (20000, [0] + [5] * 9000 + [19999]),
])
def test_edge_shapes(mgpu, oracle, count, segs):
    rng = np.random.default_rng(count + len(segs))
    values = rng.integers(-100, 100, size=count).astype(np.int32)
    check_exact(mgpu, oracle, values, np.array(segs, dtype=np.int32), "plus", -1)


@pytest.mark.parametrize("dtype", [np.int32, np.int64, np.float32, np.float64])
@pytest.mark.parametrize("op", ["plus", "max", "min"])
def test_all_types_and_ops(mgpu, oracle, dtype, op):
    rng = np.random.default_rng(17)
    count, num_segments = 3_000_001, 90_000
    seg = random_segments(rng, count, num_segments)
    if np.issubdtype(dtype, np.integer):
        values = rng.integers(-1000, 1000, size=count).astype(dtype)
        check_exact(mgpu, oracle, values, seg, op, dtype(-7))
    elif op != "plus":
        values = rng.standard_normal(count).astype(dtype)
        check_exact(mgpu, oracle, values, seg, op, dtype(-7))
    else:
        values = (rng.random(count) * 2 - 1).astype(dtype)
        check_sum(mgpu, oracle, values, seg, -7.0,
                  FP32_TOL if dtype == np.float32 else FP64_TOL)


@pytest.mark.parametrize("shift_values,shift_segments",
                         [(1, 0), (3, 0), (0, 1), (2, 3)])
def test_unaligned_pointers(mgpu, oracle, shift_values, shift_segments):
    """Arrays that start off a 16-byte boundary (views into larger tensors)."""
    rng = np.random.default_rng(23)
    count, num_segments = 1_000_003, 10_007
    values = rng.integers(-100, 100, size=count).astype(np.int32)
    seg = random_segments(rng, count, num_segments)
    v_dev = torch.zeros(count + 8, dtype=torch.int32, device="cuda")
    s_dev = torch.zeros(num_segments + 8, dtype=torch.int32, device="cuda")
    v_view = v_dev[shift_values:shift_values + count]
    s_view = s_dev[shift_segments:shift_segments + num_segments]
    v_view.copy_(torch.from_numpy(values))
    s_view.copy_(torch.from_numpy(seg))
    got = mgpu.segreduce(v_view, s_view, op="plus", init=0).cpu().numpy()
    assert np.array_equal(got, oracle.segreduce(values, seg, init=0))


def test_reference_test_shape_long_segments(mgpu, oracle):
    """tests/test_segreduce.cu:67-71 at full size for one seed: 1e8 items in
    100 segments, so a segment spans more than a thousand tiles; values are
    index % 13 materialised as int32, init = -1."""
    count, num_segments = 100_000_000, 100
    rng = np.random.default_rng(0)
    seg = random_segments(rng, count, num_segments)
    values = (torch.arange(count, device="cuda", dtype=torch.int32) % 13)
    got = mgpu.segreduce(values, dev(seg), op="plus", init=-1).cpu().numpy()
    want = oracle.segreduce_index_mod(count, seg, init=-1, modulus=13)
    assert mgpu.workspace_status() == 0
    assert np.array_equal(got, want)


@pytest.mark.parametrize("dtype", [np.int32, np.int64, np.float32, np.float64])
@pytest.mark.parametrize("length", [8, 16, 24, 31, 32, 33, 64, 100, 128])
def test_equal_length_segments(mgpu, oracle, dtype, length):
    """Rows of one fixed width: tiles whose segment starts all sit at the same
    position modulo 8 keep their run ends in shifted slots (no shared-memory
    bank holds them all); the other widths take the plain path. A tile's first
    item falls anywhere in a 16-byte granule of the input, so the starts'
    positions within the staged tile differ from tile to tile."""
    rng = np.random.default_rng(length)
    count = 1_000_003
    n = count // length
    seg = (np.arange(n, dtype=np.int64) * length).astype(np.int32)
    if np.issubdtype(dtype, np.integer):
        values = rng.integers(-1000, 1000, size=count + 3).astype(dtype)
        for off in (0, 1, 3):
            check_exact(mgpu, oracle, values[off:off + count], seg, "plus",
                        dtype(-7))
        check_exact(mgpu, oracle, values[:count], seg, "max", dtype(-7))
    else:
        values = (rng.random(count + 3) * 2 - 1).astype(dtype)
        tol = FP32_TOL if dtype == np.float32 else FP64_TOL
        for off in (0, 1):
            check_sum(mgpu, oracle, values[off:off + count], seg, -7.0, tol)
        check_exact(mgpu, oracle, values[:count], seg, "min", dtype(-7))


def test_equal_length_rows_with_empty_rows_and_one_long_row(mgpu, oracle):
    """Fixed-width rows mixed with runs of empty rows (equal starts) and one
    row that spans several tiles: aligned and unaligned tiles alternate, and a
    shifted tile may be the one that closes a segment opened tiles before."""
    rng = np.random.default_rng(5)
    starts, at = [], 0
    for block in range(400):
        kind = block % 4
        if kind == 0:
            for _ in range(300):
                starts.append(at)
                at += 32
        elif kind == 1:
            starts += [at] * 50          # empty rows
            starts.append(at)
            at += 20_000                 # one long row
        elif kind == 2:
            for _ in range(500):
                starts.append(at)
                at += 16
        else:
            for _ in range(200):
                starts.append(at)
                at += int(rng.integers(1, 60))
    count = at + 5
    seg = np.array(starts, dtype=np.int32)
    values = rng.integers(-50, 50, size=count).astype(np.int32)
    check_exact(mgpu, oracle, values, seg, "plus", -1)
    fvalues = (rng.random(count) * 2 - 1).astype(np.float32)
    check_sum(mgpu, oracle, fvalues, seg, 0.0, FP32_TOL)
    check_exact(mgpu, oracle, fvalues.astype(np.float64), seg, "max", -9.0)


def test_many_empty_segments(mgpu, oracle):
    rng = np.random.default_rng(5)
    count, num_segments = 5000, 200_000
    values = rng.integers(-9, 9, size=count).astype(np.int32)
    seg = random_segments(rng, count, num_segments)
    check_exact(mgpu, oracle, values, seg, "plus", -1)


def test_config2_reduced(mgpu, oracle):
    values, seg = workloads.config2(seed=1, count=1 << 24, num_segments=1 << 19)
    got = mgpu.segreduce(values, seg, op="plus", init=0.0).cpu().numpy()
    want, mags = oracle.segsum_wide(values.cpu().numpy(), seg.cpu().numpy())
    err = np.abs(got.astype(np.float64) - want)
    assert np.all(err <= FP32_TOL * np.maximum(np.abs(want), mags))


def test_config2_full_size_properties(mgpu, oracle):
    """268,435,456 fp32 items, 8,388,608 segments: direct comparison with the
    oracle, plus two size-independent properties."""
    values, seg = workloads.config2(seed=1)
    out = mgpu.segreduce(values, seg, op="plus", init=0.0)
    assert mgpu.workspace_status() == 0
    # Linearity: doubling every item doubles every sum exactly in fp32.
    out2 = mgpu.segreduce(values * 2, seg, op="plus", init=0.0)
    assert torch.equal(out2, out * 2)
    # Checksum of checksums: the segment sums add up to the grand total.
    total = values.sum(dtype=torch.float64).item()
    assert abs(out.sum(dtype=torch.float64).item() - total) <= 1e-6 * values.numel() ** 0.5 * 16
    # Integer-valued items make every order of summation exact.
    ints = torch.randint(-8, 9, (values.numel(),), device="cuda").to(torch.float32)
    got = mgpu.segreduce(ints, seg, op="plus", init=0.0).cpu().numpy()
    want = oracle.segreduce(ints.cpu().numpy(), seg.cpu().numpy(), init=0.0,
                            threads=oracle.max_threads())
    assert np.array_equal(got, want)
    # And the real-valued run against the wide host accumulation.
    want, mags = oracle.segsum_wide(values.cpu().numpy(), seg.cpu().numpy())
    err = np.abs(out.cpu().numpy().astype(np.float64) - want)
    assert np.all(err <= FP32_TOL * np.maximum(np.abs(want), mags))


def test_config5_shaped_fp64_single_gpu(mgpu, oracle):
    values, seg = workloads.config5_shard(4, 0, 1 << 24)
    got_max = mgpu.segreduce(values, seg, op="max", init=-1e300).cpu().numpy()
    want_max = oracle.segreduce(values.cpu().numpy(), seg.cpu().numpy(),
                                op="max", init=-1e300)
    assert np.array_equal(got_max, want_max)
    got = mgpu.segreduce(values, seg, op="plus", init=0.0).cpu().numpy()
    want, mags = oracle.segsum_wide(values.cpu().numpy(), seg.cpu().numpy())
    assert np.all(np.abs(got - want) <= FP64_TOL * np.maximum(np.abs(want), mags))


def test_repeatable_integer_results(mgpu):
    """Two runs on the same input give identical integer outputs (a race in
    the tile-status protocol would show up here)."""
    values, seg = workloads.config1(seed=3, count=1 << 24, num_segments=1 << 16)
    a = mgpu.segreduce(dev(values), dev(seg), init=0)
    b = mgpu.segreduce(dev(values), dev(seg), init=0)
    assert torch.equal(a, b)


def test_calls_replay_from_a_cuda_graph(mgpu, oracle):
    """A call only enqueues its two launches on the caller's stream (the
    reduction as a programmatic dependent of the partitioner): no allocation,
    no synchronisation, no host read of device memory. So a sequence of calls
    with a caller-supplied workspace can be captured in a CUDA graph and
    replayed, which is how a latency-bound caller takes the host's launch cost
    off small problems. Replays see the arrays' current contents."""
    values, seg = workloads.config1(seed=4)
    v, s = dev(values), dev(seg)
    ops = [("plus", 0), ("max", -5), ("min", 7)]
    outs = [torch.empty(seg.size, dtype=torch.int32, device="cuda")
            for _ in ops]
    workspace = torch.empty(4 << 20, dtype=torch.uint8, device="cuda")
    # First use sets up per-device state (function attributes, the status
    # word): outside the capture.
    for (op, init), out in zip(ops, outs):
        mgpu.segreduce(v, s, op=op, init=init, out=out, workspace=workspace)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for (op, init), out in zip(ops, outs):
            mgpu.segreduce(v, s, op=op, init=init, out=out,
                           workspace=workspace)
    rng = np.random.default_rng(9)
    for _ in range(3):
        values = rng.integers(-1000, 1000, size=values.size).astype(np.int32)
        v.copy_(torch.from_numpy(values))
        for out in outs:
            out.fill_(123456)
        graph.replay()
        torch.cuda.synchronize()
        assert mgpu.workspace_status(workspace) == 0
        for (op, init), out in zip(ops, outs):
            want = oracle.segreduce(values, seg, op=op, init=init)
            assert np.array_equal(out.cpu().numpy(), want), op


def test_host_buffer_entry_point(mgpu, oracle):
    rng = np.random.default_rng(31)
    count, num_segments = 70_000_000, 2_000_000     # three chunks
    values = torch.from_numpy(rng.integers(-50, 50, size=count).astype(np.int32))
    seg = torch.from_numpy(random_segments(rng, count, num_segments))
    got = mgpu.segreduce_host(values.pin_memory(), seg.pin_memory(), init=-1)
    want = oracle.segreduce(values.numpy(), seg.numpy(), init=-1,
                            threads=oracle.max_threads())
    assert np.array_equal(got.numpy(), want)


def test_workspace_too_small_is_reported(mgpu):
    values = torch.zeros(1 << 20, dtype=torch.float32, device="cuda")
    seg = torch.zeros(16, dtype=torch.int32, device="cuda")
    tiny = torch.empty(256, dtype=torch.uint8, device="cuda")
    with pytest.raises(mgpu.MgpuError) as info:
        mgpu.segreduce(values, seg, workspace=tiny)
    assert info.value.code == 2


MAX_MERGED = 0x7FFFFFFF - 65536      # count + num_segments a single call takes


def test_maximum_size_single_call(mgpu):
    """The largest problem one call indexes (count + num_segments =
    2^31 - 65537, as in the reference, whose grid is sized from the same sum):
    int32 ones, segment sums must equal the segment lengths; the load-balancing
    search of the same shape must number every item. One item more is refused
    with an error code instead of wrapping around."""
    num_segments = 1_000_003
    count = MAX_MERGED - num_segments
    g = torch.Generator(device="cuda").manual_seed(8)
    cuts = torch.randint(0, count, (num_segments - 1,), device="cuda", generator=g)
    segments = torch.cat([torch.zeros(1, dtype=torch.int64, device="cuda"),
                          torch.sort(cuts)[0]]).to(torch.int32)
    del cuts
    values = torch.ones(count, dtype=torch.int32, device="cuda")
    out = mgpu.segreduce(values, segments, op="plus", init=-5)
    ends = torch.cat([segments[1:], torch.tensor([count], dtype=torch.int32, device="cuda")])
    lengths = ends - segments
    want = torch.where(lengths > 0, lengths, torch.full_like(lengths, -5))
    assert torch.equal(out, want)
    assert mgpu.workspace_status() == 0
    del values, out

    seg = mgpu.load_balance_search(count, segments)
    # Every item's segment starts at or before it and the next one after it;
    # checked in slices to keep the temporaries small.
    step = 1 << 28
    for lo in range(0, count, step):
        hi = min(lo + step, count)
        index = torch.arange(lo, hi, device="cuda", dtype=torch.int64)
        s = seg[lo:hi].to(torch.int64)
        assert bool((segments[s].to(torch.int64) <= index).all())
        assert bool((ends[s].to(torch.int64) > index).all())
    del seg

    too_many = torch.empty(count + 1, dtype=torch.int32, device="cuda")
    with pytest.raises(mgpu.MgpuError):
        mgpu.segreduce(too_many, segments, op="plus", init=0)
