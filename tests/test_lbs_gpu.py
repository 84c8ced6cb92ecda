"""Load-balancing search, partitions and interval_expand: bit-exact against the
CPU oracle and the golden vectors made by the reference's merge_path."""
import json
import os

import numpy as np
import pytest
import torch

from moderngpu_b200 import workloads

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "lbs_partitions.json")


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def golden_cases():
    with open(GOLDEN) as f:
        return json.load(f)["cases"]


@pytest.mark.parametrize("case", golden_cases(), ids=lambda c: c["name"])
def test_partitions_match_golden(mgpu, case):
    seg = dev(np.array(case["segments"], dtype=np.int32))
    for spacing, expect in case["partitions"].items():
        got = mgpu.load_balance_partitions(case["count"], seg, int(spacing))
        assert got.cpu().tolist() == expect


@pytest.mark.parametrize("count,num_segments,spacing", [
    (1 << 20, 10_000, 896), (1 << 20, 10_001, 7160), (10_000_000, 10, 5112),
    (5000, 200_000, 100), (5000, 200_003, 1), (100, 1, 7),
])
def test_partitions_match_oracle(mgpu, oracle, count, num_segments, spacing):
    rng = np.random.default_rng(count % 1000 + num_segments)
    seg = np.zeros(num_segments, dtype=np.int32)
    seg[1:] = np.sort(rng.integers(0, count + 1, size=num_segments - 1))
    got = mgpu.load_balance_partitions(count, dev(seg), spacing).cpu().numpy()
    assert np.array_equal(got, oracle.load_balance_partitions(count, seg, spacing))


def test_reference_lbs_test_shape(mgpu):
    """tests/test_load_balance.cu:9-29: 200,030 items, segments of 100."""
    count, spacing = 200_030, 100
    seg = np.arange(0, count, spacing, dtype=np.int32)
    got = mgpu.load_balance_search(count, dev(seg)).cpu().numpy()
    assert np.array_equal(got, np.arange(count) // spacing)


@pytest.mark.parametrize("count,num_segments", [
    (10, 4), (1 << 20, 10_000), (3_000_001, 90_000), (5000, 200_000),
    (4096, 1), (4097, 2), (1, 1),
])
def test_seg_and_rank_match_oracle(mgpu, oracle, count, num_segments):
    rng = np.random.default_rng(count % 1000 + num_segments)
    seg = np.zeros(num_segments, dtype=np.int32)
    seg[1:] = np.sort(rng.integers(0, count + 1, size=num_segments - 1))
    got_seg, got_rank = mgpu.transform_lbs(count, dev(seg))
    want_seg, want_rank = oracle.load_balance_search(count, seg)
    assert mgpu.workspace_status() == 0
    assert np.array_equal(got_seg.cpu().numpy(), want_seg)
    assert np.array_equal(got_rank.cpu().numpy(), want_rank)


def test_unaligned_segments_pointer(mgpu, oracle):
    rng = np.random.default_rng(3)
    count, num_segments = 500_000, 7001
    seg = np.zeros(num_segments, dtype=np.int32)
    seg[1:] = np.sort(rng.integers(0, count + 1, size=num_segments - 1))
    buf = torch.zeros(num_segments + 4, dtype=torch.int32, device="cuda")
    view = buf[1:1 + num_segments]
    view.copy_(torch.from_numpy(seg))
    got_seg, got_rank = mgpu.transform_lbs(count, view)
    want_seg, want_rank = oracle.load_balance_search(count, seg)
    assert np.array_equal(got_seg.cpu().numpy(), want_seg)
    assert np.array_equal(got_rank.cpu().numpy(), want_rank)


@pytest.mark.parametrize("seg_shift,rank_shift", [(0, 0), (1, 1), (2, 3),
                                                  (3, 0), (0, 2)])
def test_outputs_at_every_alignment(mgpu, oracle, seg_shift, rank_shift):
    """A tile's ids and ranks leave shared memory by bulk copies of whole
    16-byte granules of the output arrays: the arrays may start anywhere in a
    granule, and the two arrays need not start at the same place in theirs."""
    rng = np.random.default_rng(seg_shift * 4 + rank_shift)
    count, num_segments = 777_777, 9001
    seg = np.zeros(num_segments, dtype=np.int32)
    seg[1:] = np.sort(rng.integers(0, count + 1, size=num_segments - 1))
    want_seg, want_rank = oracle.load_balance_search(count, seg)
    guard = -12345
    seg_buf = torch.full((count + 8,), guard, dtype=torch.int32, device="cuda")
    rank_buf = torch.full((count + 8,), guard, dtype=torch.int32, device="cuda")
    mgpu.transform_lbs(count, dev(seg),
                       out_seg=seg_buf[seg_shift:seg_shift + count],
                       out_rank=rank_buf[rank_shift:rank_shift + count])
    assert mgpu.workspace_status() == 0
    for buf, shift, want in ((seg_buf, seg_shift, want_seg),
                             (rank_buf, rank_shift, want_rank)):
        got = buf.cpu().numpy()
        assert np.array_equal(got[shift:shift + count], want)
        assert np.all(got[:shift] == guard) and np.all(got[shift + count:] == guard)
    ids_only = torch.full((count + 8,), guard, dtype=torch.int32, device="cuda")
    mgpu.transform_lbs(count, dev(seg), want_ranks=False,
                       out_seg=ids_only[rank_shift:rank_shift + count])
    got = ids_only.cpu().numpy()
    assert np.array_equal(got[rank_shift:rank_shift + count], want_seg)
    assert np.all(got[:rank_shift] == guard)
    assert np.all(got[rank_shift + count:] == guard)


@pytest.mark.parametrize("dtype,shift", [(torch.float32, 1), (torch.float32, 3),
                                         (torch.float64, 1), (torch.int64, 0)])
def test_interval_expand_unaligned_output(mgpu, oracle, dtype, shift):
    rng = np.random.default_rng(shift)
    count, num_segments = 600_001, 40_000
    seg = np.zeros(num_segments, dtype=np.int32)
    seg[1:] = np.sort(rng.integers(0, count + 1, size=num_segments - 1))
    vals = torch.from_numpy(rng.integers(1, 120, size=num_segments)).to(dtype)
    buf = torch.zeros(count + 8, dtype=dtype, device="cuda")
    mgpu.interval_expand(vals.cuda(), count, dev(seg),
                         out=buf[shift:shift + count])
    got = buf.cpu().numpy()
    want = oracle.interval_expand(vals.numpy(), count, seg)
    assert np.array_equal(got[shift:shift + count], want)
    assert np.all(got[:shift] == 0) and np.all(got[shift + count:] == 0)


@pytest.mark.parametrize("dtype", [torch.uint8, torch.int16, torch.float32,
                                   torch.float64, torch.int64])
def test_interval_expand(mgpu, oracle, dtype):
    rng = np.random.default_rng(9)
    count, num_segments = 1_000_000, 30_000
    seg = np.zeros(num_segments, dtype=np.int32)
    seg[1:] = np.sort(rng.integers(0, count + 1, size=num_segments - 1))
    vals = torch.from_numpy(rng.integers(0, 120, size=num_segments)).to(dtype)
    got = mgpu.interval_expand(vals.cuda(), count, dev(seg)).cpu().numpy()
    want = oracle.interval_expand(vals.numpy(), count, seg)
    assert np.array_equal(got, want)


def test_config4_reduced(mgpu, oracle):
    count, num_segments = 1 << 24, 1 << 18
    seg = workloads.config4(seed=3, count=count, num_segments=num_segments)
    got_seg, got_rank = mgpu.transform_lbs(count, seg)
    want_seg, want_rank = oracle.load_balance_search(count, seg.cpu().numpy())
    assert np.array_equal(got_seg.cpu().numpy(), want_seg)
    assert np.array_equal(got_rank.cpu().numpy(), want_rank)


def test_config4_full_size_properties(mgpu):
    """268,435,456 items over 4,194,304 Pareto-sized segments, checked on the
    device through properties that define the result uniquely:
    seg is non-decreasing, segments[seg] <= index < segments[seg + 1], and
    rank == index - segments[seg]."""
    count = 1 << 28
    seg = workloads.config4(seed=3)
    ids, rank = mgpu.transform_lbs(count, seg)
    assert mgpu.workspace_status() == 0
    index = torch.arange(count, device="cuda", dtype=torch.int32)
    starts = seg[ids.long()]
    assert bool((rank == index - starts).all())
    assert bool((rank >= 0).all())
    ends = torch.cat([seg[1:], torch.tensor([count], device="cuda",
                                            dtype=torch.int32)])[ids.long()]
    assert bool((index < ends).all())
    assert bool((ids[1:] >= ids[:-1]).all())


@pytest.mark.parametrize("dtype", [np.float32, np.float64])
@pytest.mark.parametrize("count,num_segments", [(0, 5), (1, 1), (1000, 37), (1_000_003, 30_011),
                                                (5_000_000, 11), (70_000, 200_000),
                                                (3_000_000, 500_000), (2_000_000, 250_000)])
def test_lbs_segreduce_weighted_is_exact_on_small_integers(mgpu, oracle, count, num_segments, dtype):
    """mgpu::lbs_segreduce through the C ABI (values[index] * weight cached per
    segment, plus, init 0). Small integer values and power-of-two weights keep
    every product and partial sum exact, so the result must equal the oracle's
    segment sums times the weights bit for bit. The shapes cover tiles whose
    segments' weights all fit the stage's slots (loaded once per segment),
    tiles with more segments than slots (gathered per item), and mixtures of
    both around the limits of 512 (fp32) and 256 (fp64) segments per tile."""
    rng = np.random.default_rng(count + num_segments)
    values = rng.integers(-8, 9, size=count).astype(dtype)
    seg = np.zeros(num_segments, dtype=np.int32)
    if num_segments > 1:
        seg[1:] = np.sort(rng.integers(0, count + 1, size=num_segments - 1))
    weights = (2.0 ** rng.integers(-2, 3, size=num_segments)).astype(dtype)
    got = mgpu.lbs_segreduce_weighted(torch.from_numpy(values).cuda(),
                                      torch.from_numpy(seg).cuda(),
                                      torch.from_numpy(weights).cuda()).cpu().numpy()
    sums = oracle.segreduce(values.astype(np.float64), seg, op="plus", init=0.0)
    assert np.array_equal(got.astype(np.float64), sums * weights)
    assert mgpu.workspace_status() == 0
