"""Pins the CPU oracle (oracle/oracle.c) against
 - golden vectors produced by the reference's own host-callable merge_path
   (tests/golden/lbs_partitions.json, generator oracle/ref_host_golden.cu),
 - closed-form answers for the workload of the reference's segreduce test
   (tests/test_segreduce.cu:31-49: plus-reduce index % 13, init -1),
 - independent numpy formulations.
No GPU needed."""
import json
import os

import numpy as np
import pytest

GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "lbs_partitions.json")


def golden_cases():
    with open(GOLDEN) as f:
        return json.load(f)["cases"]


@pytest.mark.parametrize("case", golden_cases(), ids=lambda c: c["name"])
def test_partitions_match_reference_merge_path(oracle, case):
    seg = np.array(case["segments"], dtype=np.int32)
    for spacing, expect in case["partitions"].items():
        got = oracle.load_balance_partitions(case["count"], seg, int(spacing))
        assert got.tolist() == expect


@pytest.mark.parametrize("case", golden_cases(), ids=lambda c: c["name"])
def test_lbs_matches_reference_merge_order(oracle, case):
    """Spacing-1 partitions spell out the whole merge order: item i sits on
    the diagonal d where the item count steps from i to i + 1, and d - i
    segment starts precede it."""
    if "1" not in case["partitions"]:
        pytest.skip("no spacing-1 golden for this case")
    count = case["count"]
    seg = np.array(case["segments"], dtype=np.int32)
    mp = np.array(case["partitions"]["1"], dtype=np.int64)
    step = np.nonzero(np.diff(mp) == 1)[0]          # diagonals holding an item
    assert step.size == count
    expect_seg = (step - np.arange(count)) - 1
    got_seg, got_rank = oracle.load_balance_search(count, seg)
    assert got_seg.tolist() == expect_seg.tolist()
    assert got_rank.tolist() == (np.arange(count) - seg[expect_seg]).tolist() \
        if count else True


def closed_form_index_mod(begin, end, modulus=13):
    """sum of (i % modulus) for i in [begin, end)."""
    def prefix(n):      # sum over [0, n)
        q, r = divmod(n, modulus)
        return q * (modulus * (modulus - 1) // 2) + r * (r - 1) // 2
    return prefix(end) - prefix(begin)


@pytest.mark.parametrize("seed", [0, 1, 2, 3])
def test_segreduce_index_mod_closed_form(oracle, seed):
    # Shape of tests/test_segreduce.cu:67-71 scaled down 100x.
    count, num_segments = 1_000_000, 10
    rng = np.random.default_rng(seed)
    seg = np.zeros(num_segments, dtype=np.int32)
    seg[1:] = np.sort(rng.integers(0, count + 1, size=num_segments - 1))
    if seed == 3:           # force empty segments, including trailing ones
        seg[4] = seg[3]
        seg[-1] = count
    got = oracle.segreduce_index_mod(count, seg, init=-1, modulus=13)
    for s in range(num_segments):
        b = int(seg[s])
        e = int(seg[s + 1]) if s + 1 < num_segments else count
        want = closed_form_index_mod(b, e) if e > b else -1
        assert int(got[s]) == want


@pytest.mark.parametrize("dtype", [np.int32, np.int64, np.float32, np.float64])
@pytest.mark.parametrize("op", ["plus", "max", "min"])
def test_segreduce_matches_numpy(oracle, dtype, op):
    rng = np.random.default_rng(7)
    count, num_segments = 5000, 300
    if np.issubdtype(dtype, np.integer):
        values = rng.integers(-50, 50, size=count).astype(dtype)
    else:
        values = rng.integers(-50, 50, size=count).astype(dtype) / 4
    seg = np.zeros(num_segments, dtype=np.int32)
    seg[1:] = np.sort(rng.integers(0, count + 1, size=num_segments - 1))
    got = oracle.segreduce(values, seg, op=op, init=-7)
    fn = {"plus": np.sum, "max": np.max, "min": np.min}[op]
    ends = np.append(seg[1:], count)
    for s in range(num_segments):
        chunk = values[seg[s]:ends[s]]
        want = fn(chunk) if chunk.size else -7
        assert got[s] == dtype(want)


def test_init_only_for_empty_segments(oracle):
    values = np.array([5, 6, 7], dtype=np.int32)
    seg = np.array([0, 0, 2, 3, 3], dtype=np.int32)
    got = oracle.segreduce(values, seg, op="plus", init=-1)
    assert got.tolist() == [-1, 11, 7, -1, -1]


def test_threaded_oracle_equals_serial(oracle):
    rng = np.random.default_rng(11)
    values = rng.standard_normal(200_000).astype(np.float32)
    seg = np.zeros(9000, dtype=np.int32)
    seg[1:] = np.sort(rng.integers(0, values.size + 1, size=seg.size - 1))
    a = oracle.segreduce(values, seg, threads=1)
    b = oracle.segreduce(values, seg, threads=max(2, oracle.max_threads()))
    assert np.array_equal(a, b)


def test_wide_sum_and_magnitude(oracle):
    values = np.array([1.5, -2.5, 4.0, 8.0], dtype=np.float32)
    seg = np.array([0, 2, 2], dtype=np.int32)
    sums, mags = oracle.segsum_wide(values, seg, init=9.0)
    assert sums.tolist() == [-1.0, 9.0, 12.0]
    assert mags.tolist() == [4.0, 0.0, 12.0]


def test_interval_expand_and_spmv(oracle):
    seg = np.array([0, 2, 2, 5], dtype=np.int32)
    vals = np.array([10, 20, 30, 40], dtype=np.int64)
    out = oracle.interval_expand(vals, 7, seg)
    assert out.tolist() == [10, 10, 30, 30, 30, 40, 40]
    matrix = np.array([1, 2, 3, 4, 5], dtype=np.float32)
    cols = np.array([0, 1, 1, 2, 0], dtype=np.int32)
    x = np.array([1, 10, 100], dtype=np.float32)
    rows = np.array([0, 2, 2, 4], dtype=np.int32)
    y, mag = oracle.spmv(matrix, cols, x, rows)
    assert y.tolist() == [21.0, 0.0, 430.0, 5.0]
    assert oracle.spmv_native_f32(matrix, cols, x, rows).tolist() == \
        [21.0, 0.0, 430.0, 5.0]


def test_lbs_segreduce_functors(oracle):
    seg = np.array([0, 3, 3, 4], dtype=np.int32)
    out = oracle.lbs_segreduce_seg_plus_rank(6, seg, init=-1)
    # seg 0: 0+0,0+1,0+2 ; seg 1: empty ; seg 2: 2+0 ; seg 3: 3+0, 3+1
    assert out.tolist() == [3, -1, 2, 7]
