"""mgpu_b200_segreduce_static: the entry point for callers that cannot
allocate device memory at the point of the call (inside a region where the
allocator is off limits, or behind a binding that only forwards the caller's
input and output pointers). Its scratch is a fixed 4 MiB block inside the
library instead of a caller-supplied workspace.

Checked here, through the C ABI: two calls in a row give the same results as
mgpu_b200_segreduce on the same inputs (the second call finds the first
call's leftovers in the shared block), and a problem too large for the block
is refused before anything runs. This file sorts last on purpose, so a run
that stops at the first failure has already run every other test."""
import ctypes

import numpy as np
import pytest
import torch

from moderngpu_b200 import workloads

pytestmark = pytest.mark.gpu

FP32_TOL = 1e-5


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def test_two_calls_in_a_row_match_the_workspace_entry_point(mgpu):
    values, seg = workloads.config1(seed=2)
    v, s = dev(values), dev(seg)
    want = mgpu.segreduce(v, s, op="plus", init=-1)
    out = torch.empty_like(want)              # preallocated by the caller
    first = mgpu.segreduce_static(v, s, op="plus", init=-1, out=out).clone()
    second = mgpu.segreduce_static(v, s, op="plus", init=-1, out=out)
    torch.cuda.synchronize()
    assert torch.equal(first, want)           # int32: bit-exact
    assert torch.equal(second, want)


def test_different_problem_after_leftovers_fp32_and_int64(mgpu, oracle):
    """A float problem, then an int64 max problem of another shape: each call
    starts from whatever the previous one left in the shared block."""
    fv, fs = workloads.config2(seed=5, count=1 << 22, num_segments=1 << 17)
    want = mgpu.segreduce(fv, fs, op="plus", init=0.0)
    for _ in range(2):
        got = mgpu.segreduce_static(fv, fs, op="plus", init=0.0)
        sums, mags = oracle.segsum_wide(fv.cpu().numpy(), fs.cpu().numpy())
        bound = FP32_TOL * np.maximum(np.abs(sums), mags)
        assert np.all(np.abs(got.cpu().numpy() - sums) <= bound)
        assert np.all(np.abs(got.cpu().numpy() - want.cpu().numpy()) <= 2 * bound)
    rng = np.random.default_rng(8)
    iv = dev(rng.integers(-10**12, 10**12, size=3_000_000))
    seg = np.zeros(1000, dtype=np.int32)
    seg[1:] = np.sort(rng.integers(0, 3_000_001, size=999))
    want = mgpu.segreduce(iv, dev(seg), op="max", init=-5)
    for _ in range(2):
        assert torch.equal(mgpu.segreduce_static(iv, dev(seg), op="max",
                                                 init=-5), want)


def test_too_large_for_the_block_is_refused_without_launching(mgpu):
    lib = mgpu.load_library()
    assert lib.mgpu_b200_static_scratch_bytes() == 4 << 20
    init = ctypes.c_double(0)
    # fp64, 1.5e9 items: needs far more than 4 MiB of scratch. All pointers
    # are NULL: the size check comes first, nothing can be dereferenced.
    code = lib.mgpu_b200_segreduce_static(1, 0, None, 1_500_000_000, None,
                                          1_000_000, None, ctypes.byref(init),
                                          None)
    assert code == 2                          # MGPU_B200_E_WORKSPACE
    assert b"workspace" in lib.mgpu_b200_error_string(code)
    # Beyond the library's overall 32-bit size limit: refused the same way.
    code = lib.mgpu_b200_segreduce_static(0, 0, None, 2**31 - 1, None, 2**20,
                                          None, ctypes.byref(init), None)
    assert code == 2


def test_largest_problem_that_fits_runs_and_the_next_tile_is_refused(mgpu):
    """At the boundary the header documents: 227,494,680 fp32 items + segments
    use the whole 4 MiB block and reduce correctly; one more element needs
    another tile and is refused."""
    lib = mgpu.load_library()
    limit = 227_494_680
    num_segments = 1 << 20
    count = limit - num_segments
    assert lib.mgpu_b200_segreduce_workspace_bytes(0, count, num_segments) \
        == 4 << 20
    g = torch.Generator(device="cuda").manual_seed(3)
    values = torch.randint(-8, 9, (count,), device="cuda", generator=g,
                           dtype=torch.int32).to(torch.float32)
    seg = (torch.arange(num_segments, device="cuda", dtype=torch.int64)
           * (count // num_segments)).to(torch.int32)
    got = mgpu.segreduce_static(values, seg, op="plus", init=0.0)
    want = mgpu.segreduce(values, seg, op="plus", init=0.0)
    torch.cuda.synchronize()
    # Small integers in fp32: every order of summation gives the same bits.
    assert torch.equal(got, want)
    sums = torch.zeros(num_segments, dtype=torch.float64, device="cuda")
    ids = torch.clamp(torch.arange(count, device="cuda") //
                      (count // num_segments), max=num_segments - 1)
    sums.index_add_(0, ids, values.double())
    assert torch.equal(got.double(), sums)
    init = ctypes.c_float(0)
    code = lib.mgpu_b200_segreduce_static(
        0, 0, values.data_ptr(), count + 1, seg.data_ptr(), num_segments,
        got.data_ptr(), ctypes.byref(init), None)
    assert code == 2                          # MGPU_B200_E_WORKSPACE
