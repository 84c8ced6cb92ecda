"""mgpu::sorted_search through the C ABI against numpy.searchsorted:
bit-exact lower and upper bounds, duplicates, needles or haystack much longer
than the other, empty haystack."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype", [np.int32, np.int64, np.float32, np.float64])
@pytest.mark.parametrize("shape", [(1, 1, 5), (1000, 1000, 10_000), (300_007, 70_001, 5_000),
                                   (5, 400_000, 1_000_000), (250_000, 3, 50),
                                   (100_000, 100_000, 7), (12_345, 0, 100)])
def test_bounds_match_searchsorted(mgpu, dtype, shape):
    num_needles, num_haystack, key_range = shape
    rng = np.random.default_rng(num_needles + num_haystack)
    needles = np.sort(rng.integers(0, key_range + 1, num_needles)).astype(dtype)
    haystack = np.sort(rng.integers(0, key_range + 1, num_haystack)).astype(dtype)
    n = torch.from_numpy(needles).cuda()
    h = torch.from_numpy(haystack).cuda()
    lower = mgpu.sorted_search(n, h).cpu().numpy()
    upper = mgpu.sorted_search(n, h, upper=True).cpu().numpy()
    assert np.array_equal(lower, np.searchsorted(haystack, needles, side="left"))
    assert np.array_equal(upper, np.searchsorted(haystack, needles, side="right"))


@pytest.mark.parametrize("shift_needles,shift_haystack", [(1, 0), (0, 3), (2, 1)])
def test_unaligned_arrays_and_ragged_ends(mgpu, shift_needles, shift_haystack):
    """Arrays that do not start on a 16-byte boundary take the kernel without
    bulk copies; lengths that are not a multiple of four exercise the ragged
    last granule of the one with them."""
    rng = np.random.default_rng(shift_needles * 10 + shift_haystack)
    needles = np.sort(rng.integers(0, 50_000, 200_003)).astype(np.int32)
    haystack = np.sort(rng.integers(0, 50_000, 150_001)).astype(np.int32)
    n = torch.from_numpy(needles).cuda()[shift_needles:]
    h = torch.from_numpy(haystack).cuda()[shift_haystack:]
    for upper, side in ((False, "left"), (True, "right")):
        got = mgpu.sorted_search(n, h, upper=upper).cpu().numpy()
        want = np.searchsorted(haystack[shift_haystack:], needles[shift_needles:], side=side)
        assert np.array_equal(got, want)
    # Aligned starts, ragged ends.
    got = mgpu.sorted_search(torch.from_numpy(needles).cuda(),
                             torch.from_numpy(haystack).cuda()).cpu().numpy()
    assert np.array_equal(got, np.searchsorted(haystack, needles, side="left"))
