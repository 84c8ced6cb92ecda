"""mgpu::scan (plus) through the C ABI against numpy cumulative sums:
bit-exact for integers, tolerance for floating point."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


# 18,432 and 9,216 are the tile sizes of the streaming kernel (4- and 8-byte
# values); counts around them and their multiples exercise whole tiles, a
# tile with a ragged last 16-byte word, and the hand-over between tiles.
@pytest.mark.parametrize("count", [0, 1, 2, 3, 4, 5, 31, 4095, 4096, 4097,
                                   9215, 9216, 9217, 18431, 18432, 18433,
                                   55297, 1_000_003])
@pytest.mark.parametrize("dtype", [torch.int32, torch.int64])
def test_integer_scan_is_exact(mgpu, count, dtype):
    g = torch.Generator(device="cuda").manual_seed(count)
    x = torch.randint(-50, 50, (count,), device="cuda", generator=g).to(dtype)
    total = torch.full((1,), -1, dtype=dtype, device="cuda")
    exc = mgpu.scan(x, total=total).cpu().numpy()
    inc = mgpu.scan(x, inclusive=True).cpu().numpy()
    want = np.cumsum(x.cpu().numpy(), dtype=exc.dtype)
    assert np.array_equal(inc, want)
    assert np.array_equal(exc, want - x.cpu().numpy())
    assert int(total.item()) == (int(want[-1]) if count else 0)
    assert mgpu.workspace_status() == 0


def test_lengths_to_offsets_at_config2_size(mgpu):
    """8,388,608 segment lengths -> start offsets, as config 2 is built."""
    g = torch.Generator(device="cuda").manual_seed(1)
    lengths = torch.randint(0, 64, (1 << 23,), device="cuda", generator=g,
                            dtype=torch.int32)
    got = mgpu.scan(lengths)
    want = torch.cumsum(lengths, 0, dtype=torch.int32) - lengths
    assert torch.equal(got, want)


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-5), (torch.float64, 1e-12)])
def test_float_scan_within_tolerance(mgpu, dtype, tol):
    g = torch.Generator(device="cuda").manual_seed(9)
    x = torch.rand(3_000_000, device="cuda", generator=g, dtype=dtype) * 2 - 1
    got = mgpu.scan(x, inclusive=True).cpu().numpy().astype(np.float64)
    want = np.cumsum(x.cpu().numpy().astype(np.longdouble)).astype(np.float64)
    mags = np.cumsum(np.abs(x.cpu().numpy().astype(np.float64)))
    assert np.all(np.abs(got - want) <= tol * np.maximum(np.abs(want), mags))


def test_in_place(mgpu):
    x = torch.arange(100_000, dtype=torch.int64, device="cuda")
    want = torch.cumsum(x, 0)
    mgpu.scan(x, inclusive=True, out=x)
    assert torch.equal(x, want)


@pytest.mark.parametrize("offset", [1, 2, 3])
@pytest.mark.parametrize("dtype", [torch.int32, torch.int64])
def test_unaligned_arrays_take_the_generic_kernel(mgpu, offset, dtype):
    """Arrays that do not start on a 16-byte boundary cannot be moved by bulk
    copies; the call falls back to the generic kernel, same results."""
    g = torch.Generator(device="cuda").manual_seed(offset)
    base = torch.randint(-9, 9, (200_000 + 8,), device="cuda", generator=g).to(dtype)
    x = base[offset:offset + 200_000]
    out = torch.empty(200_000 + 8, dtype=dtype, device="cuda")[offset:offset + 200_000]
    mgpu.scan(x, inclusive=True, out=out)
    assert torch.equal(out, torch.cumsum(x, 0).to(dtype))


def test_large_scan_in_place_many_tiles(mgpu):
    """2^26 items in place: some 25 tiles per CTA of the persistent grid,
    every tile's carry from the look-back chain."""
    x = torch.ones(1 << 26, dtype=torch.int32, device="cuda")
    x[12345] = 7
    mgpu.scan(x, out=x)
    want = torch.arange(1 << 26, dtype=torch.int32, device="cuda")
    want[12346:] += 6
    assert torch.equal(x, want)
    assert mgpu.workspace_status() == 0
