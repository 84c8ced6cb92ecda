"""CSR spmv parity: fp32 / fp64 products summed per row, compared with a
wider host accumulation (tolerance 1e-5 / 1e-12 of max(|y|, sum |a x|))."""
import numpy as np
import pytest
import torch

from moderngpu_b200 import workloads

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-5),
                                       (torch.float64, 1e-12)])
def test_config3_reduced(mgpu, oracle, dtype, tol):
    m, c, x, r = workloads.config3(seed=2, rows=1 << 18, dtype=dtype)
    y = mgpu.spmv(m, c, x, r).cpu().numpy().astype(np.float64)
    want, mags = oracle.spmv(m.cpu().numpy(), c.cpu().numpy(), x.cpu().numpy(),
                             r.cpu().numpy())
    assert mgpu.workspace_status() == 0
    assert np.all(np.abs(y - want) <= tol * np.maximum(np.abs(want), mags))


def test_integer_valued_spmv_is_exact(mgpu, oracle):
    rows, cols = 50_000, 4096
    g = torch.Generator(device="cuda").manual_seed(7)
    lengths = torch.randint(0, 40, (rows,), device="cuda", generator=g)
    nnz = int(lengths.sum())
    r = workloads.offsets_from_lengths(lengths, nnz)
    m = torch.randint(-4, 5, (nnz,), device="cuda", generator=g).float()
    c = torch.randint(0, cols, (nnz,), device="cuda", generator=g, dtype=torch.int32)
    x = torch.randint(-4, 5, (cols,), device="cuda", generator=g).float()
    y = mgpu.spmv(m, c, x, r).cpu().numpy()
    want = oracle.spmv_native_f32(m.cpu().numpy(), c.cpu().numpy(),
                                  x.cpu().numpy(), r.cpu().numpy())
    assert np.array_equal(y, want)


def test_config3_full_size(mgpu, oracle):
    m, c, x, r = workloads.config3(seed=2)
    y = mgpu.spmv(m, c, x, r)
    assert mgpu.workspace_status() == 0
    # Linearity in x is exact for a power-of-two factor.
    y2 = mgpu.spmv(m, c, x * 2, r)
    assert torch.equal(y2, y * 2)
    want, mags = oracle.spmv(m.cpu().numpy(), c.cpu().numpy(), x.cpu().numpy(),
                             r.cpu().numpy())
    err = np.abs(y.cpu().numpy().astype(np.float64) - want)
    assert np.all(err <= 1e-5 * np.maximum(np.abs(want), mags))


def test_l2_pin_leaves_results_unchanged(mgpu):
    """mgpu_b200_l2_pin / _unpin only change where the vector's lines live:
    the product is bit-identical with and without the pin, and a second
    pin/unpin cycle works."""
    g = torch.Generator(device="cuda").manual_seed(3)
    rows, per_row = 200_000, 9
    nnz = rows * per_row
    m = torch.rand(nnz, device="cuda", generator=g) * 2 - 1
    c = torch.randint(0, rows, (nnz,), device="cuda", generator=g, dtype=torch.int32)
    x = torch.rand(rows, device="cuda", generator=g) * 2 - 1
    r = torch.arange(0, nnz, per_row, device="cuda", dtype=torch.int32)
    plain = mgpu.spmv(m, c, x, r).clone()
    for _ in range(2):
        mgpu.l2_pin(x)
        pinned = mgpu.spmv(m, c, x, r).clone()
        mgpu.l2_unpin()
        assert torch.equal(plain, pinned)
    assert torch.equal(plain, mgpu.spmv(m, c, x, r))
