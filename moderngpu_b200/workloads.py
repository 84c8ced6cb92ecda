"""Seeded synthetic inputs with the shapes and value distributions of the five
benchmark configurations (the reference measures on no public data set; its
tests build segment offsets from a seeded generator, tests/test_segreduce.cu:
16-22, and these generators follow that convention: `segments` holds START
offsets, segments[0] == 0, non-decreasing, values <= count, empty segments
allowed).

Small cases are generated with numpy on the host; the full-size cases are
generated with torch directly on the device so that no multi-gigabyte array
crosses PCIe. Every generator is deterministic in (seed, size).
"""
import math

import numpy as np
import torch


def offsets_from_lengths(lengths, count):
    """Exclusive scan of segment lengths, clipped to `count`.

    Overshoot gives trailing empty segments; undershoot leaves the remainder
    to the last segment (which by convention ends at count)."""
    if isinstance(lengths, np.ndarray):
        starts = np.zeros(lengths.size, dtype=np.int64)
        np.cumsum(lengths[:-1], out=starts[1:])
        return np.minimum(starts, count).astype(np.int32)
    starts = torch.cumsum(lengths.to(torch.int64), 0) - lengths.to(torch.int64)
    return torch.clamp(starts, max=count).to(torch.int32)


# --------------------------------------------------------------------------
# Config 1: int32 plus, 1,048,576 items in [0, 100), 10,000 segments from
# sorted uniform-random offsets (offset[0] = 0, empty segments allowed).

def config1(seed=0, count=1 << 20, num_segments=10_000):
    rng = np.random.default_rng(seed)
    values = rng.integers(0, 100, size=count, dtype=np.int32)
    segments = np.zeros(num_segments, dtype=np.int32)
    if num_segments > 1:
        segments[1:] = np.sort(rng.integers(0, count + 1, size=num_segments - 1))
    return values, segments


# --------------------------------------------------------------------------
# Config 2: fp32 plus, 268,435,456 items uniform in [-1, 1), 8,388,608
# segments with geometric lengths (mean 32) and 5 % zero-length segments.

def config2_lengths(num_segments, generator, device, mean=32.0, p_empty=0.05):
    p = (1.0 - p_empty) / mean           # geometric on {1, 2, ...}, mean 1/p
    lengths = torch.empty(num_segments, device=device).geometric_(
        p, generator=generator)
    empty = torch.rand(num_segments, device=device, generator=generator) < p_empty
    return torch.where(empty, torch.zeros_like(lengths), lengths).to(torch.int64)


def config2(seed=1, count=1 << 28, num_segments=1 << 23, device="cuda",
            dtype=torch.float32):
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    values = torch.rand(count, device=device, generator=g, dtype=dtype) * 2 - 1
    lengths = config2_lengths(num_segments, g, device,
                              mean=count / num_segments)
    segments = offsets_from_lengths(lengths, count)
    return values, segments


# --------------------------------------------------------------------------
# Config 3: CSR spmv fp32, 16,777,216 rows, row lengths Zipf(alpha = 1.5) on
# {1..4096} thinned with empty rows so that the mean is about 16 non-zeros,
# column indices uniform, values and x uniform in [-1, 1).

def zipf_table(alpha=1.5, kmax=4096):
    k = np.arange(1, kmax + 1, dtype=np.float64)
    pmf = k ** (-alpha)
    pmf /= pmf.sum()
    return np.cumsum(pmf), float((k * pmf).sum())


def config3(seed=2, rows=1 << 24, cols=None, mean_nnz=16.0, device="cuda",
            dtype=torch.float32, max_nnz=(1 << 31) - (1 << 25)):
    cols = rows if cols is None else cols
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    cdf, zipf_mean = zipf_table()
    p_empty = max(0.0, 1.0 - mean_nnz / zipf_mean)
    u = torch.rand(rows, device=device, generator=g, dtype=torch.float64)
    cdf_t = torch.from_numpy(cdf).to(device)
    lengths = torch.searchsorted(cdf_t, u).clamp_(max=cdf.size - 1) + 1
    empty = torch.rand(rows, device=device, generator=g) < p_empty
    lengths = torch.where(empty, torch.zeros_like(lengths), lengths)
    nnz = int(lengths.sum().item())
    nnz = min(nnz, max_nnz - rows)
    row_starts = offsets_from_lengths(lengths, nnz)
    matrix = torch.rand(nnz, device=device, generator=g, dtype=dtype) * 2 - 1
    columns = torch.randint(0, cols, (nnz,), device=device, generator=g,
                            dtype=torch.int32)
    x = torch.rand(cols, device=device, generator=g, dtype=dtype) * 2 - 1
    return matrix, columns, x, row_starts


# --------------------------------------------------------------------------
# Config 4: load-balancing search, 268,435,456 items over 4,194,304 segments
# whose sizes follow a Pareto(alpha = 1.2) law scaled to the total.

def config4(seed=3, count=1 << 28, num_segments=1 << 22, device="cuda",
            alpha=1.2):
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    u = torch.rand(num_segments, device=device, generator=g,
                   dtype=torch.float64).clamp_(min=1e-12)
    pareto = u ** (-1.0 / alpha)
    lengths = torch.floor(pareto * (count / pareto.sum())).to(torch.int64)
    return offsets_from_lengths(lengths, count)


# --------------------------------------------------------------------------
# Config 5: fp64 max / plus, items uniform in [-1e6, 1e6), log-normal segment
# lengths (mu = 3, sigma = 1.5): many segments straddle shard boundaries.
# `count` items are generated for ONE shard; a shard's first segment start is
# usually > 0, i.e. its leading items continue the previous shard's last
# segment.

def config5_shard(seed, shard, count, mean_scale=1.0, device="cuda",
                  dtype=torch.float64):
    g = torch.Generator(device=device)
    g.manual_seed(seed * 1000003 + shard)
    values = (torch.rand(count, device=device, generator=g, dtype=dtype) * 2 - 1) * 1e6
    expected = math.exp(3 + 1.5 * 1.5 / 2) * mean_scale
    n = int(count / expected * 1.05) + 16
    z = torch.randn(n, device=device, generator=g, dtype=torch.float64)
    lengths = torch.floor(torch.exp(3 + 1.5 * z) * mean_scale).to(torch.int64)
    starts = torch.cumsum(lengths, 0) - lengths
    # A random lead-in: the first local segment starts after a few items that
    # belong to the previous shard's last segment (shard 0 starts at 0).
    lead = 0 if shard == 0 else int(torch.randint(
        1, 200, (1,), generator=g, device=device).item())
    starts = starts + lead
    starts = starts[starts <= count]
    return values, starts.to(torch.int32)


def segreduce_bytes(count, num_segments, elem_bytes):
    """Algorithmic HBM bytes of one segreduce call: every item read once,
    every offset read once, every result written once."""
    return count * elem_bytes + num_segments * 4 + num_segments * elem_bytes


def lbs_bytes(count, num_segments, with_ranks=True):
    return num_segments * 4 + count * 4 * (2 if with_ranks else 1)


def spmv_bytes(nnz, rows, cols, elem_bytes):
    return nnz * (elem_bytes + 4) + rows * 4 + rows * elem_bytes + cols * elem_bytes
