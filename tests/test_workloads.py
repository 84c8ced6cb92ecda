"""Invariants of the synthetic input generators (host side, numpy / CPU torch)."""
import numpy as np
import torch

from moderngpu_b200 import workloads


def check_offsets(seg, count):
    seg = np.asarray(seg)
    assert seg[0] == 0
    assert np.all(np.diff(seg.astype(np.int64)) >= 0)
    assert seg[-1] <= count


def test_config1_shape_and_determinism():
    v, s = workloads.config1(seed=5)
    v2, s2 = workloads.config1(seed=5)
    assert v.size == 1 << 20 and s.size == 10_000
    assert np.array_equal(v, v2) and np.array_equal(s, s2)
    assert v.min() >= 0 and v.max() < 100
    check_offsets(s, v.size)


def test_config2_small_on_cpu():
    v, s = workloads.config2(seed=1, count=1 << 16, num_segments=1 << 11,
                             device="cpu")
    assert v.dtype == torch.float32 and float(v.min()) >= -1 and float(v.max()) < 1
    check_offsets(s.numpy(), v.numel())
    lengths = np.diff(np.append(s.numpy(), v.numel()))
    assert 0.02 < np.mean(lengths == 0) < 0.10
    assert 20 < lengths.mean() < 48


def test_config3_small_on_cpu():
    m, c, x, r = workloads.config3(seed=2, rows=1 << 12, device="cpu")
    assert m.numel() == c.numel()
    check_offsets(r.numpy(), m.numel())
    assert int(c.min()) >= 0 and int(c.max()) < x.numel()
    mean = m.numel() / r.numel()
    assert 8 < mean < 32


def test_config4_small_on_cpu():
    s = workloads.config4(seed=3, count=1 << 16, num_segments=1 << 10,
                          device="cpu")
    check_offsets(s.numpy(), 1 << 16)


def test_config5_shard_on_cpu():
    v0, s0 = workloads.config5_shard(4, 0, 1 << 14, device="cpu")
    v1, s1 = workloads.config5_shard(4, 1, 1 << 14, device="cpu")
    assert v0.dtype == torch.float64
    assert int(s0[0]) == 0 and int(s1[0]) > 0
    assert int(s1[-1]) <= v1.numel()


def test_algorithmic_bytes():
    assert workloads.segreduce_bytes(1 << 28, 1 << 23, 4) == 1_140_850_688
    assert workloads.segreduce_bytes(1 << 20, 10_000, 4) == 4_274_304
    assert workloads.lbs_bytes(1 << 28, 1 << 22) == 2_164_260_864
