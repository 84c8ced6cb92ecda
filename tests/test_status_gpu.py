"""Failure detection without faulting anything: a device-side wait that cannot
be satisfied runs out after its bound, the kernel records a status word and
returns, and the context keeps working."""
import ctypes
import time

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_lookback_wait_runs_out_and_reports(mgpu):
    lib = mgpu.load_library()
    tiles = 40                                  # more than one 32-tile window
    ws = torch.empty(tiles * 128 + 256, dtype=torch.uint8, device="cuda")
    status = ctypes.c_int(-1)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    t0 = time.perf_counter()
    code = lib.mgpu_b200_debug_lookback_timeout(
        ws.data_ptr(), tiles, ctypes.c_uint64(5_000_000), ctypes.byref(status),
        stream)
    elapsed = time.perf_counter() - t0
    assert code == 0                            # the look-back returned "nothing"
    assert status.value == 1                    # MGPU_B200_STATUS_LOOKBACK_TIMEOUT
    assert elapsed < 2.0                        # bounded: ~5 ms, not forever
    # The context is still usable and a normal call still succeeds.
    v = torch.arange(100_000, dtype=torch.int32, device="cuda")
    s = torch.arange(0, 100_000, 1000, dtype=torch.int32, device="cuda")
    out = mgpu.segreduce(v, s, init=0)
    want = v.view(100, 1000).sum(dim=1, dtype=torch.int32)
    assert torch.equal(out, want)
    assert mgpu.workspace_status() == 0


def test_wait_limit_hook_round_trips(mgpu):
    lib = mgpu.load_library()
    old = lib.mgpu_b200_debug_set_wait_limit_ns(123456789)
    assert lib.mgpu_b200_debug_set_wait_limit_ns(0) == 123456789
    assert lib.mgpu_b200_debug_set_wait_limit_ns(old) > 0
