"""The C-ABI library loads and exports every entry point that
include/moderngpu_b200.h declares; argument validation that needs no GPU
behaves as documented. No compute call is made here."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "moderngpu_b200.h")


def declared_symbols():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(mgpu_b200_\w+)\s*\(", text)))


def test_header_declares_entry_points():
    names = declared_symbols()
    for expected in ["mgpu_b200_segreduce", "mgpu_b200_spmv",
                     "mgpu_b200_load_balance_search",
                     "mgpu_b200_load_balance_partitions",
                     "mgpu_b200_interval_expand", "mgpu_b200_segreduce_host",
                     "mgpu_b200_workspace_status"]:
        assert expected in names


def test_library_exports_every_declared_symbol(mgpu):
    lib = mgpu.load_library()
    for name in declared_symbols():
        assert hasattr(lib, name), "missing export: " + name


def test_version_and_error_strings(mgpu):
    lib = mgpu.load_library()
    assert lib.mgpu_b200_version() >= 100
    assert lib.mgpu_b200_error_string(0) == b"success"
    assert b"workspace" in lib.mgpu_b200_error_string(2)


def test_workspace_size_is_host_only_and_monotone(mgpu):
    lib = mgpu.load_library()
    small = lib.mgpu_b200_segreduce_workspace_bytes(0, 1000, 10)
    large = lib.mgpu_b200_segreduce_workspace_bytes(0, 1 << 28, 1 << 23)
    assert 0 < small < large < (64 << 20)
    # Size limit of the 32-bit index space.
    assert lib.mgpu_b200_segreduce_workspace_bytes(0, 2**31 - 1, 2**20) == 0
    assert lib.mgpu_b200_segreduce_workspace_bytes(99, 10, 10) == 0


def test_invalid_arguments_are_rejected_before_any_launch(mgpu):
    lib = mgpu.load_library()
    init = ctypes.c_float(0)
    E_INVALID = 1
    # negative count
    assert lib.mgpu_b200_segreduce(0, 0, None, -1, None, 0, None,
                                   ctypes.byref(init), None, 0, None) == E_INVALID
    # null init
    assert lib.mgpu_b200_segreduce(0, 0, None, 0, None, 0, None, None, None,
                                   0, None) == E_INVALID
    # items but no input pointer
    assert lib.mgpu_b200_segreduce(0, 0, None, 10, None, 1, None,
                                   ctypes.byref(init), None, 0, None) == E_INVALID
    # empty problem is a no-op
    assert lib.mgpu_b200_segreduce(0, 0, None, 0, None, 0, None,
                                   ctypes.byref(init), None, 0, None) == 0
    assert lib.mgpu_b200_load_balance_partitions(10, None, 0, 0, None,
                                                 None) == E_INVALID


def test_static_scratch_capacity_matches_the_header(mgpu):
    """The limits include/moderngpu_b200.h states for
    mgpu_b200_segreduce_static: the block is 4 MiB, 2^27 items fit, 2^28 do
    not, and the largest sizes that fit are the ones written there. Host-side
    arithmetic only (sizes are checked before any pointer is used)."""
    lib = mgpu.load_library()
    lib.mgpu_b200_static_scratch_bytes.restype = ctypes.c_size_t
    cap = lib.mgpu_b200_static_scratch_bytes()
    assert cap == 4 << 20
    need = lib.mgpu_b200_segreduce_workspace_bytes
    assert need(0, 1 << 27, 1 << 22) <= cap
    assert need(0, 1 << 28, 1 << 23) > cap
    header = open(HEADER).read()
    for dtype, limit in ((0, 227_494_680), (2, 227_494_680),
                         (1, 211_226_904), (3, 211_226_904)):
        assert need(dtype, limit, 0) <= cap < need(dtype, limit + 1, 0)
        assert "{:,}".format(limit) in header
    init = ctypes.c_float(0)
    E_WORKSPACE = 2
    # One element beyond the limit is refused before any pointer is touched.
    assert lib.mgpu_b200_segreduce_static(
        0, 0, None, 227_494_681, None, 0, None, ctypes.byref(init),
        None) == E_WORKSPACE
    assert lib.mgpu_b200_segreduce_static(
        1, 0, None, 211_226_000, None, 905, None, ctypes.byref(init),
        None) == E_WORKSPACE


def test_missing_library_fails_loudly(monkeypatch):
    import moderngpu_b200.binding as binding
    monkeypatch.setattr(binding, "_lib", None)
    monkeypatch.setattr(binding, "_LIB_PATH", "/nonexistent/libmgpu_b200.so")
    with pytest.raises(binding.LibraryMissing):
        binding.load_library()
