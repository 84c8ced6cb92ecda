"""ctypes front end of the CPU oracle (oracle/oracle.c).

TEST INFRASTRUCTURE ONLY: imported by tests/, by the smoke check and by the
CPU-baseline leg of bench.py. The shipped package never imports this module.

Every function takes and returns numpy arrays. Semantics follow the reference's
own host checks (tests/test_segreduce.cu:40-49, tests/test_load_balance.cu:22-29)
and are documented next to each C function.
"""
import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "liboracle.so")

PLUS, MAX, MIN = 0, 1, 2
OPS = {"plus": PLUS, "max": MAX, "min": MIN}


def build(force=False):
    """Compile oracle.c into liboracle.so (no-op when it is up to date)."""
    src = os.path.join(_HERE, "oracle.c")
    if (not force and os.path.exists(_LIB_PATH)
            and os.path.getmtime(_LIB_PATH) >= os.path.getmtime(src)):
        return _LIB_PATH
    subprocess.check_call(["make", "-C", _HERE, "-B", "liboracle.so"],
                          stdout=subprocess.DEVNULL)
    return _LIB_PATH


_lib = None


def lib():
    global _lib
    if _lib is None:
        build()
        _lib = ctypes.CDLL(_LIB_PATH)
        _lib.oracle_merge_path_upper.restype = ctypes.c_int64
        _lib.oracle_load_balance_partitions.restype = ctypes.c_int
        _lib.oracle_max_threads.restype = ctypes.c_int
    return _lib


def max_threads():
    return int(lib().oracle_max_threads())


def _ptr(a):
    return a.ctypes.data_as(ctypes.c_void_p)


def _seg(segments):
    s = np.ascontiguousarray(segments, dtype=np.int32)
    return s


_SEGREDUCE = {
    np.dtype(np.int32): ("oracle_segreduce_i32", ctypes.c_int32),
    np.dtype(np.int64): ("oracle_segreduce_i64", ctypes.c_int64),
    np.dtype(np.float32): ("oracle_segreduce_f32", ctypes.c_float),
    np.dtype(np.float64): ("oracle_segreduce_f64", ctypes.c_double),
}


def segreduce(values, segments, op="plus", init=0, threads=1):
    """Host loop of tests/test_segreduce.cu:40-49 in the values' own type."""
    values = np.ascontiguousarray(values)
    seg = _seg(segments)
    name, ctype = _SEGREDUCE[values.dtype]
    out = np.empty(seg.size, dtype=values.dtype)
    getattr(lib(), name)(_ptr(values), ctypes.c_int64(values.size), _ptr(seg),
                         ctypes.c_int(seg.size), _ptr(out), ctype(init),
                         ctypes.c_int(OPS[op]), ctypes.c_int(threads))
    return out


def segsum_wide(values, segments, init=0.0, threads=1):
    """Plus-reduction accumulated in a wider type; returns (sums, magnitudes).
    threads > 1 spreads the segments over OpenMP threads."""
    values = np.ascontiguousarray(values)
    seg = _seg(segments)
    sums = np.empty(seg.size, dtype=np.float64)
    mags = np.empty(seg.size, dtype=np.float64)
    fn = {np.dtype(np.float32): lib().oracle_segsum_f32_wide,
          np.dtype(np.float64): lib().oracle_segsum_f64_wide}[values.dtype]
    fn(_ptr(values), ctypes.c_int64(values.size), _ptr(seg),
       ctypes.c_int(seg.size), _ptr(sums), _ptr(mags), ctypes.c_double(init),
       ctypes.c_int(threads))
    return sums, mags


def place_by_segments(values, segments, threads):
    """A copy of the float32 array `values` whose pages were first touched by
    the OpenMP threads that segreduce(..., threads=threads) will read them
    with (timing aid of the CPU baseline)."""
    values = np.ascontiguousarray(values, dtype=np.float32)
    seg = _seg(segments)
    placed = np.empty_like(values)
    lib().oracle_place_by_segments_f32(_ptr(values), ctypes.c_int64(values.size),
                                       _ptr(seg), ctypes.c_int(seg.size),
                                       _ptr(placed), ctypes.c_int(threads))
    return placed


def segreduce_index_mod(count, segments, init=-1, modulus=13):
    """The reference test's workload: plus-reduce (index % 13), init -1."""
    seg = _seg(segments)
    out = np.empty(seg.size, dtype=np.int32)
    lib().oracle_segreduce_index_mod(ctypes.c_int64(count), _ptr(seg),
                                     ctypes.c_int(seg.size), _ptr(out),
                                     ctypes.c_int32(init), ctypes.c_int(modulus))
    return out


def merge_path_upper(count, segments, diag):
    seg = _seg(segments)
    return int(lib().oracle_merge_path_upper(ctypes.c_int64(count), _ptr(seg),
                                             ctypes.c_int64(seg.size),
                                             ctypes.c_int64(diag)))


def load_balance_partitions(count, segments, spacing):
    seg = _seg(segments)
    n = (count + seg.size + spacing - 1) // spacing + 1
    out = np.empty(n, dtype=np.int32)
    got = lib().oracle_load_balance_partitions(ctypes.c_int64(count), _ptr(seg),
                                               ctypes.c_int(seg.size),
                                               ctypes.c_int(spacing), _ptr(out))
    assert got == n
    return out


def load_balance_search(count, segments):
    """Returns (seg, rank) per item."""
    seg = _seg(segments)
    seg_out = np.empty(count, dtype=np.int32)
    rank_out = np.empty(count, dtype=np.int32)
    lib().oracle_load_balance_search(ctypes.c_int64(count), _ptr(seg),
                                     ctypes.c_int(seg.size), _ptr(seg_out),
                                     _ptr(rank_out))
    return seg_out, rank_out


def interval_expand(values, count, segments):
    values = np.ascontiguousarray(values)
    seg = _seg(segments)
    out = np.zeros(count, dtype=values.dtype)
    lib().oracle_interval_expand(_ptr(values), ctypes.c_int(values.itemsize),
                                 ctypes.c_int64(count), _ptr(seg),
                                 ctypes.c_int(seg.size), _ptr(out))
    return out


def spmv(matrix, columns, x, row_starts):
    """Returns (y, magnitudes) accumulated wider than the matrix type."""
    matrix = np.ascontiguousarray(matrix)
    columns = np.ascontiguousarray(columns, dtype=np.int32)
    x = np.ascontiguousarray(x, dtype=matrix.dtype)
    rows = _seg(row_starts)
    y = np.empty(rows.size, dtype=np.float64)
    mags = np.empty(rows.size, dtype=np.float64)
    fn = {np.dtype(np.float32): lib().oracle_spmv_f32,
          np.dtype(np.float64): lib().oracle_spmv_f64}[matrix.dtype]
    fn(_ptr(matrix), _ptr(columns), _ptr(x), ctypes.c_int64(matrix.size),
       _ptr(rows), ctypes.c_int(rows.size), _ptr(y), _ptr(mags))
    return y, mags


def spmv_native_f32(matrix, columns, x, row_starts, threads=1):
    matrix = np.ascontiguousarray(matrix, dtype=np.float32)
    columns = np.ascontiguousarray(columns, dtype=np.int32)
    x = np.ascontiguousarray(x, dtype=np.float32)
    rows = _seg(row_starts)
    y = np.empty(rows.size, dtype=np.float32)
    lib().oracle_spmv_f32_native(_ptr(matrix), _ptr(columns), _ptr(x),
                                 ctypes.c_int64(matrix.size), _ptr(rows),
                                 ctypes.c_int(rows.size), _ptr(y),
                                 ctypes.c_int(threads))
    return y


def lbs_segreduce_seg_plus_rank(count, segments, init=-1):
    seg = _seg(segments)
    out = np.empty(seg.size, dtype=np.int32)
    lib().oracle_lbs_segreduce_seg_plus_rank(ctypes.c_int64(count), _ptr(seg),
                                             ctypes.c_int(seg.size), _ptr(out),
                                             ctypes.c_int32(init))
    return out


def lbs_segreduce_scaled(values, weights, segments, init=0.0):
    values = np.ascontiguousarray(values, dtype=np.float32)
    weights = np.ascontiguousarray(weights, dtype=np.float32)
    seg = _seg(segments)
    sums = np.empty(seg.size, dtype=np.float64)
    mags = np.empty(seg.size, dtype=np.float64)
    lib().oracle_lbs_segreduce_scaled_f32(_ptr(values), _ptr(weights),
                                          ctypes.c_int64(values.size), _ptr(seg),
                                          ctypes.c_int(seg.size), _ptr(sums),
                                          _ptr(mags), ctypes.c_double(init))
    return sums, mags
