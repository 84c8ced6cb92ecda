"""ctypes binding of libmgpu_b200.so; function names follow the reference's
entry points (src/moderngpu/kernel_segreduce.hxx, kernel_load_balance.hxx,
kernel_intervalmove.hxx, search.hxx).

All tensor arguments are torch CUDA tensors; work is enqueued on torch's
current stream of the tensors' device. Results are torch tensors.
"""
import ctypes
import os

import torch

_PKG_DIR = os.path.dirname(os.path.abspath(__file__))
# MGPU_B200_LIBRARY names another build of the library to load instead of the
# in-tree one (comparing two builds on one machine).
_LIB_PATH = os.environ.get("MGPU_B200_LIBRARY") or os.path.join(
    _PKG_DIR, "lib", "libmgpu_b200.so")

F32, F64, I32, I64 = 0, 1, 2, 3
PLUS, MAX, MIN = 0, 1, 2
_OPS = {"plus": PLUS, "max": MAX, "maximum": MAX, "min": MIN, "minimum": MIN}
_DTYPES = {torch.float32: F32, torch.float64: F64, torch.int32: I32,
           torch.int64: I64}
_CTYPES = {torch.float32: ctypes.c_float, torch.float64: ctypes.c_double,
           torch.int32: ctypes.c_int32, torch.int64: ctypes.c_int64}


class LibraryMissing(RuntimeError):
    """libmgpu_b200.so is not built or cannot be loaded."""


class MgpuError(RuntimeError):
    """A library call returned a non-zero code."""

    def __init__(self, code, text):
        super().__init__("mgpu_b200 error %d: %s" % (code, text))
        self.code = code


_lib = None


def lib_path():
    return _LIB_PATH


def load_library():
    """Load (once) and return the ctypes handle; raises LibraryMissing."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(_LIB_PATH):
        raise LibraryMissing(
            "%s not found: build it with `python -m moderngpu_b200.build` "
            "(there is no CPU fallback)" % _LIB_PATH)
    try:
        lib = ctypes.CDLL(_LIB_PATH)
    except OSError as e:
        raise LibraryMissing("cannot load %s: %s" % (_LIB_PATH, e))
    c_void_p, c_int, c_size_t = ctypes.c_void_p, ctypes.c_int, ctypes.c_size_t
    lib.mgpu_b200_version.restype = c_int
    lib.mgpu_b200_error_string.restype = ctypes.c_char_p
    lib.mgpu_b200_error_string.argtypes = [c_int]
    lib.mgpu_b200_segreduce_workspace_bytes.restype = c_size_t
    lib.mgpu_b200_segreduce_workspace_bytes.argtypes = [c_int, c_int, c_int]
    lib.mgpu_b200_segreduce.restype = c_int
    lib.mgpu_b200_segreduce.argtypes = [
        c_int, c_int, c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p,
        c_void_p, c_size_t, c_void_p]
    lib.mgpu_b200_segreduce_profile.restype = c_int
    lib.mgpu_b200_segreduce_profile.argtypes = [
        c_int, c_int, c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p,
        c_void_p, c_size_t, c_void_p, ctypes.POINTER(ctypes.c_float),
        ctypes.POINTER(ctypes.c_float)]
    lib.mgpu_b200_workspace_status.restype = c_int
    lib.mgpu_b200_workspace_status.argtypes = [
        c_void_p, c_void_p, ctypes.POINTER(c_int)]
    lib.mgpu_b200_load_balance_partitions.restype = c_int
    lib.mgpu_b200_load_balance_partitions.argtypes = [
        c_int, c_void_p, c_int, c_int, c_void_p, c_void_p]
    lib.mgpu_b200_debug_lookback_timeout.restype = c_int
    lib.mgpu_b200_debug_lookback_timeout.argtypes = [
        c_void_p, c_int, ctypes.c_uint64, ctypes.POINTER(c_int), c_void_p]
    lib.mgpu_b200_debug_set_wait_limit_ns.restype = ctypes.c_uint64
    lib.mgpu_b200_debug_set_wait_limit_ns.argtypes = [ctypes.c_uint64]
    _declare_optional(lib)
    _lib = lib
    return lib


def _declare_optional(lib):
    c_void_p, c_int, c_size_t = ctypes.c_void_p, ctypes.c_int, ctypes.c_size_t
    lib.mgpu_b200_spmv_workspace_bytes.restype = c_size_t
    lib.mgpu_b200_spmv_workspace_bytes.argtypes = [c_int, c_int, c_int]
    lib.mgpu_b200_spmv.restype = c_int
    lib.mgpu_b200_spmv.argtypes = [
        c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p,
        c_void_p, c_size_t, c_void_p]
    lib.mgpu_b200_lbs_workspace_bytes.restype = c_size_t
    lib.mgpu_b200_lbs_workspace_bytes.argtypes = [c_int, c_int]
    lib.mgpu_b200_load_balance_search.restype = c_int
    lib.mgpu_b200_load_balance_search.argtypes = [
        c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_size_t,
        c_void_p]
    lib.mgpu_b200_interval_expand.restype = c_int
    lib.mgpu_b200_interval_expand.argtypes = [
        c_int, c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_size_t,
        c_void_p]
    lib.mgpu_b200_scan_workspace_bytes.restype = c_size_t
    lib.mgpu_b200_scan_workspace_bytes.argtypes = [c_int, c_int]
    lib.mgpu_b200_scan.restype = c_int
    lib.mgpu_b200_scan.argtypes = [
        c_int, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_size_t,
        c_void_p]
    lib.mgpu_b200_static_scratch_bytes.restype = c_size_t
    lib.mgpu_b200_static_scratch_bytes.argtypes = []
    lib.mgpu_b200_segreduce_static.restype = c_int
    lib.mgpu_b200_segreduce_static.argtypes = [
        c_int, c_int, c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p,
        c_void_p]
    lib.mgpu_b200_shard_pack.restype = c_int
    lib.mgpu_b200_shard_pack.argtypes = [
        c_int, c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p]
    lib.mgpu_b200_shard_lead_scratch_bytes.restype = c_size_t
    lib.mgpu_b200_shard_lead_scratch_bytes.argtypes = []
    lib.mgpu_b200_shard_lead.restype = c_int
    lib.mgpu_b200_shard_lead.argtypes = [
        c_int, c_int, c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p,
        c_void_p]
    lib.mgpu_b200_lbs_segreduce_weighted_workspace_bytes.restype = c_size_t
    lib.mgpu_b200_lbs_segreduce_weighted_workspace_bytes.argtypes = [
        c_int, c_int, c_int]
    lib.mgpu_b200_lbs_segreduce_weighted.restype = c_int
    lib.mgpu_b200_lbs_segreduce_weighted.argtypes = [
        c_int, c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p,
        c_size_t, c_void_p]
    lib.mgpu_b200_sorted_search_workspace_bytes.restype = c_size_t
    lib.mgpu_b200_sorted_search_workspace_bytes.argtypes = [c_int, c_int]
    lib.mgpu_b200_sorted_search.restype = c_int
    lib.mgpu_b200_sorted_search.argtypes = [
        c_int, c_int, c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p,
        c_size_t, c_void_p]
    lib.mgpu_b200_l2_pin.restype = c_int
    lib.mgpu_b200_l2_pin.argtypes = [c_void_p, c_size_t, c_void_p]
    lib.mgpu_b200_l2_unpin.restype = c_int
    lib.mgpu_b200_l2_unpin.argtypes = [c_void_p]
    lib.mgpu_b200_mailbox_bytes.restype = c_size_t
    lib.mgpu_b200_mailbox_bytes.argtypes = []
    lib.mgpu_b200_mailbox_create.restype = c_int
    lib.mgpu_b200_mailbox_create.argtypes = [ctypes.POINTER(c_void_p),
                                             c_void_p]
    lib.mgpu_b200_mailbox_open.restype = c_int
    lib.mgpu_b200_mailbox_open.argtypes = [c_void_p,
                                           ctypes.POINTER(c_void_p)]
    lib.mgpu_b200_mailbox_close.restype = c_int
    lib.mgpu_b200_mailbox_close.argtypes = [c_void_p]
    lib.mgpu_b200_mailbox_destroy.restype = c_int
    lib.mgpu_b200_mailbox_destroy.argtypes = [c_void_p]
    lib.mgpu_b200_mailbox_status.restype = c_int
    lib.mgpu_b200_mailbox_status.argtypes = [c_void_p, c_void_p,
                                             ctypes.POINTER(c_int)]
    lib.mgpu_b200_shard_post.restype = c_int
    lib.mgpu_b200_shard_post.argtypes = [
        c_int, c_int, c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p,
        c_int, c_int, c_int, ctypes.c_uint, ctypes.c_uint64, c_void_p]
    lib.mgpu_b200_shard_collect.restype = c_int
    lib.mgpu_b200_shard_collect.argtypes = [
        c_int, c_int, c_void_p, c_void_p, c_int, c_int, c_int, ctypes.c_uint,
        c_void_p, c_int, c_void_p, ctypes.c_uint64, c_void_p]
    lib.mgpu_b200_shard_begin.restype = c_int
    lib.mgpu_b200_shard_begin.argtypes = [
        c_int, c_int, c_void_p, c_int, c_void_p, c_int, c_void_p, c_size_t,
        c_void_p, c_void_p, c_int, c_int, c_int, ctypes.c_uint,
        ctypes.c_uint64, c_void_p]
    lib.mgpu_b200_shard_finish.restype = c_int
    lib.mgpu_b200_shard_finish.argtypes = [
        c_int, c_int, c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p,
        c_void_p, c_size_t, c_void_p, c_void_p, c_int, c_int, c_int,
        ctypes.c_uint, ctypes.c_uint64, c_void_p]
    lib.mgpu_b200_mailbox_clear_status.restype = c_int
    lib.mgpu_b200_mailbox_clear_status.argtypes = [c_void_p, c_void_p]
    lib.mgpu_b200_shard_fold.restype = c_int
    lib.mgpu_b200_shard_fold.argtypes = [
        c_int, c_int, c_void_p, c_int, c_int, c_void_p, c_int, c_void_p,
        c_void_p]
    lib.mgpu_b200_segreduce_host.restype = c_int
    lib.mgpu_b200_segreduce_host.argtypes = [
        c_int, c_int, c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p,
        c_void_p]


def _check(code):
    if code:
        text = load_library().mgpu_b200_error_string(code).decode()
        raise MgpuError(code, text)


class _NoSwitch(object):
    def __enter__(self):
        return None

    def __exit__(self, *exc):
        return False


_NO_SWITCH = _NoSwitch()


def _on(device):
    """Context in which `device` is the current CUDA device. When it already
    is (the usual case) nothing is switched: torch's own context manager costs
    several microseconds per call, which a latency-bound caller notices."""
    if not isinstance(device, torch.device):
        device = torch.device(device)
    if device.index is None or device.index == torch.cuda.current_device():
        return _NO_SWITCH
    return torch.cuda.device(device)


def _stream(device):
    return ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)


def _require_cuda(t, name, dtype=None):
    if not isinstance(t, torch.Tensor) or not t.is_cuda:
        raise TypeError("%s must be a CUDA tensor" % name)
    if not t.is_contiguous():
        raise ValueError("%s must be contiguous" % name)
    if dtype is not None and t.dtype != dtype:
        raise TypeError("%s must have dtype %s" % (name, dtype))


# One scratch buffer per (device, stream), grown on demand. Calls on one stream
# run in order, so they can share it; calls on different streams cannot.
_scratch = {}


def _workspace(device, nbytes):
    key = (device.index, torch.cuda.current_stream(device).cuda_stream)
    buf = _scratch.get(key)
    if buf is None or buf.numel() < nbytes:
        buf = torch.empty(max(nbytes, 1 << 20), dtype=torch.uint8,
                          device=device)
        _scratch[key] = buf
    return buf


def segreduce(input, segments, op="plus", init=0, out=None, workspace=None):
    """mgpu::segreduce: out[s] = fold_op(input[segments[s]:segments[s+1]]).

    segments: int32 start offsets (segments[0] == 0, non-decreasing, <= count);
    empty segments yield `init`, which is never folded into non-empty ones.
    """
    lib = load_library()
    _require_cuda(input, "input")
    _require_cuda(segments, "segments", torch.int32)
    if input.dtype not in _DTYPES:
        raise TypeError("unsupported dtype %s" % input.dtype)
    count, num_segments = input.numel(), segments.numel()
    if out is None:
        out = torch.empty(num_segments, dtype=input.dtype, device=input.device)
    else:
        _require_cuda(out, "out", input.dtype)
        if out.numel() != num_segments:
            raise ValueError("out must have one element per segment")
    dtype = _DTYPES[input.dtype]
    if workspace is None:
        workspace = _workspace(input.device,
                               lib.mgpu_b200_segreduce_workspace_bytes(
                                   dtype, count, num_segments))
    init_c = _CTYPES[input.dtype](init)
    with _on(input.device):
        _check(lib.mgpu_b200_segreduce(
            dtype, _OPS[op], input.data_ptr(), count, segments.data_ptr(),
            num_segments, out.data_ptr(), ctypes.byref(init_c),
            workspace.data_ptr(), workspace.numel(), _stream(input.device)))
    return out


def lbs_segreduce_weighted(values, segments, weights, out=None,
                           workspace=None):
    """mgpu::lbs_segreduce with f(index, seg, rank, (weight,)) =
    values[index] * weight and the weights cached per segment:
    out[s] = sum of values[i] * weights[s] over segment s (0 when empty)."""
    lib = load_library()
    _require_cuda(values, "values")
    _require_cuda(segments, "segments", torch.int32)
    _require_cuda(weights, "weights", values.dtype)
    if values.dtype not in (torch.float32, torch.float64):
        raise TypeError("unsupported dtype %s" % values.dtype)
    count, num_segments = values.numel(), segments.numel()
    if weights.numel() != num_segments:
        raise ValueError("one weight per segment")
    if out is None:
        out = torch.empty(num_segments, dtype=values.dtype,
                          device=values.device)
    dtype = _DTYPES[values.dtype]
    need = lib.mgpu_b200_lbs_segreduce_weighted_workspace_bytes(
        dtype, count, num_segments)
    if workspace is None:
        workspace = _workspace(values.device, need)
    with _on(values.device):
        _check(lib.mgpu_b200_lbs_segreduce_weighted(
            dtype, values.data_ptr(), count, segments.data_ptr(),
            num_segments, weights.data_ptr(), out.data_ptr(),
            workspace.data_ptr(), workspace.numel(), _stream(values.device)))
    return out


def sorted_search(needles, haystack, upper=False, out=None, workspace=None):
    """mgpu::sorted_search with less-than: for every key of the sorted 1-D
    CUDA tensor `needles` its lower (or upper) bound in the sorted `haystack`
    (same dtype), as int32."""
    lib = load_library()
    _require_cuda(needles, "needles")
    _require_cuda(haystack, "haystack", needles.dtype)
    if needles.dtype not in _DTYPES:
        raise TypeError("unsupported dtype %s" % needles.dtype)
    if out is None:
        out = torch.empty(needles.numel(), dtype=torch.int32,
                          device=needles.device)
    need = lib.mgpu_b200_sorted_search_workspace_bytes(needles.numel(),
                                                       haystack.numel())
    if workspace is None:
        workspace = _workspace(needles.device, need)
    with _on(needles.device):
        _check(lib.mgpu_b200_sorted_search(
            _DTYPES[needles.dtype], 1 if upper else 0, needles.data_ptr(),
            needles.numel(), haystack.data_ptr(), haystack.numel(),
            out.data_ptr(), workspace.data_ptr(), workspace.numel(),
            _stream(needles.device)))
    return out


def l2_pin(array):
    """Keep `array` (the vector later spmv calls on the current stream gather
    from) resident in the L2: mgpu_b200_l2_pin. Undo with l2_unpin()."""
    lib = load_library()
    _require_cuda(array, "array")
    with _on(array.device):
        _check(lib.mgpu_b200_l2_pin(array.data_ptr(),
                                    array.numel() * array.element_size(),
                                    _stream(array.device)))


def l2_unpin(device=None):
    lib = load_library()
    if device is None:
        device = torch.device("cuda", torch.cuda.current_device())
    with _on(device):
        _check(lib.mgpu_b200_l2_unpin(_stream(device)))


def scan(input, inclusive=False, out=None, total=None, workspace=None):
    """mgpu::scan with plus: prefix sums of a 1-D CUDA tensor.

    Returns `out` (exclusive by default). `total`, a 1-element tensor of the
    same dtype, receives the sum of all elements when given."""
    lib = load_library()
    _require_cuda(input, "input")
    if input.dtype not in _DTYPES:
        raise TypeError("unsupported dtype %s" % input.dtype)
    count = input.numel()
    if out is None:
        out = torch.empty_like(input)
    dtype = _DTYPES[input.dtype]
    need = lib.mgpu_b200_scan_workspace_bytes(dtype, count)
    if workspace is None:
        workspace = _workspace(input.device, need)
    with _on(input.device):
        _check(lib.mgpu_b200_scan(
            dtype, 1 if inclusive else 0, input.data_ptr(), count,
            out.data_ptr(), None if total is None else total.data_ptr(),
            workspace.data_ptr(), workspace.numel(), _stream(input.device)))
    return out


def segreduce_static(input, segments, op="plus", init=0, out=None):
    """segreduce without a caller-supplied workspace and without any device
    allocation inside the library: the scratch is a fixed 4 MiB block that
    ships with the library (mgpu_b200_segreduce_static). For callers that must
    not allocate at the point of the call. `out` should be preallocated by
    such callers; it is created here only as a convenience. Calls that overlap
    on one GPU race on the shared block."""
    lib = load_library()
    _require_cuda(input, "input")
    _require_cuda(segments, "segments", torch.int32)
    if input.dtype not in _DTYPES:
        raise TypeError("unsupported dtype %s" % input.dtype)
    if out is None:
        out = torch.empty(segments.numel(), dtype=input.dtype,
                          device=input.device)
    init_c = _CTYPES[input.dtype](init)
    with _on(input.device):
        _check(lib.mgpu_b200_segreduce_static(
            _DTYPES[input.dtype], _OPS[op], input.data_ptr(), input.numel(),
            segments.data_ptr(), segments.numel(), out.data_ptr(),
            ctypes.byref(init_c), _stream(input.device)))
    return out


def segreduce_profile(input, segments, op="plus", init=0, out=None,
                      workspace=None):
    """segreduce that waits for the device and returns
    (out, partition_ms, reduce_ms): the device time of its two kernels."""
    lib = load_library()
    _require_cuda(input, "input")
    _require_cuda(segments, "segments", torch.int32)
    count, num_segments = input.numel(), segments.numel()
    if out is None:
        out = torch.empty(num_segments, dtype=input.dtype, device=input.device)
    dtype = _DTYPES[input.dtype]
    need = lib.mgpu_b200_segreduce_workspace_bytes(dtype, count, num_segments)
    if workspace is None:
        workspace = _workspace(input.device, need)
    init_c = _CTYPES[input.dtype](init)
    part, red = ctypes.c_float(0), ctypes.c_float(0)
    with _on(input.device):
        _check(lib.mgpu_b200_segreduce_profile(
            dtype, _OPS[op], input.data_ptr(), count, segments.data_ptr(),
            num_segments, out.data_ptr(), ctypes.byref(init_c),
            workspace.data_ptr(), workspace.numel(), _stream(input.device),
            ctypes.byref(part), ctypes.byref(red)))
    return out, part.value, red.value


def workspace_status(workspace=None, device=None):
    """Status word of the last call that used the workspace (synchronises)."""
    lib = load_library()
    if workspace is None:
        device = torch.device("cuda", torch.cuda.current_device()) \
            if device is None else torch.device(device)
        workspace = _workspace(device, 0)
    status = ctypes.c_int(0)
    with _on(workspace.device):
        code = lib.mgpu_b200_workspace_status(
            workspace.data_ptr(), _stream(workspace.device),
            ctypes.byref(status))
    if code not in (0, 4):
        _check(code)
    return status.value


def load_balance_partitions(count, segments, spacing):
    """mgpu::load_balance_partitions: merge-path cut points every `spacing`."""
    lib = load_library()
    _require_cuda(segments, "segments", torch.int32)
    num_segments = segments.numel()
    n = (count + num_segments + spacing - 1) // spacing + 1
    out = torch.empty(n, dtype=torch.int32, device=segments.device)
    with _on(segments.device):
        _check(lib.mgpu_b200_load_balance_partitions(
            count, segments.data_ptr(), num_segments, spacing, out.data_ptr(),
            _stream(segments.device)))
    return out


def spmv(matrix, columns, vector, row_starts, out=None, workspace=None):
    """mgpu::spmv: y = A x for CSR (matrix, columns, row_starts)."""
    lib = load_library()
    _require_cuda(matrix, "matrix")
    _require_cuda(columns, "columns", torch.int32)
    _require_cuda(vector, "vector", matrix.dtype)
    _require_cuda(row_starts, "row_starts", torch.int32)
    if matrix.dtype not in (torch.float32, torch.float64):
        raise TypeError("spmv supports float32 and float64")
    nnz, rows = matrix.numel(), row_starts.numel()
    if columns.numel() != nnz:
        raise ValueError("columns and matrix must have equal length")
    if out is None:
        out = torch.empty(rows, dtype=matrix.dtype, device=matrix.device)
    dtype = _DTYPES[matrix.dtype]
    need = lib.mgpu_b200_spmv_workspace_bytes(dtype, nnz, rows)
    if workspace is None:
        workspace = _workspace(matrix.device, need)
    with _on(matrix.device):
        _check(lib.mgpu_b200_spmv(
            dtype, matrix.data_ptr(), columns.data_ptr(), vector.data_ptr(),
            nnz, row_starts.data_ptr(), rows, out.data_ptr(),
            workspace.data_ptr(), workspace.numel(), _stream(matrix.device)))
    return out


def transform_lbs(count, segments, want_ranks=True, workspace=None,
                  out_seg=None, out_rank=None):
    """mgpu::transform_lbs with the functor that records (seg, rank) per item.

    Returns (seg, rank) int32 tensors of `count` elements (rank is None when
    want_ranks is False, which is mgpu::load_balance_search). out_seg and
    out_rank, when given, receive the results.
    """
    lib = load_library()
    _require_cuda(segments, "segments", torch.int32)
    num_segments = segments.numel()
    dev = segments.device
    if out_seg is None:
        out_seg = torch.empty(count, dtype=torch.int32, device=dev)
    if want_ranks and out_rank is None:
        out_rank = torch.empty(count, dtype=torch.int32, device=dev)
    for name, t in (("out_seg", out_seg), ("out_rank", out_rank)):
        if t is not None:
            _require_cuda(t, name, torch.int32)
            if t.numel() != count:
                raise ValueError("%s must have one element per item" % name)
    seg, rank = out_seg, (out_rank if want_ranks else None)
    need = lib.mgpu_b200_lbs_workspace_bytes(count, num_segments)
    if workspace is None:
        workspace = _workspace(dev, need)
    with _on(dev):
        _check(lib.mgpu_b200_load_balance_search(
            count, segments.data_ptr(), num_segments, seg.data_ptr(),
            rank.data_ptr() if want_ranks else None,
            workspace.data_ptr(), workspace.numel(), _stream(dev)))
    return seg, rank


def load_balance_search(count, segments, workspace=None):
    """mgpu::load_balance_search: segment index of every item."""
    return transform_lbs(count, segments, want_ranks=False,
                         workspace=workspace)[0]


def interval_expand(input, count, segments, out=None, workspace=None):
    """mgpu::interval_expand: out[i] = input[segment of item i]."""
    lib = load_library()
    _require_cuda(input, "input")
    _require_cuda(segments, "segments", torch.int32)
    num_segments = segments.numel()
    if input.numel() != num_segments:
        raise ValueError("input must have one element per segment")
    if out is None:
        out = torch.empty(count, dtype=input.dtype, device=input.device)
    need = lib.mgpu_b200_lbs_workspace_bytes(count, num_segments)
    if workspace is None:
        workspace = _workspace(input.device, need)
    with _on(input.device):
        _check(lib.mgpu_b200_interval_expand(
            input.element_size(), input.data_ptr(), count,
            segments.data_ptr(), num_segments, out.data_ptr(),
            workspace.data_ptr(), workspace.numel(), _stream(input.device)))
    return out


def segreduce_host(input, segments, op="plus", init=0, out=None):
    """segreduce on HOST tensors: the library copies the inputs to the current
    device in chunks overlapped with the reduction, and copies the result
    back. Blocks until the result is in `out`. Pinned tensors copy fastest."""
    lib = load_library()
    if input.is_cuda or segments.is_cuda:
        raise TypeError("segreduce_host takes CPU tensors")
    if segments.dtype != torch.int32 or input.dtype not in _DTYPES:
        raise TypeError("unsupported dtype")
    input = input.contiguous()
    segments = segments.contiguous()
    if out is None:
        out = torch.empty(segments.numel(), dtype=input.dtype)
    init_c = _CTYPES[input.dtype](init)
    _check(lib.mgpu_b200_segreduce_host(
        _DTYPES[input.dtype], _OPS[op], input.data_ptr(), input.numel(),
        segments.data_ptr(), segments.numel(), out.data_ptr(),
        ctypes.byref(init_c), None))
    return out
