"""moderngpu_b200: B200-native segmented reduction, load-balancing search and
CSR spmv behind moderngpu's names.

This package is a thin ctypes binding of libmgpu_b200.so (C ABI declared in
include/moderngpu_b200.h). torch supplies device memory and streams only; all
computation happens in the library's CUDA kernels. There is no CPU fallback:
importing works without the library, but the first call raises if the library
has not been built (python -m moderngpu_b200.build) or cannot be loaded.
"""
from .binding import (  # noqa: F401
    LibraryMissing,
    MgpuError,
    interval_expand,
    l2_pin,
    l2_unpin,
    lbs_segreduce_weighted,
    lib_path,
    load_balance_partitions,
    load_balance_search,
    load_library,
    scan,
    segreduce,
    sorted_search,
    segreduce_host,
    segreduce_profile,
    segreduce_static,
    spmv,
    transform_lbs,
    workspace_status,
)

__all__ = [
    "LibraryMissing", "MgpuError", "interval_expand", "l2_pin", "l2_unpin", "lbs_segreduce_weighted", "lib_path",
    "load_balance_partitions", "load_balance_search", "load_library", "scan",
    "sorted_search",
    "segreduce", "segreduce_host", "segreduce_profile",
    "segreduce_static", "spmv", "transform_lbs", "workspace_status",
]
