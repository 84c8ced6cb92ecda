"""Builds libmgpu_b200.so (the C-ABI library) in-tree with nvcc for sm_100a.

The library is compiled from moderngpu_b200/csrc/*.cu against the template
headers in include/moderngpu/. nvcc cross-compiles without a GPU present.
"""
import glob
import os
import subprocess
import sys

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(PKG_DIR)
LIB_DIR = os.path.join(PKG_DIR, "lib")
LIB_PATH = os.path.join(LIB_DIR, "libmgpu_b200.so")

NVCC_FLAGS = [
    "-std=c++17",
    "-gencode", "arch=compute_100a,code=sm_100a",
    "--expt-extended-lambda", "--expt-relaxed-constexpr",
    "-O3", "-lineinfo",
    "-Xcompiler", "-fPIC", "-shared",
]


def sources():
    return sorted(glob.glob(os.path.join(PKG_DIR, "csrc", "*.cu")))


def _inputs():
    deps = sources()
    deps += glob.glob(os.path.join(ROOT, "include", "*.h"))
    deps += glob.glob(os.path.join(ROOT, "include", "moderngpu", "*.hxx"))
    deps += glob.glob(os.path.join(ROOT, "include", "moderngpu", "b200", "*.hxx"))
    return deps


def up_to_date():
    if not os.path.exists(LIB_PATH):
        return False
    built = os.path.getmtime(LIB_PATH)
    return all(os.path.getmtime(p) <= built for p in _inputs())


def build(force=False, verbose=False):
    """Compile the library if any source or header is newer than it."""
    if not force and up_to_date():
        return LIB_PATH
    os.makedirs(LIB_DIR, exist_ok=True)
    nvcc = os.environ.get("NVCC", "nvcc")
    cmd = [nvcc] + NVCC_FLAGS + ["-I", os.path.join(ROOT, "include"),
                                 "-o", LIB_PATH] + sources()
    if verbose:
        cmd.insert(1, "-Xptxas")
        cmd.insert(2, "-v")
        print(" ".join(cmd))
    subprocess.check_call(cmd)
    return LIB_PATH


if __name__ == "__main__":
    build(force="--force" in sys.argv, verbose=True)
