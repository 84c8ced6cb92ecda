"""Runs tests/cpp/test_template_api.cu (built by __graft_entry__.build()):
the C++ template entry points with user functors, a 24-byte user type, lambda
and store iterators, cached tuples, the interval_* family -- each checked
against a host loop inside the program."""
import os
import subprocess

import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
EXE = os.path.join(ROOT, "tests", "cpp", "build", "test_template_api")


PIPELINE = os.path.join(ROOT, "tests", "cpp", "build", "test_nearest_pipeline")


def run_program(exe):
    if not os.path.exists(exe):
        pytest.fail("%s is not built: run "
                    "python -c 'import __graft_entry__ as g; g.build()'"
                    % os.path.relpath(exe, ROOT))
    return subprocess.run([exe], capture_output=True, text=True, timeout=300)


def test_nearest_pipeline():
    """tests/cpp/test_nearest_pipeline.cu: scan -> interval_expand ->
    transform_lbs -> scan in place -> lbs_segreduce with a 24-byte type and a
    user-written merge operator, the call chain of the reference's
    demo/cities.cu:143-236 on seeded synthetic points, bit for bit against a
    brute-force host loop."""
    run = run_program(PIPELINE)
    print(run.stdout)
    assert "FAIL" not in run.stdout, run.stdout
    assert "ALL PASSED" in run.stdout, run.stdout + run.stderr
    assert run.returncode == 0


def test_workcreate_bfs():
    """tests/cpp/test_workcreate_bfs.cu: breadth-first search whose frontier
    is expanded by expt::lbs_workcreate (upsweep / downsweep), the way the
    reference's demo/bfs2.cu:23-65 uses it, on seeded synthetic graphs;
    levels against a host search, every round's segment array against the
    scan of the claimed vertices' degrees."""
    run = run_program(os.path.join(ROOT, "tests", "cpp", "build",
                                   "test_workcreate_bfs"))
    print(run.stdout)
    assert "FAIL" not in run.stdout, run.stdout
    assert "ALL PASSED" in run.stdout, run.stdout + run.stderr
    assert run.returncode == 0


def test_template_entry_points():
    run = run_program(EXE)
    print(run.stdout)
    assert "FAIL" not in run.stdout, run.stdout
    assert "ALL PASSED" in run.stdout, run.stdout + run.stderr
    assert run.returncode == 0


def test_sharded_segreduce_program():
    """tests/cpp/test_sharded.cu: mgpu::sharded_segreduce, the C++ entry of the
    multi-GPU layer -- one global table of 64-bit segment starts cut into
    shard-local tables on the devices, two shards on every GPU of the machine
    (up to four; one GPU runs the same chain of boundary records through its
    own mailbox), 70 steps per case, the assembled outputs against the host
    loop of tests/test_segreduce.cu:40-49 over the whole array."""
    run = run_program(os.path.join(ROOT, "tests", "cpp", "build",
                                   "test_sharded"))
    print(run.stdout)
    assert "FAIL" not in run.stdout, run.stdout
    assert "ALL PASSED" in run.stdout, run.stdout + run.stderr
    assert run.returncode == 0
