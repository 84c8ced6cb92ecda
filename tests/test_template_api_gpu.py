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


def test_template_entry_points():
    if not os.path.exists(EXE):
        pytest.fail("tests/cpp/build/test_template_api is not built: run "
                    "python -c 'import __graft_entry__ as g; g.build()'")
    run = subprocess.run([EXE], capture_output=True, text=True, timeout=300)
    print(run.stdout)
    assert "FAIL" not in run.stdout, run.stdout
    assert "ALL PASSED" in run.stdout, run.stdout + run.stderr
    assert run.returncode == 0
