"""The bounds-check build of the library (every row lookup through a tsa_ptr2d checked against its extent, a lookup outside
counted and redirected instead of trapping) on small forward / backward / decode cases: no lookup outside the callers'
buffers, and the check itself fires when asked to."""
import json
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
BOUNDS_LIB = os.path.join(ROOT, "tscale_b200", "libtsa_b200_bounds.so")


def test_production_build_reports_no_checks():
    from tscale_b200 import abi
    assert abi.lib().tsa_bounds_check_hits(0) == -1
    assert abi.lib().tsa_selftest_bounds_check(None, None) == -1


@pytest.mark.gpu
def test_bounds_check_build_small_cases():
    if not os.path.exists(BOUNDS_LIB):
        pytest.skip("bounds-check build missing: make -C tscale_b200/csrc bounds")
    env = dict(os.environ, TSA_B200_LIB=BOUNDS_LIB, PYTHONPATH=ROOT + os.pathsep + os.environ.get("PYTHONPATH", ""))
    res = subprocess.run([sys.executable, "-m", "tests.bounds_cases"], cwd=ROOT, env=env, capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-2000:]
    line = json.loads([x for x in res.stdout.splitlines() if x.startswith("{")][-1])
    assert line["selftest_caught"] == 1, line   # the deliberate out-of-range lookup was seen (and redirected)
    assert line["hits"] == 0, line              # and none in the library's own kernels
    assert line["cases"] >= 7
