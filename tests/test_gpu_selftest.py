"""The stand-alone C++ check of the library (numerics against a CPU loop, timing against cuBLAS).

Opt-in (CCFUSER_TEST_SELFTEST=1): it compiles a program with nvcc at test time and links cuBLAS."""
import json
import os
import subprocess

import pytest

pytestmark = [pytest.mark.gpu,
              pytest.mark.skipif(os.environ.get("CCFUSER_TEST_SELFTEST") != "1", reason="opt-in: CCFUSER_TEST_SELFTEST=1")]


@pytest.mark.parametrize("argv", [["1000", "4", "512", "1024", "3"], ["129", "3", "64", "256", "2"]])
def test_cpp_selftest(argv):
    from ccfuser_b200.build import build_selftest
    exe = build_selftest()
    out = subprocess.run([exe] + argv, capture_output=True, text=True, timeout=600)
    recs = [json.loads(l) for l in out.stdout.splitlines() if l.startswith("{")]
    assert out.returncode == 0, out.stdout + out.stderr
    assert {r["variant"] for r in recs} == {"one_cta_128x256", "cta_pair_256x256", "cublas_per_group"}
    assert all(r["ok"] for r in recs if "ok" in r)
