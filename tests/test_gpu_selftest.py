"""The stand-alone C++ check of the library (numerics against a CPU loop, timing against cuBLAS). It compiles a
program with nvcc at test time and links cuBLAS; without nvcc on the machine the test is skipped."""
import json
import os
import subprocess

import pytest

import shutil

pytestmark = [pytest.mark.gpu,
              pytest.mark.skipif(shutil.which("nvcc") is None and not os.path.exists("/usr/local/cuda/bin/nvcc"),
                                 reason="needs nvcc")]


@pytest.mark.parametrize("argv", [["1000", "4", "512", "1024", "3"], ["129", "3", "64", "256", "2"]])
def test_cpp_selftest(argv):
    from ccfuser_b200.build import build_selftest
    exe = build_selftest()
    out = subprocess.run([exe] + argv, capture_output=True, text=True, timeout=600)
    recs = [json.loads(l) for l in out.stdout.splitlines() if l.startswith("{")]
    assert out.returncode == 0, out.stdout + out.stderr
    assert {r["variant"] for r in recs} == {"one_cta_128x256", "cta_pair_256x256", "cublas_per_group"}
    assert all(r["ok"] for r in recs if "ok" in r)
