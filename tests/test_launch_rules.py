"""The late-wait launch bookkeeping (csrc/kernels/common.cuh) as a host-only program: which
kernel may start before its predecessor has finished, for sequences of normal, late and side
kernels.  Needs nvcc (host compilation only), no GPU."""
import os
import shutil
import subprocess
import tempfile

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _nvcc():
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", shutil.which("nvcc")):
        if cand and os.path.exists(cand):
            return cand
    return None


@pytest.mark.skipif(_nvcc() is None, reason="nvcc not found")
def test_late_wait_rules_host_program():
    with tempfile.TemporaryDirectory() as d:
        exe = os.path.join(d, "late_wait_rules")
        r = subprocess.run([_nvcc(), "-std=c++17", "-O1", "-I", os.path.join(ROOT, "csrc", "kernels"),
                            "-gencode", "arch=compute_100a,code=sm_100a",
                            os.path.join(ROOT, "tests", "cpp", "late_wait_rules.cu"), "-o", exe],
                           capture_output=True, text=True, timeout=300)
        assert r.returncode == 0, r.stderr[-3000:]
        r = subprocess.run([exe], capture_output=True, text=True, timeout=60)
        assert r.returncode == 0 and "RULES_OK" in r.stdout, (r.stdout, r.stderr)
