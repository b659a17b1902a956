"""The index-checking build flavour (``-DHPB_DEBUG_BOUNDS``, selected with ``HPB_DEBUG_BOUNDS=1``) is
the stand-in for a memory checker: the kernels whose indices come from device-side tables (expert
dispatch / combine, grouped GEMMs, the weight-gather work queue, the router) run their small-shape
oracle tests under it, and no check may fire (a fired check records status code 7, which
``native.check_status()`` turns into an exception inside those tests)."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_small_shape_kernel_tests_pass_under_the_index_checking_build():
    env = dict(os.environ, HPB_DEBUG_BOUNDS="1")
    probe = subprocess.run([sys.executable, "-c",
                            "from hyper_parallel_b200.ops import native; print(native.lib()._name)"],
                           cwd=ROOT, env=env, capture_output=True, text=True, timeout=900)
    assert probe.returncode == 0, probe.stderr[-2000:]
    assert "libhpb200_dbg.so" in probe.stdout
    r = subprocess.run([sys.executable, "-m", "pytest", "tests/test_gpu_kernels.py", "-q", "-x", "-k",
                        "grouped_linear or fused_expert_ffn or fused_weight_allgather or rides_on or moe_router "
                        "or fp8_grouped"],
                       cwd=ROOT, env=env, capture_output=True, text=True, timeout=1800)
    assert r.returncode == 0, (r.stdout[-3000:], r.stderr[-2000:])
    assert " passed" in r.stdout
