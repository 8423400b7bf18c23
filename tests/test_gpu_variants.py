"""Kernel variants that an environment variable selects must give the same stage-by-stage results
as the default path: the swapped-operand decode GEMMs at their 64-token tile (B200MOE_DECODE=64), plain stream-ordered
launches instead of programmatic dependent launches (B200MOE_PDL=0), and the separate routing, scan
and placement kernels at decode sizes, where one fused kernel is the default (B200MOE_FRONT=0).  The switches are read once
per process, so the stage tests are re-run in a child process with the variable set."""
import os
import subprocess
import sys

import pytest

from conftest import ROOT


@pytest.mark.gpu
def test_small_shapes_stage_by_stage_with_decode_kernels_up_to_64_tokens():
    env = dict(os.environ, B200MOE_DECODE="64")
    r = subprocess.run([sys.executable, "-m", "pytest", "-q", "-x", "-m", "gpu", "-k",
                        "T64_off0 or T57_off240 or T64_ts0 or T1_off0",
                        os.path.join(ROOT, "tests", "test_gpu_layer.py")],
                       env=env, cwd=ROOT, capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-2000:]
    assert "passed" in r.stdout


@pytest.mark.gpu
def test_small_shapes_stage_by_stage_without_dependent_launches():
    env = dict(os.environ, B200MOE_PDL="0")
    r = subprocess.run([sys.executable, "-m", "pytest", "-q", "-x", "-m", "gpu", "-k",
                        "small_shapes or T64_ts0 or run_twice",
                        os.path.join(ROOT, "tests", "test_gpu_layer.py")],
                       env=env, cwd=ROOT, capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-2000:]
    assert "passed" in r.stdout


@pytest.mark.gpu
def test_decode_sizes_with_separate_front_kernels():
    env = dict(os.environ, B200MOE_FRONT="0")
    r = subprocess.run([sys.executable, "-m", "pytest", "-q", "-x", "-m", "gpu", "-k",
                        "T1_off0 or T8_ or T1_ts1 or (oracle and 4-1) or (oracle and 16-0)",
                        os.path.join(ROOT, "tests", "test_gpu_layer.py")],
                       env=env, cwd=ROOT, capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-2000:]
    assert "passed" in r.stdout
