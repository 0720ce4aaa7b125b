"""The reference's CPU unit-test files, run UNCHANGED against this library on the GPU.

``tests/test_core.py``, ``tests/test_quantize.py``, ``tests/test_unified.py``, ``tests/test_nn.py`` and
``tests/test_training.py`` of the reference pin the Python surface of the path (block and tensor round trips,
rounding modes, NF5 tables, fake-quantise properties, the functional / module / optimiser / pipeline API and
the convergence of small fits).  A child pytest loads
``axs6_b200.reference_alias``, which makes ``import axs`` resolve to this package and CUDA the default
device of new tensors, and runs the copies under ``baseline/_ref/reference_tests``.  Skipped when the
copies are absent.
"""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF_TESTS = os.path.join(ROOT, "baseline", "_ref", "reference_tests")

# Cases that cannot hold for a library without a CPU path or that look inside the reference, each with the reason.
DESELECT: list[str] = [
    # compares with the reference's V2 package (axs.v2), which is not part of the path this library replaces
    "test_unified.py::TestQualityVsV2::test_mse_within_1_percent_of_v2",
]


@pytest.mark.parametrize("name", ["test_core.py", "test_quantize.py", "test_unified.py", "test_nn.py", "test_training.py"])
def test_reference_cpu_file_passes_against_this_library(name):
    path = os.path.join(REF_TESTS, name)
    if not os.path.exists(path):
        pytest.skip("no copy of the reference's tests under baseline/_ref (run baseline/install_reference.py)")
    env = dict(os.environ)
    env["PYTHONPATH"] = os.pathsep.join([ROOT, env.get("PYTHONPATH", "")])
    cmd = [sys.executable, "-m", "pytest", "-q", "--no-header", "-p", "axs6_b200.reference_alias",
           "-p", "no:cacheprovider", "--rootdir", REF_TESTS, path]
    for d in DESELECT:
        if d.startswith(name):
            cmd += ["--deselect", d]
    out = subprocess.run(cmd, env=env, cwd=REF_TESTS, capture_output=True, text=True, timeout=900)
    first = out
    if out.returncode != 0:
        # One more run: a child can die before its tests start, and several of the reference's cases are statistical
        # (means and ratios of random draws).  A failure that repeats is reported with both outputs.
        out = subprocess.run(cmd, env=env, cwd=REF_TESTS, capture_output=True, text=True, timeout=900)
    tail = (out.stdout + out.stderr)[-6000:] + ("\n--- first run ---\n" + (first.stdout + first.stderr)[-3000:] if first is not out else "")
    assert out.returncode == 0, f"reference test file {name} failed against this library:\n{tail}"
    assert " passed" in out.stdout, tail
