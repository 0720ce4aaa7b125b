"""Puts an UNMODIFIED copy of the reference next to the benchmark so that it travels to the GPU box.

    python baseline/install_reference.py [/path/to/reference/checkout]

* installs the reference package (pure Python, `axs/`) into ``baseline/_ref/`` with pip
  (``--no-index --no-deps --target``; the checkout is copied to a temporary folder first because
  pip writes build files into the source tree and the checkout is read-only);
* copies the reference's three CUDA-only test files (``tests/test_triton_kernels.py``,
  ``tests/test_triton_fused_linear.py``, ``tests/test_mixed_precision.py``) and five of its CPU test
  files (``tests/test_core.py``, ``tests/test_quantize.py``, ``tests/test_unified.py``, ``tests/test_nn.py``,
  ``tests/test_training.py``) into
  ``baseline/_ref/reference_tests/`` so that they can be run, unchanged, against this library on a
  machine with a GPU (``axs6_b200.reference_shim`` / ``axs6_b200.reference_alias``).

``baseline/_ref/`` is git-ignored: nothing of the reference enters this repository's history.
``bench.py --impl reference`` and the ``cpu_baseline`` leg time the reference's own eager
``fused_fake_quantize`` from there; when the folder is absent they fall back to the C port under
``oracle/`` and say so (``kind: "port"``).
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
import tempfile

HERE = os.path.dirname(os.path.abspath(__file__))
TARGET = os.path.join(HERE, "_ref")
TESTS = ("test_triton_kernels.py", "test_triton_fused_linear.py", "test_mixed_precision.py",
         "test_core.py", "test_quantize.py", "test_unified.py", "test_nn.py", "test_training.py")


def install(checkout: str = "/root/reference", force: bool = False) -> str | None:
    """Returns the target folder, or None when no checkout is present (e.g. on the GPU box)."""
    if not os.path.isdir(os.path.join(checkout, "axs")):
        return TARGET if os.path.isdir(os.path.join(TARGET, "axs")) else None
    complete = os.path.isdir(os.path.join(TARGET, "axs")) and all(
        os.path.exists(os.path.join(TARGET, "reference_tests", name)) for name in TESTS)
    if complete and not force:
        return TARGET
    if os.path.isdir(TARGET):
        shutil.rmtree(TARGET)
    with tempfile.TemporaryDirectory() as tmp:
        src = os.path.join(tmp, "reference")
        shutil.copytree(checkout, src, ignore=shutil.ignore_patterns(".git", "__pycache__", "*.pyc"))
        cmd = [sys.executable, "-m", "pip", "install", "--quiet", "--no-index", "--no-build-isolation", "--no-deps",
               "--find-links", "/opt/wheelhouse", "--target", TARGET, src]
        subprocess.check_call(cmd)
        tdir = os.path.join(TARGET, "reference_tests")
        os.makedirs(tdir, exist_ok=True)
        for name in TESTS:
            p = os.path.join(src, "tests", name)
            if os.path.exists(p):
                shutil.copy(p, os.path.join(tdir, name))
    return TARGET


if __name__ == "__main__":
    paths = [a for a in sys.argv[1:] if not a.startswith("--")]
    print(install(paths[0] if paths else "/root/reference", force="--force" in sys.argv))
