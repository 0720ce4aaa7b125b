"""Makes ``import axs`` resolve to this package, with CUDA as torch's default device.

The reference's CPU test files (tests/test_core.py, tests/test_quantize.py, tests/test_unified.py,
tests/test_nn.py, tests/test_training.py of the reference) import ``axs.core``, ``axs.quantize``, ``axs.unified.*`` and build their inputs with plain
``torch.randn(...)``.  Loaded as a pytest plugin (``pytest -p axs6_b200.reference_alias <files>``) this
module registers every mirrored module of this package under the reference's name and makes new
tensors land on the GPU, so that those files run UNCHANGED against this library: same names, same
arguments, same return types, only the device differs.  It is a test aid; a program that wants the
same effect writes ``import axs6_b200 as axs``.
"""
from __future__ import annotations

import importlib
import sys

MODULES = ("core", "quantize", "nn", "nn.functional", "nn.modules", "nn.optim", "unified", "unified.quantize_unified",
           "unified.functional_unified", "unified.modules_unified", "unified.training_unified", "unified.backend",
           "unified.triton_kernels", "unified.mixed_precision", "unified.distributed", "triton_kernels")


def install(default_device: str | None = "cuda") -> None:
    import torch

    import axs6_b200
    sys.modules["axs"] = axs6_b200
    for name in MODULES:
        sys.modules["axs." + name] = importlib.import_module("axs6_b200." + name)
    if default_device is not None:
        torch.set_default_device(default_device)


def pytest_configure(config):      # pytest -p axs6_b200.reference_alias
    install()
