"""Routes an installed copy of the reference package (``import axs``) onto this library.

The reference reaches its GPU kernels through a handful of dispatch functions
(``axs/unified/backend.py:495-671``: ``accelerated_fake_quantize``, ``accelerated_linear``,
``accelerated_matmul``) and two Triton launchers (``axs/unified/triton_kernels.py:295-482``);
every module and autograd function of ``axs.unified`` calls one of those.  ``install()`` rebinds
these names -- in the modules that define them and in the modules that imported them under an
alias -- to the functions of ``axs6_b200`` with the same signatures, and swaps the mixed-precision
autograd function (``axs/unified/mixed_precision.py:65-155``) for the one that runs the tcgen05
GEMMs.  Nothing else of the reference changes: its modules, training pipeline and tests keep
running their own Python code on top.

    import axs6_b200.reference_shim as shim
    shim.install()           # after this, axs.unified.* runs on libaxs6_b200.so for CUDA tensors

The module is also a pytest plugin (``pytest -p axs6_b200.reference_shim <reference tests>``):
the hook below installs the shim before test collection, so the reference's own CUDA tests run
unchanged against this library.

CPU tensors keep the reference's own eager path (this library has no CPU path), exactly as the
reference's dispatcher does for them (``backend.py:128-144``).
"""
from __future__ import annotations

import importlib

_installed = False


def _cuda_or(ours, theirs):
    """Call ``ours`` for CUDA tensors and the reference's original for anything else."""
    def fn(tensor, *args, **kwargs):
        if getattr(tensor, "is_cuda", False):
            return ours(tensor, *args, **kwargs)
        return theirs(tensor, *args, **kwargs)
    fn.__name__ = getattr(ours, "__name__", "fn")
    fn.__doc__ = getattr(ours, "__doc__", None)
    return fn


def install() -> None:
    """Rebind the reference's dispatch functions to this library (idempotent)."""
    global _installed
    if _installed:
        return
    rb = importlib.import_module("axs.unified.backend")
    rt = importlib.import_module("axs.unified.triton_kernels")
    rf = importlib.import_module("axs.unified.functional_unified")
    rm = importlib.import_module("axs.unified.mixed_precision")
    ru = importlib.import_module("axs.unified")
    ob = importlib.import_module("axs6_b200.unified.backend")
    ot = importlib.import_module("axs6_b200.unified.triton_kernels")
    om = importlib.import_module("axs6_b200.unified.mixed_precision")

    fq = _cuda_or(ob.accelerated_fake_quantize, rb.accelerated_fake_quantize)
    lin = _cuda_or(ob.accelerated_linear, rb.accelerated_linear)
    mm = _cuda_or(ob.accelerated_matmul, rb.accelerated_matmul)
    rb.accelerated_fake_quantize, rb.accelerated_linear, rb.accelerated_matmul = fq, lin, mm
    ru.accelerated_fake_quantize, ru.accelerated_linear, ru.accelerated_matmul = fq, lin, mm
    # modules that bound the dispatchers under an alias at import time
    rf._accel_fq, rf._accel_linear, rf._accel_mm = fq, lin, mm
    rm._accel_fq = fq
    # the launchers keep their names; they raise for CPU tensors as the reference's do
    rt.triton_fused_fake_quantize = ot.triton_fused_fake_quantize
    rt.triton_fused_linear = ot.triton_fused_linear
    rt.has_triton = lambda: True
    ru.triton_fused_fake_quantize = ot.triton_fused_fake_quantize
    ru.triton_fused_linear = ot.triton_fused_linear
    # mixed-precision Linear: fake-quantise kernels + tcgen05 GEMMs in one C-ABI call per direction
    ref_fn = rm._AXSLinearBF16Function

    class _Routed:
        """``apply`` with the reference Function's signature: CUDA -> this library, CPU -> the reference."""

        @staticmethod
        def apply(input, weight, bias, block_size, quantize_input, quantize_grad):
            target = om._AXSLinearBF16Function if input.is_cuda else ref_fn
            return target.apply(input, weight, bias, block_size, quantize_input, quantize_grad)

    rm._AXSLinearBF16Function = _Routed
    _installed = True


def pytest_configure(config):        # pytest plugin hook
    install()
