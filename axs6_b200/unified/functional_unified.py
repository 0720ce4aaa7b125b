"""Autograd functions of the NF5 path (mirror of ``axs/unified/functional_unified.py``)."""
from __future__ import annotations

from typing import Literal

import torch

from .. import ops
from .._linear_fn import AXSLinearFP32Function
from ..core import DEFAULT_BLOCK_SIZE
from .backend import accelerated_fake_quantize as _accel_fq


class _FusedQuantizeSTE(torch.autograd.Function):
    """Forward: NF5 fake-quantise; backward: identity (functional_unified.py:38-60)."""

    @staticmethod
    def forward(ctx, tensor: torch.Tensor, block_size: int, rounding: str) -> torch.Tensor:
        return _accel_fq(tensor, block_size=block_size, rounding=rounding)

    @staticmethod
    def backward(ctx, grad_output: torch.Tensor):
        return grad_output, None, None


def fake_quantize_unified(tensor: torch.Tensor, block_size: int = DEFAULT_BLOCK_SIZE,
                          rounding: Literal["nearest", "stochastic"] = "nearest") -> torch.Tensor:
    """NF5 fake-quantise with a straight-through gradient (functional_unified.py:63-82)."""
    return _FusedQuantizeSTE.apply(tensor, block_size, rounding)


def axs_linear_unified(input: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None = None,
                       block_size: int = DEFAULT_BLOCK_SIZE, quantize_input: bool = True,
                       quantize_grad: bool = True) -> torch.Tensor:
    """NF5 quantised linear with autograd (functional_unified.py:173-201): weights and
    (optionally) activations fake-quantised to nearest, gradient fake-quantised stochastically,
    three tensor-core products.  fp32 tensors in -> fp32 out."""
    return AXSLinearFP32Function.apply(input, weight, bias, block_size, quantize_input, quantize_grad,
                                       ops.GRID_NF5, "axs_linear_unified")


def axs_matmul_unified(a: torch.Tensor, b: torch.Tensor, block_size: int = DEFAULT_BLOCK_SIZE,
                       quantize_inputs: bool = True) -> torch.Tensor:
    """NF5 quantised matmul, forward only (functional_unified.py:204-227): both operands are
    fake-quantised along their LAST dimension, then multiplied; ``a`` (*, M, K), ``b`` (K, N)."""
    from .backend import accelerated_matmul
    if quantize_inputs:
        a = _accel_fq(a, block_size, "nearest")
        b = _accel_fq(b, block_size, "nearest")
    return accelerated_matmul(a, b)
