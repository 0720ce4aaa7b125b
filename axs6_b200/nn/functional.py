"""V1 functional ops (mirror of ``axs/nn/functional.py``)."""
from __future__ import annotations

from typing import Literal

import torch

from .. import ops
from .._linear_fn import AXSLinearFP32Function
from ..core import DEFAULT_BLOCK_SIZE, VALID_BLOCK_SIZES


class _QuantizeSTE(torch.autograd.Function):
    """Forward: dequantize(quantize(x)) on the uniform grid, fused in one kernel, fp32 result
    whatever the input dtype; backward: identity (nn/functional.py:35-63)."""

    @staticmethod
    def forward(ctx, tensor: torch.Tensor, block_size: int, rounding: str) -> torch.Tensor:
        assert block_size in VALID_BLOCK_SIZES, f"Block size must be one of {VALID_BLOCK_SIZES}"
        return ops.fake_quantize(tensor, block_size, ops.GRID_UNIFORM, rounding, out_dtype=torch.float32,
                                 who="fake_quantize")

    @staticmethod
    def backward(ctx, grad_output: torch.Tensor):
        return grad_output, None, None


def fake_quantize(tensor: torch.Tensor, block_size: int = DEFAULT_BLOCK_SIZE,
                  rounding: Literal["nearest", "stochastic"] = "nearest") -> torch.Tensor:
    """Uniform-grid fake-quantise with a straight-through gradient (nn/functional.py:66-85)."""
    return _QuantizeSTE.apply(tensor, block_size, rounding)


def axs_linear(input: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None = None,
               block_size: int = DEFAULT_BLOCK_SIZE, quantize_input: bool = True,
               quantize_grad: bool = True) -> torch.Tensor:
    """Uniform-grid quantised linear with autograd (nn/functional.py:93-180)."""
    return AXSLinearFP32Function.apply(input, weight, bias, block_size, quantize_input, quantize_grad,
                                       ops.GRID_UNIFORM, "axs_linear")


def axs_matmul(a: torch.Tensor, b: torch.Tensor, block_size: int = DEFAULT_BLOCK_SIZE,
               quantize_inputs: bool = True) -> torch.Tensor:
    """Uniform-grid quantised matmul, forward only: operands fake-quantised along their last
    dimension, then multiplied on the tensor cores (nn/functional.py, ``axs_matmul``)."""
    from ..unified.backend import accelerated_matmul
    if quantize_inputs:
        a = fake_quantize(a, block_size, "nearest")
        b = fake_quantize(b, block_size, "nearest")
    return accelerated_matmul(a, b)
