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


class _ConvSTE(torch.autograd.Function):
    """Convolution of fake-quantised operands (nn/functional.py:220-288).  The weight is quantised as a
    (C_out, C_in/groups * kH * kW) matrix, the input along its last dimension, the incoming gradient
    (stochastically) along its last dimension; the convolutions themselves are the library's (cuDNN):
    this package accelerates the quantiser, not the convolution."""

    @staticmethod
    def forward(ctx, input, weight, bias, stride, padding, dilation, groups, block_size):
        wq = fake_quantize(weight.reshape(weight.shape[0], -1), block_size, "nearest").reshape(weight.shape)
        xq = fake_quantize(input, block_size, "nearest") if input.numel() else input
        ctx.save_for_backward(xq, wq)
        ctx.has_bias = bias is not None
        ctx.conv = (stride, padding, dilation, groups)
        ctx.block_size = block_size
        return torch.nn.functional.conv2d(xq, wq, bias, stride, padding, dilation, groups)

    @staticmethod
    def backward(ctx, grad_output):
        xq, wq = ctx.saved_tensors
        stride, padding, dilation, groups = ctx.conv
        gq = fake_quantize(grad_output, ctx.block_size, "stochastic") if grad_output.numel() else grad_output
        dx = dw = db = None
        if ctx.needs_input_grad[0]:
            dx = torch.nn.grad.conv2d_input(xq.shape, wq, gq, stride, padding, dilation, groups)
        if ctx.needs_input_grad[1]:
            dw = torch.nn.grad.conv2d_weight(xq, wq.shape, gq, stride, padding, dilation, groups)
        if ctx.has_bias and ctx.needs_input_grad[2]:
            db = gq.sum(dim=(0, 2, 3))
        return dx, dw, db, None, None, None, None, None


def _pair(v):
    return v if isinstance(v, tuple) else (v, v)


def axs_conv2d(input: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None = None, stride=1, padding=0,
               dilation=1, groups: int = 1, block_size: int = DEFAULT_BLOCK_SIZE) -> torch.Tensor:
    """Uniform-grid quantised 2-D convolution with autograd (nn/functional.py:291-323)."""
    return _ConvSTE.apply(input, weight, bias, _pair(stride), _pair(padding), _pair(dilation), groups, block_size)
