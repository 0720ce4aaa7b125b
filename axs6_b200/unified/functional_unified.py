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
    fake-quantised along their LAST dimension, then multiplied; ``a`` (*, M, K), ``b`` (*, K, N) with
    broadcasting batch dimensions.  Without quantisation the reference's function IS ``torch.matmul``
    (nothing of the AXS-6 path takes part), and so is this one."""
    from .backend import accelerated_matmul
    if not quantize_inputs:
        return torch.matmul(a, b)
    a = _accel_fq(a, block_size, "nearest")
    b = _accel_fq(b, block_size, "nearest")
    if b.dim() <= 2:
        return accelerated_matmul(a, b)
    # batched right operand: one product per batch entry
    batch = torch.broadcast_shapes(a.shape[:-2], b.shape[:-2])
    a3 = a.expand(*batch, *a.shape[-2:]).reshape(-1, *a.shape[-2:])
    b3 = b.expand(*batch, *b.shape[-2:]).reshape(-1, *b.shape[-2:])
    out = torch.stack([accelerated_matmul(a3[i], b3[i]) for i in range(a3.shape[0])])
    return out.reshape(*batch, a.shape[-2], b.shape[-1])
