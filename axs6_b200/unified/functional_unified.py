"""Autograd functions of the NF5 path (mirror of ``axs/unified/functional_unified.py``)."""
from __future__ import annotations

from typing import Literal

import torch

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
