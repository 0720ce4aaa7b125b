"""V1 functional ops (mirror of ``axs/nn/functional.py``)."""
from __future__ import annotations

from typing import Literal

import torch

from .. import ops
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
