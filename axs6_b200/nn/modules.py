"""V1 module: ``AXSLinear`` (mirror of ``axs/nn/modules.py:36-102``)."""
from __future__ import annotations

import math

import torch
import torch.nn as nn

from ..core import DEFAULT_BLOCK_SIZE
from .functional import axs_linear


class AXSLinear(nn.Module):
    """``nn.Linear`` whose weights, activations and gradients pass through the uniform-grid
    AXS-6 quantiser."""

    def __init__(self, in_features: int, out_features: int, bias: bool = True,
                 block_size: int = DEFAULT_BLOCK_SIZE, quantize_input: bool = True,
                 quantize_grad: bool = True) -> None:
        super().__init__()
        self.in_features, self.out_features = in_features, out_features
        self.block_size, self.quantize_input, self.quantize_grad = block_size, quantize_input, quantize_grad
        self.weight = nn.Parameter(torch.empty(out_features, in_features))
        if bias:
            self.bias = nn.Parameter(torch.empty(out_features))
        else:
            self.register_parameter("bias", None)
        self.reset_parameters()

    def reset_parameters(self) -> None:
        nn.init.kaiming_uniform_(self.weight, a=math.sqrt(5))
        if self.bias is not None:
            bound = 1 / math.sqrt(self.weight.shape[1])
            nn.init.uniform_(self.bias, -bound, bound)

    def forward(self, input: torch.Tensor) -> torch.Tensor:
        return axs_linear(input, self.weight, self.bias, self.block_size, self.quantize_input, self.quantize_grad)

    def extra_repr(self) -> str:
        return (f"in_features={self.in_features}, out_features={self.out_features}, bias={self.bias is not None}, "
                f"block_size={self.block_size}, quantize_input={self.quantize_input}, quantize_grad={self.quantize_grad}")
