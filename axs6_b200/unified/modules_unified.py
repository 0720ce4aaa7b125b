"""Unified module: ``AXSLinearUnified`` and ``convert_to_axs_unified`` for Linear layers (mirror of
``axs/unified/modules_unified.py:43-113`` and the Linear branch of ``:271-368``)."""
from __future__ import annotations

import copy
import math

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..core import DEFAULT_BLOCK_SIZE
from .functional_unified import axs_linear_unified


class AXSLinearUnified(nn.Module):
    """``nn.Linear`` through the NF5 quantiser; ``_warmup_active`` bypasses quantisation."""

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
        self._warmup_active: bool = False
        self.reset_parameters()

    def reset_parameters(self) -> None:
        nn.init.kaiming_uniform_(self.weight, a=math.sqrt(5))
        if self.bias is not None:
            bound = 1 / math.sqrt(self.weight.shape[1])
            nn.init.uniform_(self.bias, -bound, bound)

    def forward(self, input: torch.Tensor) -> torch.Tensor:
        if self._warmup_active:
            return F.linear(input, self.weight, self.bias)
        return axs_linear_unified(input, self.weight, self.bias, self.block_size, self.quantize_input,
                                  self.quantize_grad)

    def extra_repr(self) -> str:
        return (f"in_features={self.in_features}, out_features={self.out_features}, bias={self.bias is not None}, "
                f"block_size={self.block_size}, quant_input={self.quantize_input}, quant_grad={self.quantize_grad}")


def convert_to_axs_unified(model: nn.Module, block_size: int = DEFAULT_BLOCK_SIZE, quantize_input: bool = True,
                           quantize_grad: bool = True, skip_layers: set[str] | None = None,
                           inplace: bool = False) -> nn.Module:
    """Swap every ``nn.Linear`` for :class:`AXSLinearUnified`, sharing the parameters."""
    if not inplace:
        model = copy.deepcopy(model)
    skip = skip_layers or set()

    def swap(parent: nn.Module, prefix: str) -> None:
        for name, child in list(parent.named_children()):
            full = f"{prefix}.{name}" if prefix else name
            if full in skip:
                continue
            if type(child) is nn.Linear:
                new = AXSLinearUnified(child.in_features, child.out_features, child.bias is not None, block_size,
                                       quantize_input, quantize_grad).to(child.weight.device)
                new.weight = child.weight
                if child.bias is not None:
                    new.bias = child.bias
                setattr(parent, name, new)
            else:
                swap(child, full)

    swap(model, "")
    return model
