"""V1 (uniform grid) modules, mirror of ``axs/nn/modules.py``: ``AXSLinear`` (:36-102), ``AXSLayerNorm`` (:190-216),
``AXSEmbedding`` (:223-252), ``AXSMultiheadAttention`` (:259-319), ``AXSConv2d`` (:110-183: this package's
quantiser around the library's convolution) and ``convert_to_axs`` (:326-411)."""
from __future__ import annotations

import math

import copy

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..core import DEFAULT_BLOCK_SIZE
from .functional import axs_conv2d, axs_linear, fake_quantize


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


class AXSConv2d(nn.Module):
    """``nn.Conv2d`` whose weight, input and gradient pass through the uniform-grid quantiser."""

    def __init__(self, in_channels: int, out_channels: int, kernel_size, stride=1, padding=0, dilation=1,
                 groups: int = 1, bias: bool = True, block_size: int = DEFAULT_BLOCK_SIZE) -> None:
        super().__init__()
        as_pair = lambda v: v if isinstance(v, tuple) else (v, v)
        self.in_channels, self.out_channels, self.groups, self.block_size = in_channels, out_channels, groups, block_size
        self.kernel_size, self.stride = as_pair(kernel_size), as_pair(stride)
        self.padding, self.dilation = as_pair(padding), as_pair(dilation)
        self.weight = nn.Parameter(torch.empty(out_channels, in_channels // groups, *self.kernel_size))
        if bias:
            self.bias = nn.Parameter(torch.empty(out_channels))
        else:
            self.register_parameter("bias", None)
        self.reset_parameters()

    def reset_parameters(self) -> None:
        nn.init.kaiming_uniform_(self.weight, a=math.sqrt(5))
        if self.bias is not None:
            bound = 1 / math.sqrt(self.weight.shape[1] * self.kernel_size[0] * self.kernel_size[1])
            nn.init.uniform_(self.bias, -bound, bound)

    def forward(self, input: torch.Tensor) -> torch.Tensor:
        return axs_conv2d(input, self.weight, self.bias, self.stride, self.padding, self.dilation, self.groups,
                          self.block_size)

    def extra_repr(self) -> str:
        return (f"{self.in_channels}, {self.out_channels}, kernel_size={self.kernel_size}, stride={self.stride}, "
                f"padding={self.padding}, block_size={self.block_size}")


class AXSLayerNorm(nn.Module):
    """LayerNorm in full precision whose OUTPUT is fake-quantised on the uniform grid."""

    def __init__(self, normalized_shape, eps: float = 1e-5, block_size: int = DEFAULT_BLOCK_SIZE) -> None:
        super().__init__()
        self.normalized_shape = [normalized_shape] if isinstance(normalized_shape, int) else list(normalized_shape)
        self.eps, self.block_size = eps, block_size
        self.weight = nn.Parameter(torch.ones(self.normalized_shape))
        self.bias = nn.Parameter(torch.zeros(self.normalized_shape))

    def forward(self, input: torch.Tensor) -> torch.Tensor:
        return fake_quantize(F.layer_norm(input, self.normalized_shape, self.weight, self.bias, self.eps), self.block_size)


class AXSEmbedding(nn.Module):
    """Embedding whose looked-up rows are fake-quantised on the uniform grid (straight-through gradient)."""

    def __init__(self, num_embeddings: int, embedding_dim: int, padding_idx: int | None = None,
                 block_size: int = DEFAULT_BLOCK_SIZE) -> None:
        super().__init__()
        self.num_embeddings, self.embedding_dim = num_embeddings, embedding_dim
        self.padding_idx, self.block_size = padding_idx, block_size
        self.weight = nn.Parameter(torch.empty(num_embeddings, embedding_dim))
        nn.init.normal_(self.weight)
        if padding_idx is not None:
            with torch.no_grad():
                self.weight[padding_idx].zero_()

    def forward(self, input: torch.Tensor) -> torch.Tensor:
        if self.weight.is_cuda and input.is_cuda and self.weight.dtype in (torch.float32, torch.bfloat16):
            from .. import ops
            from ..unified.modules_unified import _EmbeddingFQ     # gather and fake-quantise in one kernel, fp32 out
            return _EmbeddingFQ.apply(input, self.weight, self.padding_idx, self.block_size, ops.GRID_UNIFORM, torch.float32)
        return fake_quantize(F.embedding(input, self.weight, self.padding_idx), self.block_size)


class AXSMultiheadAttention(nn.Module):
    """Batch-first multi-head attention with :class:`AXSLinear` projections; scores, softmax and the weighted
    sum run in full precision."""

    def __init__(self, embed_dim: int, num_heads: int, dropout: float = 0.0, bias: bool = True,
                 block_size: int = DEFAULT_BLOCK_SIZE) -> None:
        super().__init__()
        assert embed_dim % num_heads == 0, "embed_dim must be divisible by num_heads"
        self.embed_dim, self.num_heads, self.head_dim = embed_dim, num_heads, embed_dim // num_heads
        self.block_size, self.dropout = block_size, dropout
        self.q_proj, self.k_proj, self.v_proj, self.out_proj = (
            AXSLinear(embed_dim, embed_dim, bias=bias, block_size=block_size) for _ in range(4))
        self.scale = self.head_dim ** -0.5

    def forward(self, query: torch.Tensor, key: torch.Tensor, value: torch.Tensor,
                attn_mask: torch.Tensor | None = None) -> torch.Tensor:
        def heads(t):
            return t.reshape(t.shape[0], t.shape[1], self.num_heads, self.head_dim).transpose(1, 2)
        q, k, v = heads(self.q_proj(query)), heads(self.k_proj(key)), heads(self.v_proj(value))
        scores = torch.matmul(q, k.transpose(-2, -1)) * self.scale
        if attn_mask is not None:
            scores = scores + attn_mask
        weights = F.softmax(scores, dim=-1)
        if self.dropout > 0 and self.training:
            weights = F.dropout(weights, p=self.dropout)
        ctx = torch.matmul(weights, v).transpose(1, 2).reshape(query.shape[0], query.shape[1], self.embed_dim)
        return self.out_proj(ctx)


def convert_to_axs(model: nn.Module, block_size: int = DEFAULT_BLOCK_SIZE, quantize_input: bool = True,
                   quantize_grad: bool = True, skip_layers: set[str] | None = None, inplace: bool = False) -> nn.Module:
    """Swap ``nn.Linear`` / ``nn.Conv2d`` / ``nn.LayerNorm`` / ``nn.Embedding`` for their V1 AXS-6 counterparts, which
    take over the old modules' parameters; deep copy unless ``inplace``."""
    if not inplace:
        model = copy.deepcopy(model)
    skip = skip_layers or set()

    def swap(parent: nn.Module, prefix: str) -> None:
        for name, child in list(parent.named_children()):
            full = f"{prefix}.{name}" if prefix else name
            if full in skip or isinstance(child, (AXSLinear, AXSConv2d, AXSLayerNorm, AXSEmbedding)):
                continue
            if isinstance(child, nn.Linear):
                new = AXSLinear(child.in_features, child.out_features, child.bias is not None, block_size,
                                quantize_input, quantize_grad).to(child.weight.device)
                new.weight = child.weight
                if child.bias is not None:
                    new.bias = child.bias
                setattr(parent, name, new)
            elif isinstance(child, nn.Conv2d) and isinstance(child.padding, tuple) and child.padding_mode == "zeros":
                new = AXSConv2d(child.in_channels, child.out_channels, child.kernel_size, child.stride, child.padding,
                                child.dilation, child.groups, child.bias is not None, block_size).to(child.weight.device)
                new.weight = child.weight
                if child.bias is not None:
                    new.bias = child.bias
                setattr(parent, name, new)
            elif isinstance(child, nn.LayerNorm) and child.elementwise_affine and child.bias is not None:
                new = AXSLayerNorm(list(child.normalized_shape), child.eps, block_size).to(child.weight.device)
                new.weight, new.bias = child.weight, child.bias
                setattr(parent, name, new)
            elif isinstance(child, nn.Embedding):
                new = AXSEmbedding(child.num_embeddings, child.embedding_dim, child.padding_idx, block_size)
                new = new.to(child.weight.device)
                new.weight = child.weight
                setattr(parent, name, new)
            else:
                swap(child, full)

    swap(model, "")
    return model
