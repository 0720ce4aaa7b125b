"""Unified modules (mirror of ``axs/unified/modules_unified.py``): ``AXSLinearUnified`` (:43-113),
``AXSLayerNormUnified`` (:120-144), ``AXSEmbeddingUnified`` (:151-185), ``AXSMultiheadAttentionUnified``
(:192-264) and ``convert_to_axs_unified`` (:271-368).  All of them reach the CUDA kernels through
``fake_quantize_unified`` / ``axs_linear_unified``."""
from __future__ import annotations

import copy
import math

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import ops
from ..core import DEFAULT_BLOCK_SIZE
from .functional_unified import axs_linear_unified, fake_quantize_unified


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


class AXSLayerNormUnified(nn.Module):
    """Plain LayerNorm: its output is not quantised, the Linear that follows quantises its own input."""

    def __init__(self, normalized_shape, eps: float = 1e-5) -> None:
        super().__init__()
        self.normalized_shape = [normalized_shape] if isinstance(normalized_shape, int) else list(normalized_shape)
        self.eps = eps
        self.weight = nn.Parameter(torch.ones(self.normalized_shape))
        self.bias = nn.Parameter(torch.zeros(self.normalized_shape))

    def forward(self, input: torch.Tensor) -> torch.Tensor:
        return F.layer_norm(input, self.normalized_shape, self.weight, self.bias, self.eps)


class _EmbeddingFQ(torch.autograd.Function):
    """fake_quantize_unified(F.embedding(index, weight)) as one kernel (modules_unified.py:181-185); straight-through
    gradient: the rows' gradients are summed into the table as in ``F.embedding``'s backward, the padding row gets none."""

    @staticmethod
    def forward(ctx, index, weight, padding_idx, block_size, grid=ops.GRID_NF5, out_dtype=None):
        ctx.save_for_backward(index)
        ctx.num_weights, ctx.padding_idx = weight.shape[0], -1 if padding_idx is None else padding_idx
        ctx.w_dtype = weight.dtype
        return ops.fake_quantize_gather(weight, index, block_size, grid, "nearest", out_dtype, who="AXSEmbedding")

    @staticmethod
    def backward(ctx, grad_output):
        (index,) = ctx.saved_tensors
        gw = torch.ops.aten.embedding_dense_backward(grad_output.contiguous(), index, ctx.num_weights, ctx.padding_idx, False)
        return None, gw.to(ctx.w_dtype), None, None, None, None


class AXSEmbeddingUnified(nn.Module):
    """Embedding whose looked-up rows (not the whole table) go through the NF5 fake-quantiser, with a
    straight-through gradient; ``_warmup_active`` returns the raw rows."""

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
        self._warmup_active: bool = False

    def forward(self, input: torch.Tensor) -> torch.Tensor:
        if self._warmup_active:
            return F.embedding(input, self.weight, self.padding_idx)
        if self.weight.is_cuda and input.is_cuda and self.weight.dtype in (torch.float32, torch.bfloat16):
            # gather and fake-quantise in one kernel: the raw rows never go to HBM
            return _EmbeddingFQ.apply(input, self.weight, self.padding_idx, self.block_size)
        return fake_quantize_unified(F.embedding(input, self.weight, self.padding_idx), self.block_size, "nearest")


class AXSMultiheadAttentionUnified(nn.Module):
    """Batch-first multi-head attention: q/k/v/out projections are :class:`AXSLinearUnified`, the scores
    and the softmax stay in full precision, and the attention weights are fake-quantised with stochastic
    rounding (blocks along the key dimension) before they multiply the values."""

    def __init__(self, embed_dim: int, num_heads: int, dropout: float = 0.0, bias: bool = True,
                 block_size: int = DEFAULT_BLOCK_SIZE) -> None:
        super().__init__()
        assert embed_dim % num_heads == 0, "embed_dim must be divisible by num_heads"
        self.embed_dim, self.num_heads, self.head_dim = embed_dim, num_heads, embed_dim // num_heads
        self.block_size, self.dropout = block_size, dropout
        self.q_proj, self.k_proj, self.v_proj, self.out_proj = (
            AXSLinearUnified(embed_dim, embed_dim, bias=bias, block_size=block_size) for _ in range(4))
        self.scale = self.head_dim ** -0.5

    def _heads(self, t: torch.Tensor) -> torch.Tensor:
        return t.reshape(t.shape[0], t.shape[1], self.num_heads, self.head_dim).transpose(1, 2)

    def forward(self, query: torch.Tensor, key: torch.Tensor, value: torch.Tensor,
                attn_mask: torch.Tensor | None = None) -> torch.Tensor:
        q, k, v = self._heads(self.q_proj(query)), self._heads(self.k_proj(key)), self._heads(self.v_proj(value))
        scores = torch.matmul(q, k.transpose(-2, -1)) * self.scale
        if attn_mask is not None:
            scores = scores + attn_mask
        weights = F.softmax(scores, dim=-1)
        if self.dropout > 0 and self.training:
            weights = F.dropout(weights, p=self.dropout)
        weights = fake_quantize_unified(weights, self.block_size, "stochastic")
        ctx = torch.matmul(weights, v).transpose(1, 2).reshape(query.shape[0], query.shape[1], self.embed_dim)
        return self.out_proj(ctx)


def convert_to_axs_unified(model: nn.Module, block_size: int = DEFAULT_BLOCK_SIZE, quantize_input: bool = True,
                           quantize_grad: bool = True, skip_layers: set[str] | None = None,
                           inplace: bool = False) -> nn.Module:
    """Swap ``nn.Linear`` (and the V1 ``AXSLinear``) for :class:`AXSLinearUnified`, ``nn.LayerNorm`` for
    :class:`AXSLayerNormUnified` and ``nn.Embedding`` for :class:`AXSEmbeddingUnified`; the new modules take
    over the old modules' parameters.  RMSNorm and other norms are left alone.  Deep copy unless ``inplace``."""
    from ..nn.modules import AXSEmbedding, AXSLayerNorm, AXSLinear
    if not inplace:
        model = copy.deepcopy(model)
    skip = skip_layers or set()
    already = (AXSLinearUnified, AXSLayerNormUnified, AXSEmbeddingUnified)

    def swap(parent: nn.Module, prefix: str) -> None:
        for name, child in list(parent.named_children()):
            full = f"{prefix}.{name}" if prefix else name
            if full in skip or isinstance(child, already):
                continue
            if isinstance(child, (nn.Linear, AXSLinear)):
                new = AXSLinearUnified(child.in_features, child.out_features, child.bias is not None, block_size,
                                       quantize_input, quantize_grad).to(child.weight.device)
                new.weight = child.weight
                if child.bias is not None:
                    new.bias = child.bias
                setattr(parent, name, new)
            elif isinstance(child, AXSLayerNorm) or (isinstance(child, nn.LayerNorm) and child.elementwise_affine
                                                     and child.bias is not None):
                new = AXSLayerNormUnified(list(child.normalized_shape), eps=child.eps).to(child.weight.device)
                new.weight, new.bias = child.weight, child.bias
                setattr(parent, name, new)
            elif isinstance(child, (nn.Embedding, AXSEmbedding)):
                new = AXSEmbeddingUnified(child.num_embeddings, child.embedding_dim, child.padding_idx, block_size)
                new = new.to(child.weight.device)
                new.weight = child.weight
                setattr(parent, name, new)
            else:
                swap(child, full)

    swap(model, "")
    return model
