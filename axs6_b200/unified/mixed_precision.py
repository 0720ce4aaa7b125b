"""AXS-6 Linear with bf16 tensor-core compute and fp32 master weights.

Same names, arguments and dtypes as ``axs/unified/mixed_precision.py``: the autograd function
(:65-155), ``axs_linear_mixed_precision`` (:158-185), the module ``AXSLinearMixedPrecision``
(:193-269) and ``convert_to_axs_mixed_precision`` (:277-349).  Forward and backward each run as
one C-ABI call: fake-quantise kernels for the operands, then the tcgen05 GEMMs.
"""
from __future__ import annotations

import math

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import ops
from ..core import DEFAULT_BLOCK_SIZE, VALID_BLOCK_SIZES

# Keep the forward's quantised weight (bf16, N x K) alive until backward instead of recomputing it there:
# one fake-quantise pass less per layer and step, for 2 bytes per weight of extra memory between the two.
KEEP_QUANTIZED_WEIGHT = True

# Quantise-on-load variant: activations, weight and gradient go to HBM as 6-bit codes (0.78 bytes per value instead
# of 2) and the GEMMs decode them in shared memory; the activation saved for backward shrinks by 2.56x.  Off by
# default: the two-pass path is the one that reproduces the reference at exact zeros (codes have no zero).
PACKED_OPERANDS = False

# Saved activation as 25-byte wire records (0.78 bytes per value instead of 2) WITHOUT the decode-on-load GEMM: the
# forward packs the bf16 input once more (the codes decode to the fake-quantised input, except at exact zeros, which
# codes cannot express), the backward unpacks them into a transient bf16 buffer for the weight-gradient product.
# Costs one pack and one unpack pass per layer and step (about 6 % of the step at 16384 x 4096 x 4096).  Off by
# default for the same reason as PACKED_OPERANDS.
SAVE_PACKED_INPUT = False

# Test hook: when set to a tensor, the next backward uses these U[0,1) draws for the gradient's
# stochastic rounding (padded (M, nblk, block) layout) instead of the Philox stream.
_noise_for_next_backward: torch.Tensor | None = None


def _rows(t: torch.Tensor) -> torch.Tensor:
    t2 = t.reshape(-1, t.shape[-1])
    if t2.dtype not in (torch.float32, torch.bfloat16):
        t2 = t2.float()
    if t2.stride(-1) != 1 or (t2.shape[0] > 1 and t2.stride(0) < t2.shape[1]):
        t2 = t2.contiguous()
    return t2


class _AXSLinearBF16Function(torch.autograd.Function):
    """Forward: cast to bf16, NF5 fake-quantise weight (always) and input (optionally), bf16
    GEMM with fp32 accumulation, bf16 output.  Saved: the quantised bf16 input, the leaf weight,
    the bias.  Backward: recompute the quantised weight, stochastic fake-quantise of the bf16
    gradient, dX in bf16, dW and db in fp32 (mixed_precision.py:86-155)."""

    @staticmethod
    def forward(ctx, input, weight, bias, block_size, quantize_input, quantize_grad):
        if not input.is_cuda:
            raise RuntimeError("axs_linear_mixed_precision requires CUDA tensors")
        assert block_size in VALID_BLOCK_SIZES, f"block_size must be one of {VALID_BLOCK_SIZES}"
        x2 = _rows(input)
        w = weight if weight.dtype in (torch.float32, torch.bfloat16) else weight.float()
        w = w if w.stride(-1) == 1 else w.contiguous()
        b32 = None
        if bias is not None:                      # F.linear sees bf16(bias): rounded inside the GEMM epilogue
            b32 = bias if (bias.dtype == torch.float32 and bias.is_contiguous()) else bias.float().contiguous()
        packed = PACKED_OPERANDS and x2.shape[0] % 8 == 0 and ops.linear_packed_ok(
            weight.shape[0], weight.shape[1], block_size, bool(quantize_input), bool(quantize_grad))
        y, xq, wq = ops.linear_fwd(x2, w, b32, block_size, ops.GRID_NF5, bool(quantize_input), torch.bfloat16,
                                   bias_via_bf16=True, return_wq=True, packed=packed)
        ctx.packed = packed
        ctx.x_records = None
        if (SAVE_PACKED_INPUT and not packed and quantize_input and block_size == 32 and x2.shape[1] % 32 == 0
                and ctx.needs_input_grad[1]):
            xb = x2 if x2.dtype == torch.bfloat16 else x2.to(torch.bfloat16)
            ctx.x_records = (x2.shape[0], x2.shape[1])
            xq = ops.pack(xb, 32, ops.GRID_NF5, "nearest", ops.LAYOUT_WIRE, who="axs_linear_mixed_precision")
        ctx.save_for_backward(xq, weight, bias)
        # The quantised weight is kept for backward and used there if the weight is still the same version
        # (the reference recomputes it, mixed_precision.py:130, to save memory; the bits are the same).
        ctx.wq = wq if KEEP_QUANTIZED_WEIGHT else None
        ctx.w_version = weight._version
        ctx.block_size = block_size
        ctx.quantize_grad = bool(quantize_grad)
        ctx.in_shape = input.shape
        return y.reshape(*input.shape[:-1], weight.shape[0])

    @staticmethod
    def backward(ctx, grad_output):
        global _noise_for_next_backward
        xq, weight, bias = ctx.saved_tensors
        N, K = weight.shape
        g2 = _rows(grad_output)
        M = g2.shape[0]
        w = weight if weight.dtype in (torch.float32, torch.bfloat16) else weight.float()
        w = w if w.stride(-1) == 1 else w.contiguous()
        noise, _noise_for_next_backward = _noise_for_next_backward, None
        if ctx.x_records is not None:             # the saved activation is a buffer of records: back to bf16 for the product
            xq = ops.unpack(ops.LAYOUT_WIRE, xq, ctx.x_records[0], ctx.x_records[1], 32, ops.GRID_NF5, torch.bfloat16)
        dx, dw, db = ops.linear_bwd(g2, xq, w, M, N, K, ctx.block_size, ops.GRID_NF5, ctx.quantize_grad,
                                    ctx.needs_input_grad[0], ctx.needs_input_grad[1],
                                    bias is not None and ctx.needs_input_grad[2], torch.bfloat16, noise,
                                    wq=ctx.wq if weight._version == ctx.w_version else None, packed=ctx.packed)
        ctx.wq = None
        if dx is not None:
            dx = dx.reshape(ctx.in_shape)
        return dx, dw, db, None, None, None


def axs_linear_mixed_precision(input: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None = None,
                               block_size: int = DEFAULT_BLOCK_SIZE, quantize_input: bool = True,
                               quantize_grad: bool = True) -> torch.Tensor:
    """bf16 output ``(*, out_features)``; fp32 weight gradient (mixed_precision.py:158-185)."""
    return _AXSLinearBF16Function.apply(input, weight, bias, block_size, quantize_input, quantize_grad)


class AXSLinearMixedPrecision(nn.Module):
    """Drop-in ``nn.Linear`` replacement: fp32 master weights, AXS-6 NF5 fake-quantised bf16
    compute (mixed_precision.py:193-269).  ``_warmup_active`` bypasses quantisation."""

    def __init__(self, in_features: int, out_features: int, bias: bool = True,
                 block_size: int = DEFAULT_BLOCK_SIZE, quantize_input: bool = True,
                 quantize_grad: bool = True) -> None:
        super().__init__()
        self.in_features = in_features
        self.out_features = out_features
        self.block_size = block_size
        self.quantize_input = quantize_input
        self.quantize_grad = quantize_grad
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
            return F.linear(input.to(torch.bfloat16), self.weight.to(torch.bfloat16),
                            self.bias.to(torch.bfloat16) if self.bias is not None else None)
        return axs_linear_mixed_precision(input, self.weight, self.bias, self.block_size, self.quantize_input,
                                          self.quantize_grad)

    def extra_repr(self) -> str:
        return (f"in_features={self.in_features}, out_features={self.out_features}, "
                f"bias={self.bias is not None}, block_size={self.block_size}, "
                f"quant_input={self.quantize_input}, quant_grad={self.quantize_grad}, mixed_precision=bf16")


def convert_to_axs_mixed_precision(model: nn.Module, block_size: int = DEFAULT_BLOCK_SIZE,
                                   quantize_input: bool = True, quantize_grad: bool = True,
                                   skip_layers: set[str] | None = None, inplace: bool = False) -> nn.Module:
    """Replace every ``nn.Linear`` -- and the V1 / unified AXS-6 Linear modules of this package --
    by :class:`AXSLinearMixedPrecision` with fp32 copies of their parameters; deep copy unless
    ``inplace`` (mixed_precision.py:277-349)."""
    import copy
    from ..nn.modules import AXSLinear
    from .modules_unified import AXSLinearUnified
    if not inplace:
        model = copy.deepcopy(model)
    skip = skip_layers or set()
    linear_types = (nn.Linear, AXSLinear, AXSLinearUnified)

    def swap(parent: nn.Module, prefix: str) -> None:
        for name, child in list(parent.named_children()):
            full = f"{prefix}.{name}" if prefix else name
            if full in skip:
                continue
            if isinstance(child, linear_types) and not isinstance(child, AXSLinearMixedPrecision):
                new = AXSLinearMixedPrecision(child.in_features, child.out_features, child.bias is not None,
                                              block_size, quantize_input, quantize_grad)
                new.weight.data.copy_(child.weight.data.float())
                if child.bias is not None:
                    new.bias.data.copy_(child.bias.data.float())
                setattr(parent, name, new.to(child.weight.device))
            else:
                swap(child, full)

    swap(model, "")
    return model


def estimate_memory_savings(model: nn.Module, batch_size: int = 1, seq_len: int = 1) -> dict[str, float]:
    """Activation memory kept for backward by the mixed-precision Linears of ``model``: fp32 baseline
    (quantised input and quantised weight in fp32) against this scheme (quantised input in bf16, weight
    recomputed), in MiB, and their ratio (mixed_precision.py:357-401)."""
    fp32_bytes = 0
    bf16_bytes = 0
    for m in model.modules():
        if isinstance(m, AXSLinearMixedPrecision):
            act = batch_size * seq_len * m.in_features
            fp32_bytes += (act + m.out_features * m.in_features) * 4
            bf16_bytes += act * 2
    fp32_mb, bf16_mb = fp32_bytes / 2 ** 20, bf16_bytes / 2 ** 20
    return {"fp32_mb": round(fp32_mb, 2), "bf16_recomp_mb": round(bf16_mb, 2),
            "savings_ratio": round(fp32_mb / bf16_mb, 1) if bf16_mb > 0 else float("inf")}
