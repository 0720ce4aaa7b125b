"""Shared autograd function of the fp32 AXS-6 Linears (NF5 "unified" and uniform-grid V1).

Graph (both references): w_q = FQ(w) nearest, x_q = FQ(x) nearest (optional), y = x_q w_q^T + b;
backward: g_q = FQ(g) stochastic (optional), dx = g_q w_q, dw = g_q^T x_q, db = column sums of g_q
(axs/unified/functional_unified.py:89-170, axs/nn/functional.py:93-148).  Here every product
runs on the TF32 tensor cores over operands rounded to TF32, which keeps the result within
1e-3 (relative Frobenius) of an fp32 matmul of the fake-quantised operands; fp32 in, fp32 out.
bf16 inputs with bf16 weights take the bf16 tensor-core path instead.
"""
from __future__ import annotations

import torch

from . import ops

# Test hook, as in unified.mixed_precision: draws for the next backward's stochastic rounding.
_noise_for_next_backward: torch.Tensor | None = None


def _rows(t: torch.Tensor) -> torch.Tensor:
    t2 = t.reshape(-1, t.shape[-1])
    if t2.dtype not in (torch.float32, torch.bfloat16):
        t2 = t2.float()
    if t2.stride(-1) != 1 or (t2.shape[0] > 1 and t2.stride(0) < t2.shape[1]):
        t2 = t2.contiguous()
    return t2


class AXSLinearFP32Function(torch.autograd.Function):
    @staticmethod
    def forward(ctx, input, weight, bias, block_size, quantize_input, quantize_grad, grid, who):
        if not input.is_cuda:
            raise RuntimeError(f"{who} requires CUDA tensors")
        assert block_size in ops.VALID_BLOCK_SIZES, f"block_size must be one of {ops.VALID_BLOCK_SIZES}"
        x2 = _rows(input)
        w = weight if weight.dtype in (torch.float32, torch.bfloat16) else weight.float()
        w = w if w.stride(-1) == 1 else w.contiguous()
        all_bf16 = x2.dtype == torch.bfloat16 and w.dtype == torch.bfloat16
        tf32 = not all_bf16
        out_dtype = torch.bfloat16 if all_bf16 else torch.float32
        b32 = bias.float().contiguous() if bias is not None else None
        y, xq = ops.linear_fwd(x2, w, b32, block_size, grid, bool(quantize_input), out_dtype, tf32=tf32, fp32_accuracy=tf32)
        ctx.save_for_backward(xq, weight, bias)
        ctx.cfg = (block_size, bool(quantize_grad), grid, tf32, out_dtype, input.shape)
        return y.reshape(*input.shape[:-1], weight.shape[0])

    @staticmethod
    def backward(ctx, grad_output):
        global _noise_for_next_backward
        xq, weight, bias = ctx.saved_tensors
        block_size, quantize_grad, grid, tf32, out_dtype, in_shape = ctx.cfg
        N, K = weight.shape
        g2 = _rows(grad_output)
        M = g2.shape[0]
        w = weight if weight.dtype in (torch.float32, torch.bfloat16) else weight.float()
        w = w if w.stride(-1) == 1 else w.contiguous()
        noise, _noise_for_next_backward = _noise_for_next_backward, None
        dx, dw, db = ops.linear_bwd(g2, xq, w, M, N, K, block_size, grid, quantize_grad,
                                    ctx.needs_input_grad[0], ctx.needs_input_grad[1],
                                    bias is not None and ctx.needs_input_grad[2], out_dtype, noise, tf32=tf32,
                                    bias_from_quantized=True)
        if dx is not None:
            dx = dx.reshape(in_shape)
        if dw is not None and weight.dtype != torch.float32:
            dw = dw.to(weight.dtype)
        if db is not None and bias is not None and bias.dtype != torch.float32:
            db = db.to(bias.dtype)
        return dx, dw, db, None, None, None, None, None
