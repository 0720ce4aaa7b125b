"""Entry points named like the reference's GPU launchers (``axs/unified/triton_kernels.py``).

The module keeps the reference's file and function names so call sites need no edit; nothing
here uses Triton -- the work is done by the sm_100a CUDA library.
"""
from __future__ import annotations

from typing import Literal

import torch

from .. import ops
from ..core import DEFAULT_BLOCK_SIZE, VALID_BLOCK_SIZES


def has_triton() -> bool:
    """The reference asks whether Triton can be imported (triton_kernels.py:50-53).  These launchers do not
    need it; the answer says whether they can run: a CUDA device and the library are present."""
    try:
        from .. import _lib
        return bool(torch.cuda.is_available() and _lib.load().axs6_query(0))
    except Exception:
        return False


def triton_fused_fake_quantize(tensor: torch.Tensor, block_size: int = DEFAULT_BLOCK_SIZE,
                               rounding: Literal["nearest", "stochastic"] = "nearest", *,
                               n_blocks: int = 32) -> torch.Tensor:
    """NF5 fake-quantise of a CUDA tensor, same shape and dtype (triton_kernels.py:295-370).
    ``n_blocks`` was a tile-size knob of the reference kernel and is accepted and ignored."""
    if not tensor.is_cuda:
        raise RuntimeError("triton_fused_fake_quantize requires a CUDA tensor")
    assert block_size in VALID_BLOCK_SIZES, f"block_size must be one of {VALID_BLOCK_SIZES}"
    return ops.fake_quantize(tensor, block_size, ops.GRID_NF5, rounding, who="triton_fused_fake_quantize")


def triton_fused_linear(input: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None = None,
                        block_size: int = DEFAULT_BLOCK_SIZE, quantize_input: bool = True) -> torch.Tensor:
    """``FQ(input) @ FQ(weight).T + bias`` computed in fp32 arithmetic (TF32 tensor cores), result
    cast back to the input dtype (triton_kernels.py:385-482).  Like the reference's fused kernel it
    accepts ``block_size=32`` only and raises ``ValueError`` otherwise; a ragged K behaves as if
    zero-padded."""
    if not input.is_cuda:
        raise RuntimeError("triton_fused_linear requires CUDA tensors")
    if block_size != 32:
        raise ValueError(f"triton_fused_linear requires block_size=32, got {block_size}. "
                         "Use the separate FQ + F.linear path for other block sizes.")
    orig_dtype = input.dtype
    x2 = input.reshape(-1, input.shape[-1]).contiguous().float()
    w = weight.contiguous().float()
    b32 = bias.float().contiguous() if bias is not None else None
    y, _ = ops.linear_fwd(x2, w, b32, 32, ops.GRID_NF5, bool(quantize_input), torch.float32, tf32=True, fp32_accuracy=True)
    y = y.reshape(*input.shape[:-1], weight.shape[0])
    return y if orig_dtype == torch.float32 else y.to(orig_dtype)
