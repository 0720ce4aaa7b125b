"""Entry points named like the reference's GPU launchers (``axs/unified/triton_kernels.py``).

The module keeps the reference's file and function names so call sites need no edit; nothing
here uses Triton -- the work is done by the sm_100a CUDA library.
"""
from __future__ import annotations

from typing import Literal

import torch

from .. import ops
from ..core import DEFAULT_BLOCK_SIZE, VALID_BLOCK_SIZES


def triton_fused_fake_quantize(tensor: torch.Tensor, block_size: int = DEFAULT_BLOCK_SIZE,
                               rounding: Literal["nearest", "stochastic"] = "nearest", *,
                               n_blocks: int = 32) -> torch.Tensor:
    """NF5 fake-quantise of a CUDA tensor, same shape and dtype (triton_kernels.py:295-370).
    ``n_blocks`` was a tile-size knob of the reference kernel and is accepted and ignored."""
    if not tensor.is_cuda:
        raise RuntimeError("triton_fused_fake_quantize requires a CUDA tensor")
    assert block_size in VALID_BLOCK_SIZES, f"block_size must be one of {VALID_BLOCK_SIZES}"
    return ops.fake_quantize(tensor, block_size, ops.GRID_NF5, rounding, who="triton_fused_fake_quantize")
