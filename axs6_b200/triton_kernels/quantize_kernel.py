"""``triton_quantize`` / ``triton_dequantize`` / ``triton_fake_quantize`` of the reference
(``axs/triton_kernels/quantize_kernel.py:224-346``) on the CUDA kernels: uniform grid (magnitudes 0..31),
2-D input whose row length is a multiple of the block size.

One deliberate difference: the reference's kernels round with ``floor(x + 0.5)``, its eager path (which is the
parity target of this package) with round-half-to-even; results differ only on exact ties, and these functions
follow the eager path, like every other entry point here.
"""
from __future__ import annotations

import torch

from .. import ops


def _check(tensor: torch.Tensor, block_size: int, who: str) -> None:
    if not tensor.is_cuda:
        raise RuntimeError(f"{who} requires a CUDA tensor")
    assert tensor.ndim == 2, "Input must be 2D"
    assert block_size in ops.VALID_BLOCK_SIZES, f"block_size must be one of {ops.VALID_BLOCK_SIZES}"
    assert tensor.shape[1] % block_size == 0, f"D ({tensor.shape[1]}) must be a multiple of block_size ({block_size})"


def triton_quantize(tensor: torch.Tensor, block_size: int = 32, stochastic: bool = False):
    """-> ``(exponents (N, nblk) uint8, signs (N, D) bool, magnitudes (N, D) uint8)``."""
    _check(tensor, block_size, "triton_quantize")
    se, sg, mg = ops.pack(tensor, block_size, ops.GRID_UNIFORM, "stochastic" if stochastic else "nearest",
                          ops.LAYOUT_PLANES, who="triton_quantize")
    n, d = tensor.shape
    return se, sg.reshape(n, d), mg.reshape(n, d)


def triton_dequantize(exponents: torch.Tensor, signs: torch.Tensor, magnitudes: torch.Tensor,
                      block_size: int = 32) -> torch.Tensor:
    """-> fp32 ``(N, nblk * block_size)``."""
    n, nblk = exponents.shape
    d = nblk * block_size
    return ops.unpack(ops.LAYOUT_PLANES, (exponents, signs.reshape(n, nblk, block_size), magnitudes.reshape(n, nblk, block_size)),
                      n, d, block_size, ops.GRID_UNIFORM, torch.float32)


def triton_fake_quantize(tensor: torch.Tensor, block_size: int = 32, stochastic: bool = False) -> torch.Tensor:
    """Quantise + dequantise in one kernel; same shape and dtype as the input."""
    _check(tensor, block_size, "triton_fake_quantize")
    return ops.fake_quantize(tensor, block_size, ops.GRID_UNIFORM, "stochastic" if stochastic else "nearest",
                             who="triton_fake_quantize")
