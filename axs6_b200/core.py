"""Uniform-grid (V1) AXS-6 tensor quantisation on the GPU.

Same names, arguments and results as ``axs/core.py`` of the reference for the tensor-level
entry points: ``quantize`` (core.py:294-369), ``dequantize`` (core.py:372-403) and the
``AXSTensor`` container (core.py:160-206), plus whole-tensor serialisation in the 26-byte
block layout that ``AXSBlock.to_bytes`` / ``from_bytes`` (core.py:97-152) define per block.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Literal

import torch

from . import ops

AXS6_MANTISSA_BITS: int = 5
AXS6_SIGN_BITS: int = 1
AXS6_VALUE_BITS: int = 6
AXS6_EXPONENT_BITS: int = 8
AXS6_CONFIG_BITS: int = 2
AXS6_HEADER_BITS: int = 10
AXS6_MAX_MAGNITUDE: int = 31
AXS6_EXPONENT_BIAS: int = 127
DEFAULT_BLOCK_SIZE: int = 32
VALID_BLOCK_SIZES: tuple[int, ...] = (8, 16, 32)


@dataclass
class AXSTensor:
    """Planes of a quantised tensor (field for field the reference's container):
    ``shared_exponents`` u8 ``(rows, num_blocks)``, ``signs`` bool and ``magnitudes`` u8
    ``(rows, num_blocks, block_size)``; rows = product of the leading dimensions."""

    shared_exponents: torch.Tensor
    signs: torch.Tensor
    magnitudes: torch.Tensor
    block_size: int
    original_shape: torch.Size
    num_blocks: int

    @property
    def effective_bits_per_value(self) -> float:
        return AXS6_VALUE_BITS + AXS6_HEADER_BITS / self.block_size

    @property
    def compression_ratio_vs_fp32(self) -> float:
        return 32.0 / self.effective_bits_per_value

    @property
    def compression_ratio_vs_fp8(self) -> float:
        return 8.0 / self.effective_bits_per_value

    @property
    def memory_bytes(self) -> int:
        numel = 1
        for s in self.original_shape:
            numel *= s
        bits = numel * AXS6_VALUE_BITS + (numel // self.block_size) * AXS6_HEADER_BITS
        return math.ceil(bits / 8)


def _quantize_planes(tensor: torch.Tensor, block_size: int, rounding: str, grid: int, who: str,
                     noise: torch.Tensor | None = None) -> AXSTensor:
    assert block_size in VALID_BLOCK_SIZES, f"Block size must be one of {VALID_BLOCK_SIZES}"
    se, sg, mg = ops.pack(tensor, block_size, grid, rounding, ops.LAYOUT_PLANES, noise=noise, who=who)
    return AXSTensor(shared_exponents=se, signs=sg, magnitudes=mg, block_size=block_size,
                     original_shape=tensor.shape, num_blocks=se.shape[-1])


def _dequantize_planes(axs_tensor: AXSTensor, grid: int) -> torch.Tensor:
    shape = axs_tensor.original_shape
    cols = shape[-1]
    rows = axs_tensor.magnitudes.shape[0]
    y = ops.unpack(ops.LAYOUT_PLANES, (axs_tensor.shared_exponents, axs_tensor.signs, axs_tensor.magnitudes),
                   rows, cols, axs_tensor.block_size, grid, torch.float32)
    return y.reshape(shape)


def quantize(tensor: torch.Tensor, block_size: int = DEFAULT_BLOCK_SIZE,
             rounding: Literal["nearest", "stochastic"] = "nearest") -> AXSTensor:
    """Uniform-grid quantisation of the last dimension in blocks (reference: core.py:294-369)."""
    return _quantize_planes(tensor, block_size, rounding, ops.GRID_UNIFORM, "quantize")


def dequantize(axs_tensor: AXSTensor) -> torch.Tensor:
    """Back to fp32 with the original shape (reference: core.py:372-403)."""
    return _dequantize_planes(axs_tensor, ops.GRID_UNIFORM)


def tensor_to_bytes(tensor: torch.Tensor, block_size: int = DEFAULT_BLOCK_SIZE,
                    rounding: Literal["nearest", "stochastic"] = "nearest", nf5: bool = False) -> torch.Tensor:
    """Quantise and serialise every block as ``AXSBlock.to_bytes`` does (core.py:97-118): a u16
    little-endian header ``(exponent << 2) | config`` (config 0 = dense) followed by the 6-bit
    codes as a little-endian bit stream; 26 bytes per block of 32.  Returns a flat uint8 tensor of
    ``rows * num_blocks`` records in row-major block order."""
    return ops.pack(tensor, block_size, ops.GRID_NF5 if nf5 else ops.GRID_UNIFORM, rounding, ops.LAYOUT_SPEC,
                    who="tensor_to_bytes")


def tensor_from_bytes(data: torch.Tensor, shape, block_size: int = DEFAULT_BLOCK_SIZE, nf5: bool = False,
                      dtype: torch.dtype = torch.float32) -> torch.Tensor:
    """Inverse of :func:`tensor_to_bytes` (per block: core.py:120-152, then dequantise)."""
    shape = torch.Size(shape)
    cols = shape[-1]
    rows = 1
    for s in shape[:-1]:
        rows *= s
    y = ops.unpack(ops.LAYOUT_SPEC, data, rows, cols, block_size, ops.GRID_NF5 if nf5 else ops.GRID_UNIFORM, dtype)
    return y.reshape(shape)
