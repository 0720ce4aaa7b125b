"""Gradient packing in the 25-byte wire layout (mirror of the codec half of
``axs/unified/distributed.py``: ``_pack_gradient`` :70-120, ``_unpack_gradient`` :123-144,
``_pack_to_flat_buffer`` :147-198, ``_unpack_from_flat_buffer`` :201-232).

``pack_wire`` / ``unpack_wire`` do value -> bytes and bytes -> value in ONE kernel each; the
four reference-named helpers are kept for call-site compatibility and go through the planes.
"""
from __future__ import annotations

import torch

from .. import ops
from ..core import DEFAULT_BLOCK_SIZE


def pack_wire(tensor: torch.Tensor, block_size: int = DEFAULT_BLOCK_SIZE, rounding: str = "nearest") -> torch.Tensor:
    """tensor -> flat int8 buffer: per block 1 exponent byte + 6-bit codes (25 B per 32 values)."""
    return ops.pack(tensor, block_size, ops.GRID_NF5, rounding, ops.LAYOUT_WIRE, who="pack_wire").view(torch.int8)


def unpack_wire(buffer: torch.Tensor, shape, block_size: int = DEFAULT_BLOCK_SIZE,
                dtype: torch.dtype = torch.float32) -> torch.Tensor:
    """Inverse of :func:`pack_wire`; returns a tensor of ``shape``."""
    shape = torch.Size(shape)
    rows = 1
    for s in shape[:-1]:
        rows *= s
    y = ops.unpack(ops.LAYOUT_WIRE, buffer.view(torch.uint8), rows, shape[-1], block_size, ops.GRID_NF5, dtype)
    return y.reshape(shape)


def _pack_gradient(tensor: torch.Tensor, block_size: int = DEFAULT_BLOCK_SIZE):
    se, sg, mg = ops.pack(tensor, block_size, ops.GRID_NF5, "nearest", ops.LAYOUT_PLANES, who="_pack_gradient")
    return se, sg, mg, tensor.shape


def _unpack_gradient(shared_exponents, signs, magnitudes, original_shape, block_size: int = DEFAULT_BLOCK_SIZE):
    rows = magnitudes.shape[0]
    y = ops.unpack(ops.LAYOUT_PLANES, (shared_exponents, signs, magnitudes), rows, original_shape[-1], block_size,
                   ops.GRID_NF5, torch.float32)
    return y.reshape(original_shape)
