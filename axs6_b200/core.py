"""Uniform-grid (V1) AXS-6 tensor quantisation on the GPU.

Same names, arguments and results as ``axs/core.py`` of the reference for the tensor-level
entry points: ``quantize`` (core.py:294-369), ``dequantize`` (core.py:372-403) and the
``AXSTensor`` container (core.py:160-206), plus whole-tensor serialisation in the 26-byte
block layout that ``AXSBlock.to_bytes`` / ``from_bytes`` (core.py:97-152) define per block.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from enum import IntEnum
from typing import Literal

import numpy as np
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


class BlockConfig(IntEnum):
    """2-bit mode field of a block header (core.py:44-50); only DENSE is produced."""

    DENSE = 0b00
    SPARSE = 0b01
    HIGH_PREC = 0b10
    RESERVED = 0b11


@dataclass
class AXSBlock:
    """One encoded block, field for field the reference's host-side container (core.py:59-152): the biased
    8-bit ``shared_exponent`` (scale = 2^(shared_exponent - 127)), the 2-bit ``config``, ``signs`` (bool, True =
    negative) and ``magnitudes`` (uint8 in [0, 31]), both of shape ``(block_size,)``.

    This is a format utility on numpy arrays for single blocks (the reference's is a Python loop);
    whole tensors go through :func:`tensor_to_bytes` / :func:`tensor_from_bytes`, which run on the GPU
    and produce the same bytes."""

    shared_exponent: int
    config: BlockConfig
    signs: np.ndarray
    magnitudes: np.ndarray
    block_size: int = DEFAULT_BLOCK_SIZE

    @property
    def scale(self) -> float:
        return math.ldexp(1.0, self.shared_exponent - AXS6_EXPONENT_BIAS)

    @property
    def total_bits(self) -> int:
        return AXS6_HEADER_BITS + self.block_size * AXS6_VALUE_BITS

    @property
    def bits_per_value(self) -> float:
        return self.total_bits / self.block_size

    def to_bytes(self) -> bytes:
        """u16 little-endian header ``(exponent << 2) | config``, then the codes ``(sign << 5) | magnitude`` as a
        little-endian stream of 6-bit fields (core.py:97-118): 2 + ceil(6 B / 8) bytes."""
        header = ((int(self.shared_exponent) << 2) | int(self.config)) & 0xFFFF
        codes = (np.asarray(self.signs, dtype=bool).astype(np.uint8) << 5) | (np.asarray(self.magnitudes, dtype=np.uint8) & 31)
        codes = codes[: self.block_size]
        field_bits = (codes[:, None] >> np.arange(6, dtype=np.uint8)) & 1            # (B, 6), least significant first
        payload = np.packbits(field_bits.reshape(-1).astype(np.uint8), bitorder="little")
        return header.to_bytes(2, "little") + payload.tobytes()

    @classmethod
    def from_bytes(cls, data: bytes, block_size: int = DEFAULT_BLOCK_SIZE) -> "AXSBlock":
        """Inverse of :meth:`to_bytes` (core.py:120-152)."""
        header = int.from_bytes(data[:2], "little")
        nbytes = (6 * block_size + 7) // 8
        stream = np.unpackbits(np.frombuffer(data[2:2 + nbytes], dtype=np.uint8), bitorder="little")[: 6 * block_size]
        codes = (stream.reshape(block_size, 6).astype(np.uint8) << np.arange(6, dtype=np.uint8)).sum(axis=1).astype(np.uint8)
        return cls(shared_exponent=header >> 2, config=BlockConfig(header & 3), signs=(codes >> 5).astype(bool),
                   magnitudes=(codes & 31).astype(np.uint8), block_size=block_size)


def axs_encode_block(values: np.ndarray, rounding: Literal["nearest", "stochastic"] = "nearest") -> AXSBlock:
    """Encode one block given as a 1-D array of 8, 16 or 32 values, in double precision on the host, following
    the reference's per-block encoder (core.py:214-270): exponent = floor(log2(max |v|)) + 1 + 127 clamped to
    [0, 255] (0 for an all-zero block), magnitude = round-half-even(|v| / scale * 31) clamped to [0, 31], or
    floor + Bernoulli(fraction) with ``np.random.uniform`` draws for ``"stochastic"``."""
    v = np.asarray(values, dtype=np.float64).reshape(-1)
    n = v.shape[0]
    assert n in VALID_BLOCK_SIZES, f"Block size must be one of {VALID_BLOCK_SIZES}"
    mag_abs = np.abs(v)
    top = float(mag_abs.max())
    if top == 0.0:
        return AXSBlock(0, BlockConfig.DENSE, np.zeros(n, dtype=bool), np.zeros(n, dtype=np.uint8), n)
    se = min(255, max(0, math.floor(math.log2(top)) + 1 + AXS6_EXPONENT_BIAS))
    steps = mag_abs / math.ldexp(1.0, se - AXS6_EXPONENT_BIAS) * AXS6_MAX_MAGNITUDE
    if rounding == "stochastic":
        low = np.floor(steps)
        draws = np.random.uniform(0, 1, size=n)
        q = low + (draws < (steps - low))
    else:
        q = np.round(steps)
    q = np.clip(q, 0, AXS6_MAX_MAGNITUDE).astype(np.uint8)
    return AXSBlock(se, BlockConfig.DENSE, v < 0, q, n)


def axs_decode_block(block: AXSBlock) -> np.ndarray:
    """float64 values of one block: magnitude / 31 * scale, negated where the sign is set (core.py:273-286)."""
    out = block.magnitudes.astype(np.float64) / AXS6_MAX_MAGNITUDE * block.scale
    return np.where(np.asarray(block.signs, dtype=bool), -out, out)


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


def quantization_error(original: torch.Tensor, block_size: int = DEFAULT_BLOCK_SIZE,
                       rounding: Literal["nearest", "stochastic"] = "nearest") -> dict[str, float]:
    """Error statistics of quantise -> dequantise on ``original`` (core.py:411-440): ``mse``, ``rmse``,
    ``max_abs_error``, ``mean_abs_error``, ``signal_to_noise_db``."""
    back = dequantize(quantize(original, block_size=block_size, rounding=rounding))
    err = (original - back).float()
    mse = err.pow(2).mean().item()
    power = original.float().pow(2).mean().item()
    return {"mse": mse, "rmse": math.sqrt(mse), "max_abs_error": err.abs().max().item(),
            "mean_abs_error": err.abs().mean().item(), "signal_to_noise_db": 10 * math.log10(power / max(mse, 1e-45))}


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
