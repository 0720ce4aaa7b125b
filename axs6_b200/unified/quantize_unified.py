"""NF5 fake-quantise and NF5 codes on the GPU.

Same names, arguments and results as ``axs/unified/quantize_unified.py``:
``fused_fake_quantize`` (:121-204), ``quantize_unified`` (:211-282), ``dequantize_unified``
(:285-308).  The three tables are exposed for inspection only (host copies of what the kernels
bake in); they are rebuilt from the 32 codebook bit patterns and the code boundaries, not
recomputed from erfinv.
"""
from __future__ import annotations

from typing import Literal

import torch

from .. import ops
from ..core import DEFAULT_BLOCK_SIZE, VALID_BLOCK_SIZES, AXSTensor, _dequantize_planes, _quantize_planes

# fp32 bit patterns of the 32 half-normal levels (quantize_unified.py:50-58) and the first LUT
# index of every code (quantize_unified.py:68-114).
_CODEBOOK_BITS = [
    0x3c04b96e, 0x3cc7303e, 0x3d26292a, 0x3d68fc26, 0x3d96163b, 0x3db7eb43, 0x3dda0c14, 0x3dfc887b,
    0x3e0fb8b1, 0x3e216c8a, 0x3e3369c5, 0x3e45bb68, 0x3e586dbb, 0x3e6b8e8e, 0x3e7f2d9b, 0x3e89ae7a,
    0x3e9418d0, 0x3e9ee22e, 0x3eaa1958, 0x3eb5d02b, 0x3ec21ca7, 0x3ecf1a59, 0x3edcec91, 0x3eebc1b0,
    0x3efbd888, 0x3f06c4be, 0x3f10ab83, 0x3f1c0741, 0x3f2988ae, 0x3f3a8bf4, 0x3f5273dc, 0x3f800000,
]
_CODE_STARTS = [0, 17, 34, 50, 67, 84, 101, 118, 135, 153, 171, 189, 207, 226, 246, 266, 286, 307, 329, 352,
                376, 401, 428, 457, 488, 521, 559, 601, 651, 712, 794, 932]

NF5_CODEBOOK: torch.Tensor = torch.tensor(_CODEBOOK_BITS, dtype=torch.int64).to(torch.int32).view(torch.float32)
REVERSE_NF5_LUT: torch.Tensor = (torch.bucketize(torch.arange(1024), torch.tensor(_CODE_STARTS), right=True) - 1).to(torch.uint8)
FUSED_NF5_LUT: torch.Tensor = NF5_CODEBOOK[REVERSE_NF5_LUT.long()]
_LUT_MAX_IDX: int = 1023


def fused_fake_quantize(tensor: torch.Tensor, block_size: int = DEFAULT_BLOCK_SIZE,
                        rounding: Literal["nearest", "stochastic"] = "nearest") -> torch.Tensor:
    """NF5 quantise-dequantise in one kernel; same shape and dtype as the input
    (reference: quantize_unified.py:121-204)."""
    assert block_size in VALID_BLOCK_SIZES, f"block_size must be one of {VALID_BLOCK_SIZES}"
    return ops.fake_quantize(tensor, block_size, ops.GRID_NF5, rounding, who="fused_fake_quantize")


def fused_fake_quantize_host(tensor: torch.Tensor, out: torch.Tensor | None = None, block_size: int = DEFAULT_BLOCK_SIZE,
                             rounding: Literal["nearest", "stochastic"] = "nearest") -> torch.Tensor:
    """:func:`fused_fake_quantize` for a tensor in pinned host memory: computed on the GPU with the host-to-device
    copy, the kernel and the device-to-host copy pipelined over chunks of rows (``ops.fake_quantize_host``).  The
    reference's call on a CPU tensor runs its eager CPU path; here the work still happens on the device."""
    return ops.fake_quantize_host(tensor, out, block_size, ops.GRID_NF5, rounding)


def quantize_unified(tensor: torch.Tensor, block_size: int = DEFAULT_BLOCK_SIZE,
                     rounding: Literal["nearest", "stochastic"] = "nearest") -> AXSTensor:
    """NF5 codes as an ``AXSTensor`` (reference: quantize_unified.py:211-282)."""
    assert block_size in VALID_BLOCK_SIZES
    return _quantize_planes(tensor, block_size, rounding, ops.GRID_NF5, "quantize_unified")


def dequantize_unified(axs_tensor: AXSTensor) -> torch.Tensor:
    """codebook[magnitude] * 2^(exponent - 127), fp32 (reference: quantize_unified.py:285-308)."""
    return _dequantize_planes(axs_tensor, ops.GRID_NF5)


def quantization_error_unified(original: torch.Tensor, block_size: int = DEFAULT_BLOCK_SIZE) -> dict[str, float]:
    """Error statistics of the NF5 fake-quantise (reference: quantize_unified.py:315-339)."""
    import math
    rec = fused_fake_quantize(original, block_size=block_size)
    err = (original - rec).float()
    mse = err.pow(2).mean().item()
    sig = original.float().pow(2).mean().item()
    return {"mse": mse, "rmse": math.sqrt(mse), "max_abs_error": err.abs().max().item(),
            "mean_abs_error": err.abs().mean().item(),
            "signal_to_noise_db": 10 * math.log10(sig / max(mse, 1e-45))}
