"""axs6_b200 -- B200 (sm_100a) implementation of the AXS-6 hot path.

Mirrors the module layout and function names of the reference package ``axs`` for the path it
covers (fake-quantise, 6-bit codec, AXS-6 Linear), so ``import axs6_b200 as axs`` drops in for
that path.  All arithmetic runs in hand-written CUDA kernels behind a C ABI
(``include/axs6_b200.h``); there is no CPU or PyTorch fallback.
"""
from .core import (AXS6_EXPONENT_BIAS, AXS6_MAX_MAGNITUDE, DEFAULT_BLOCK_SIZE, VALID_BLOCK_SIZES, AXSBlock, AXSTensor,
                   BlockConfig, axs_decode_block, axs_encode_block, dequantize, quantization_error, quantize)
from .quantize import RoundingMode, quantize_nearest, quantize_stochastic, quantize_with_error_feedback

__all__ = ["AXSBlock", "AXSTensor", "BlockConfig", "quantize", "dequantize", "axs_encode_block", "axs_decode_block",
           "quantization_error", "RoundingMode", "quantize_nearest", "quantize_stochastic", "quantize_with_error_feedback",
           "DEFAULT_BLOCK_SIZE", "VALID_BLOCK_SIZES", "AXS6_EXPONENT_BIAS", "AXS6_MAX_MAGNITUDE"]
__version__ = "0.1.0"
