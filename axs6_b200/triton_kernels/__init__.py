"""Launchers named like the reference's first-generation GPU kernels (``axs/triton_kernels``): uniform-grid
quantise / dequantise / fake-quantise of 2-D tensors and the quantised matmul.  Nothing here uses Triton; the
work is done by the sm_100a CUDA library."""
from .matmul_kernel import triton_axs_matmul
from .quantize_kernel import triton_dequantize, triton_fake_quantize, triton_quantize

TRITON_AVAILABLE = False          # kept for call sites that test it; the functions below do not need it

__all__ = ["TRITON_AVAILABLE", "triton_quantize", "triton_dequantize", "triton_fake_quantize", "triton_axs_matmul"]
