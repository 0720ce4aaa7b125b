"""V1 (uniform grid) surface: mirror of ``axs.nn`` for the accelerated path."""
from .functional import axs_linear, axs_matmul, fake_quantize
from .modules import AXSLinear

__all__ = ["fake_quantize", "axs_linear", "axs_matmul", "AXSLinear"]
