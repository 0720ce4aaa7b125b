"""V1 (uniform grid) surface: mirror of ``axs.nn`` for the accelerated path."""
from .functional import axs_linear, axs_matmul, fake_quantize
from .modules import AXSEmbedding, AXSLayerNorm, AXSLinear, AXSMultiheadAttention, convert_to_axs

__all__ = ["fake_quantize", "axs_linear", "axs_matmul", "AXSLinear", "AXSLayerNorm", "AXSEmbedding",
           "AXSMultiheadAttention", "convert_to_axs"]
