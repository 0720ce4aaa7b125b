"""V1 (uniform grid) surface: mirror of ``axs.nn``."""
from .functional import axs_conv2d, axs_linear, axs_matmul, fake_quantize
from .modules import AXSConv2d, AXSEmbedding, AXSLayerNorm, AXSLinear, AXSMultiheadAttention, convert_to_axs
from .optim import AXSAdamW, AXSTrainingWrapper

__all__ = ["fake_quantize", "axs_linear", "axs_matmul", "axs_conv2d", "AXSLinear", "AXSConv2d", "AXSLayerNorm",
           "AXSEmbedding", "AXSMultiheadAttention", "convert_to_axs", "AXSAdamW", "AXSTrainingWrapper"]
