"""NF5 ("unified") quantiser surface: same names as ``axs.unified`` for the accelerated path."""
from .quantize_unified import (FUSED_NF5_LUT, NF5_CODEBOOK, REVERSE_NF5_LUT, dequantize_unified,
                               fused_fake_quantize, quantize_unified)
from .backend import (BackendType, accelerated_fake_quantize, accelerated_linear, accelerated_matmul, backend_info,
                      clear_int8_weight_cache, detect_best_backend, get_backend, set_backend)
from .distributed import AXS6GradCompressor, axs6_gradient_hook, axs6_gradient_hook_packed
from .quantize_unified import quantization_error_unified
from .triton_kernels import has_triton, triton_fused_fake_quantize, triton_fused_linear
from .functional_unified import axs_linear_unified, axs_matmul_unified, fake_quantize_unified
from .mixed_precision import (AXSLinearMixedPrecision, axs_linear_mixed_precision, convert_to_axs_mixed_precision,
                              estimate_memory_savings)
from .modules_unified import (AXSEmbeddingUnified, AXSLayerNormUnified, AXSLinearUnified, AXSMultiheadAttentionUnified,
                              convert_to_axs_unified)
from .training_unified import AmaxEMA, AXSTrainingPipelineUnified

__all__ = ["fused_fake_quantize", "quantize_unified", "dequantize_unified", "NF5_CODEBOOK", "FUSED_NF5_LUT",
           "REVERSE_NF5_LUT", "accelerated_fake_quantize", "fake_quantize_unified", "get_backend",
           "set_backend", "backend_info", "accelerated_linear", "accelerated_matmul", "axs_linear_unified",
           "axs_matmul_unified", "axs_linear_mixed_precision", "AXSLinearMixedPrecision",
           "convert_to_axs_mixed_precision", "estimate_memory_savings", "AXSLinearUnified", "convert_to_axs_unified",
           "AXSLayerNormUnified", "AXSEmbeddingUnified", "AXSMultiheadAttentionUnified", "AmaxEMA",
           "AXSTrainingPipelineUnified", "quantization_error_unified", "BackendType", "clear_int8_weight_cache",
           "detect_best_backend", "has_triton", "triton_fused_fake_quantize", "triton_fused_linear", "AXS6GradCompressor",
           "axs6_gradient_hook", "axs6_gradient_hook_packed"]
