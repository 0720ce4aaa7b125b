"""Rounding-strategy wrappers over :func:`axs6_b200.core.quantize`.

Mirrors ``axs/quantize.py`` for the strategies on the hot path: ``quantize_nearest``
(quantize.py:120-129), ``quantize_stochastic`` (:132-146), error feedback (:149-200, a host
composition of quantise / dequantise kernels) and the dispatcher ``quantize_adaptive`` (:315-352).
"""
from __future__ import annotations

from enum import Enum

import torch

from .core import DEFAULT_BLOCK_SIZE, AXSTensor, dequantize, quantize


class RoundingMode(Enum):
    NEAREST = "nearest"
    STOCHASTIC = "stochastic"
    ERROR_FEEDBACK = "error_feedback"
    GASR = "gasr"


class ErrorFeedbackState:
    """Per-parameter residual buffers for error-feedback quantisation (quantize.py:47-88)."""

    def __init__(self) -> None:
        self._buffers: dict[str, torch.Tensor] = {}

    def get_error(self, name: str, shape: torch.Size, device: torch.device) -> torch.Tensor:
        buf = self._buffers.get(name)
        if buf is None or buf.shape != shape:
            buf = torch.zeros(shape, device=device, dtype=torch.float32)
            self._buffers[name] = buf
        return buf

    def update_error(self, name: str, error: torch.Tensor) -> None:
        self._buffers[name] = error.detach().clone()

    def reset(self) -> None:
        self._buffers.clear()


_global_ef_state = ErrorFeedbackState()


def quantize_nearest(tensor: torch.Tensor, block_size: int = DEFAULT_BLOCK_SIZE) -> AXSTensor:
    return quantize(tensor, block_size=block_size, rounding="nearest")


def quantize_stochastic(tensor: torch.Tensor, block_size: int = DEFAULT_BLOCK_SIZE) -> AXSTensor:
    return quantize(tensor, block_size=block_size, rounding="stochastic")


def quantize_with_error_feedback(tensor: torch.Tensor, block_size: int = DEFAULT_BLOCK_SIZE,
                                 rounding: str = "nearest", param_name: str = "default",
                                 state: ErrorFeedbackState | None = None) -> AXSTensor:
    """x + residual -> quantise -> residual = corrected - dequantise (quantize.py:149-200)."""
    st = state if state is not None else _global_ef_state
    err = st.get_error(param_name, tensor.shape, tensor.device)
    corrected = tensor.float() + err
    q = quantize(corrected, block_size=block_size, rounding=rounding)
    st.update_error(param_name, corrected - dequantize(q))
    return q


def quantize_adaptive(tensor: torch.Tensor, mode: RoundingMode = RoundingMode.NEAREST,
                      block_size: int = DEFAULT_BLOCK_SIZE, gradient: torch.Tensor | None = None,
                      param_name: str = "default", ef_state: ErrorFeedbackState | None = None,
                      gasr_temperature: float = 1.0) -> AXSTensor:
    if mode == RoundingMode.NEAREST:
        return quantize_nearest(tensor, block_size)
    if mode == RoundingMode.STOCHASTIC:
        return quantize_stochastic(tensor, block_size)
    if mode == RoundingMode.ERROR_FEEDBACK:
        return quantize_with_error_feedback(tensor, block_size, "nearest", param_name, ef_state)
    if mode == RoundingMode.GASR:
        raise NotImplementedError("gradient-aware stochastic rounding is outside the accelerated path")
    raise ValueError(f"Unknown rounding mode: {mode}")
