"""Rounding-strategy wrappers over :func:`axs6_b200.core.quantize`.

Mirrors ``axs/quantize.py``: ``quantize_nearest`` (quantize.py:120-129), ``quantize_stochastic``
(:132-146), error feedback (:149-200, a host composition of quantise / dequantise kernels),
gradient-aware stochastic rounding (:203-307, the stochastic kernel fed with transformed draws) and
the dispatcher ``quantize_adaptive`` (:315-352).
"""
from __future__ import annotations

from enum import Enum

import torch

from . import ops
from .core import DEFAULT_BLOCK_SIZE, VALID_BLOCK_SIZES, AXSTensor, _quantize_planes, dequantize, quantize


class RoundingMode(Enum):
    NEAREST = "nearest"
    STOCHASTIC = "stochastic"
    ERROR_FEEDBACK = "error_feedback"
    GASR = "gasr"


class ErrorFeedbackState:
    """Per-parameter residual buffers for error-feedback quantisation: same methods as the
    reference's class (quantize.py:47-88)."""

    def __init__(self) -> None:
        self._buffers: dict[str, torch.Tensor] = {}

    def get_buffer(self, name: str, like: torch.Tensor) -> torch.Tensor:
        """The residual of ``name`` (zeros the first time, and again when the shape changes)."""
        buf = self._buffers.get(name)
        if buf is None or buf.shape != like.shape:
            buf = torch.zeros_like(like)
            self._buffers[name] = buf
        return buf

    def update_buffer(self, name: str, error: torch.Tensor) -> None:
        self._buffers[name] = error.detach()

    def reset(self) -> None:
        self._buffers.clear()

    @property
    def buffer_names(self) -> list[str]:
        return list(self._buffers.keys())


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
    buf = st.get_buffer(param_name, tensor)
    # one kernel (add the residual, quantise, write the new residual) when the tensors qualify ...
    planes = ops.pack_error_feedback(tensor, buf, block_size, ops.GRID_UNIFORM, rounding) if tensor.is_cuda else None
    if planes is not None:
        se, sg, mg = planes
        return AXSTensor(shared_exponents=se, signs=sg, magnitudes=mg, block_size=block_size,
                         original_shape=tensor.shape, num_blocks=se.shape[-1])
    # ... else the same arithmetic as four tensor operations
    corrected = tensor + buf
    q = quantize(corrected, block_size=block_size, rounding=rounding)
    st.update_buffer(param_name, corrected - dequantize(q).to(corrected.dtype))
    return q


def quantize_gasr(tensor: torch.Tensor, gradient: torch.Tensor, block_size: int = DEFAULT_BLOCK_SIZE,
                  temperature: float = 1.0, noise: torch.Tensor | None = None) -> AXSTensor:
    """Gradient-aware stochastic rounding (quantize.py:203-307): a value between two levels goes up with
    probability ``frac ** (2 - w)``, ``w = sigmoid(temperature * |g| / mean_block(|g|))``, so values with large
    gradients round closer to nearest.

    ``rand < frac ** e`` holds exactly when ``rand ** (1 / e) < frac`` (e >= 1, both sides in [0, 1]), so the
    rule is the stochastic uniform-grid kernel fed with the transformed draws ``rand ** (1 / (2 - w))``: the
    weights and the transformed draws are elementwise torch ops on the device, exponent, magnitudes and signs
    come from the pack kernel.  ``noise``: the U[0,1) draws ``rand`` in the zero-padded (rows, nblk, block)
    layout (default: ``torch.rand``), which makes the result reproducible."""
    assert tensor.shape == gradient.shape, "Tensor and gradient must have same shape"
    assert block_size in VALID_BLOCK_SIZES
    if not tensor.is_cuda:
        raise RuntimeError("quantize_gasr requires a CUDA tensor")
    last = tensor.shape[-1]
    g = gradient.reshape(-1, last).float().abs()
    pad = (-last) % block_size
    if pad:
        g = torch.nn.functional.pad(g, (0, pad))
    gb = g.view(g.shape[0], -1, block_size)
    weight = torch.sigmoid(temperature * gb / gb.mean(dim=-1, keepdim=True).clamp(min=1e-45))
    rand = torch.rand_like(weight) if noise is None else noise.to(device=tensor.device, dtype=torch.float32).reshape(weight.shape)
    draws = rand.pow(1.0 / (2.0 - weight))
    return _quantize_planes(tensor, block_size, "stochastic", ops.GRID_UNIFORM, "quantize_gasr", noise=draws)


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
        if gradient is None:
            raise ValueError("GASR mode requires a gradient tensor")
        return quantize_gasr(tensor, gradient, block_size, gasr_temperature)
    raise ValueError(f"Unknown rounding mode: {mode}")
