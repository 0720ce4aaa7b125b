"""Optimiser-side callers of the quantiser (mirror of ``axs/nn/optim.py``).

``AXSAdamW`` (:33-140) is AdamW on fp32 master weights whose gradients can first be replaced by their
AXS-6 reconstruction (error feedback or stochastic rounding, through this package's quantiser);
``AXSTrainingWrapper`` (:143-266) is a training step with dynamic loss scaling, overflow skipping and
gradient clipping.  Host logic around the GPU path; the arithmetic of the update is torch's AdamW.
"""
from __future__ import annotations

from typing import Any

import torch
import torch.nn as nn

from ..core import DEFAULT_BLOCK_SIZE, dequantize
from ..quantize import ErrorFeedbackState, quantize_stochastic, quantize_with_error_feedback


class AXSAdamW(torch.optim.AdamW):
    """Decoupled-weight-decay Adam; with ``quantize_gradients`` every gradient goes through
    quantise -> dequantise before the update (nearest rounding with a per-parameter residual when
    ``use_error_feedback``, stochastic rounding otherwise)."""

    def __init__(self, params: Any, lr: float = 1e-3, betas: tuple[float, float] = (0.9, 0.999), eps: float = 1e-8,
                 weight_decay: float = 0.01, block_size: int = DEFAULT_BLOCK_SIZE, quantize_gradients: bool = False,
                 use_error_feedback: bool = True) -> None:
        super().__init__(params, lr=lr, betas=betas, eps=eps, weight_decay=weight_decay)
        for group in self.param_groups:
            group.setdefault("block_size", block_size)
        self.quantize_gradients = quantize_gradients
        self.use_error_feedback = use_error_feedback
        self._ef_state = ErrorFeedbackState() if use_error_feedback else None

    @torch.no_grad()
    def step(self, closure: Any = None):
        if self.quantize_gradients:
            for gi, group in enumerate(self.param_groups):
                for pi, p in enumerate(group["params"]):
                    if p.grad is None:
                        continue
                    if self._ef_state is not None:
                        q = quantize_with_error_feedback(p.grad, group["block_size"], "nearest", f"group_{gi}_param_{pi}",
                                                         self._ef_state)
                    else:
                        q = quantize_stochastic(p.grad, group["block_size"])
                    p.grad = dequantize(q).to(p.grad.dtype)
        return super().step(closure)


class AXSTrainingWrapper:
    """``training_step(inputs, loss_fn)``: forward, scaled backward, unscale, skip the update and halve the scale on
    inf / nan, else clip the gradient norm and step; the scale doubles after ``loss_scale_growth_interval`` clean steps."""

    def __init__(self, model: nn.Module, optimizer: torch.optim.Optimizer, loss_scale_init: float = 2.0 ** 16,
                 loss_scale_growth_interval: int = 2000, loss_scale_backoff: float = 0.5, loss_scale_growth: float = 2.0,
                 max_grad_norm: float = 1.0) -> None:
        self.model, self.optimizer = model, optimizer
        self.loss_scale = loss_scale_init
        self.growth_interval, self.backoff, self.growth = loss_scale_growth_interval, loss_scale_backoff, loss_scale_growth
        self.max_grad_norm = max_grad_norm
        self._steps_since_scale_change = self._total_steps = self._overflow_count = 0

    def training_step(self, inputs: Any, loss_fn: Any) -> dict[str, float]:
        self.model.train()
        self.optimizer.zero_grad()
        loss = loss_fn(self.model(inputs), inputs)
        (loss * self.loss_scale).backward()
        grads = [p.grad for p in self.model.parameters() if p.grad is not None]
        for g in grads:
            g.div_(self.loss_scale)
        if any(not bool(torch.isfinite(g).all()) for g in grads):
            self.loss_scale *= self.backoff
            self._steps_since_scale_change = 0
            self._overflow_count += 1
            self.optimizer.zero_grad()
            return {"loss": loss.item(), "loss_scale": self.loss_scale, "grad_norm": 0.0, "overflow": True}
        grad_norm = torch.nn.utils.clip_grad_norm_(self.model.parameters(), self.max_grad_norm)
        self.optimizer.step()
        self._steps_since_scale_change += 1
        if self._steps_since_scale_change >= self.growth_interval:
            self.loss_scale *= self.growth
            self._steps_since_scale_change = 0
        self._total_steps += 1
        return {"loss": loss.item(), "loss_scale": self.loss_scale, "grad_norm": float(grad_norm), "overflow": False}

    @property
    def stats(self) -> dict[str, Any]:
        return {"total_steps": self._total_steps, "overflow_count": self._overflow_count,
                "current_loss_scale": self.loss_scale}
