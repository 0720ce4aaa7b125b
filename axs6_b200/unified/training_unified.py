"""Training loop helper for models built from the AXS-6 layers (mirror of
``axs/unified/training_unified.py``: ``AmaxEMA`` :63-108, ``AXSTrainingPipelineUnified`` :115-410).

Same constructor arguments, ``training_step`` result keys, checkpoint contents and ``stats`` as the
reference.  Two things are done the GPU way: the gradients are unscaled and checked for inf/NaN by ONE
fused multi-tensor kernel with a single host read (the reference divides and scans parameter by parameter,
with two host syncs per parameter), and the checkpoint also carries this library's Philox counter (the
host-side offset and the device-resident epoch that CUDA-graph replays advance), so a resumed run continues
the stochastic-rounding stream where the saved one stopped.  The fused unscale multiplies by ``1 / loss_scale``
where the reference divides by ``loss_scale``: identical for the power-of-two scales the pipeline itself
produces (initial 2^k, doubling / halving), up to one ulp for any other scale a caller sets.
"""
from __future__ import annotations

import logging
import math
from pathlib import Path
from typing import Any, Callable

import torch
import torch.nn as nn

from .. import ops

logger = logging.getLogger(__name__)


def _warmup_types() -> tuple[type, ...]:
    from .mixed_precision import AXSLinearMixedPrecision
    from .modules_unified import AXSEmbeddingUnified, AXSLinearUnified
    return (AXSLinearUnified, AXSEmbeddingUnified, AXSLinearMixedPrecision)


class AmaxEMA:
    """Exponential moving average of per-tensor maxima, for delayed scaling: ``get_scale`` is the power of
    two just above the smoothed maximum."""

    def __init__(self, decay: float = 0.999) -> None:
        self.decay = decay
        self._values: dict[str, float] = {}

    def update(self, name: str, amax: float) -> None:
        old = self._values.get(name)
        self._values[name] = amax if old is None else self.decay * old + (1.0 - self.decay) * amax

    def get_amax(self, name: str, default: float = 1.0) -> float:
        return self._values.get(name, default)

    def get_scale(self, name: str, default: float = 1.0) -> float:
        amax = self.get_amax(name, default)
        return 1.0 if amax <= 0 else 2.0 ** (math.floor(math.log2(amax)) + 1)

    def state_dict(self) -> dict[str, Any]:
        return {"decay": self.decay, "values": dict(self._values)}

    def load_state_dict(self, state: dict[str, Any]) -> None:
        self.decay = state["decay"]
        self._values = dict(state["values"])


class AXSTrainingPipelineUnified:
    """Warm-up without quantisation for the first ``warmup_steps`` steps, dynamic loss scaling with overflow
    back-off, gradient clipping, optimiser and scheduler step, checkpoints."""

    def __init__(self, model: nn.Module, optimizer, scheduler=None, warmup_steps: int = 0,
                 loss_scale_init: float = 2.0 ** 16, loss_scale_growth_interval: int = 2000,
                 loss_scale_backoff: float = 0.5, loss_scale_growth: float = 2.0, max_grad_norm: float = 1.0,
                 use_amax_ema: bool = False, amax_ema_decay: float = 0.999) -> None:
        self.model, self.optimizer, self.scheduler = model, optimizer, scheduler
        self.warmup_steps = warmup_steps
        self.loss_scale = loss_scale_init
        self._loss_scale_init = loss_scale_init
        self.growth_interval, self.backoff, self.growth = loss_scale_growth_interval, loss_scale_backoff, loss_scale_growth
        self.max_grad_norm = max_grad_norm
        self.amax_ema = AmaxEMA(decay=amax_ema_decay) if use_amax_ema else None
        self._steps_since_scale_change = 0
        self._total_steps = 0
        self._overflow_count = 0
        self._grad_norms: list[float] = []

    # ------------------------------------------------------------------ warm-up
    def _set_warmup(self, active: bool) -> None:
        types = _warmup_types()
        for m in self.model.modules():
            if isinstance(m, types):
                m._warmup_active = active

    @property
    def is_warmup(self) -> bool:
        return self._total_steps < self.warmup_steps

    # ------------------------------------------------------------------ one step
    def _unscale_and_check(self) -> bool:
        """grad /= loss_scale for every parameter; True if any gradient holds inf or NaN."""
        grads = [p.grad for p in self.model.parameters() if p.grad is not None]
        if not grads:
            return False
        found = False
        by_key: dict[tuple, list[torch.Tensor]] = {}
        for g in grads:
            by_key.setdefault((g.device, g.dtype), []).append(g)
        flags = []
        for (dev, _), gs in by_key.items():
            if dev.type == "cuda":
                flag = torch.zeros(1, dtype=torch.float32, device=dev)
                inv = torch.full((1,), 1.0 / self.loss_scale, dtype=torch.float32, device=dev)
                torch._amp_foreach_non_finite_check_and_unscale_(gs, flag, inv)
                flags.append(flag)
            else:
                for g in gs:
                    g.div_(self.loss_scale)
                    found = found or not bool(torch.isfinite(g).all())
        if flags:
            found = found or bool(torch.stack([f.to(flags[0].device) for f in flags]).sum().item() > 0)
        return found

    def _current_lr(self) -> float:
        return self.optimizer.param_groups[0]["lr"]

    def training_step(self, inputs: Any, loss_fn: Callable[..., torch.Tensor]) -> dict[str, Any]:
        """forward, scaled backward, unscale, overflow check, clip, optimiser (+ scheduler) step.
        ``loss_fn(model_output, inputs) -> loss``.  Returns loss, loss_scale, grad_norm, overflow, step,
        warmup, lr."""
        self.model.train()
        self.optimizer.zero_grad()
        warmup = self.is_warmup
        self._set_warmup(warmup)
        loss = loss_fn(self.model(inputs), inputs)
        (loss * self.loss_scale).backward()
        if self._unscale_and_check():
            self.loss_scale *= self.backoff
            self._steps_since_scale_change = 0
            self._overflow_count += 1
            self.optimizer.zero_grad()
            return {"loss": float(loss.detach()), "loss_scale": self.loss_scale, "grad_norm": 0.0, "overflow": True,
                    "step": self._total_steps, "warmup": warmup, "lr": self._current_lr()}
        norm = torch.nn.utils.clip_grad_norm_(self.model.parameters(), self.max_grad_norm)
        norm = float(norm.detach()) if isinstance(norm, torch.Tensor) else float(norm)
        self._grad_norms.append(norm)
        self.optimizer.step()
        if self.scheduler is not None:
            self.scheduler.step()
        self._steps_since_scale_change += 1
        if self._steps_since_scale_change >= self.growth_interval:
            self.loss_scale *= self.growth
            self._steps_since_scale_change = 0
        self._total_steps += 1
        return {"loss": float(loss.detach()), "loss_scale": self.loss_scale, "grad_norm": norm, "overflow": False,
                "step": self._total_steps, "warmup": warmup, "lr": self._current_lr()}

    # ------------------------------------------------------------------ checkpoints
    def save_checkpoint(self, path, *, extra: dict[str, Any] | None = None) -> Path:
        path = Path(path)
        path.parent.mkdir(parents=True, exist_ok=True)
        state: dict[str, Any] = {
            "model": self.model.state_dict(), "optimizer": self.optimizer.state_dict(),
            "total_steps": self._total_steps, "loss_scale": self.loss_scale,
            "steps_since_scale_change": self._steps_since_scale_change, "overflow_count": self._overflow_count,
            "warmup_steps": self.warmup_steps,
            "rng": {"python": torch.random.get_rng_state(),
                    "cuda": torch.cuda.get_rng_state() if torch.cuda.is_available() else None,
                    "axs6_philox_offset": ops.philox_offset(),
                    # the device-resident addend that CUDA-graph replays advance (zero unless philox_advance is used)
                    "axs6_philox_epoch": ops.philox_epoch() if torch.cuda.is_available() else 0},
        }
        if self.scheduler is not None:
            state["scheduler"] = self.scheduler.state_dict()
        if self.amax_ema is not None:
            state["amax_ema"] = self.amax_ema.state_dict()
        if extra is not None:
            state["extra"] = extra
        torch.save(state, path)
        logger.info("Saved checkpoint to %s (step %d)", path, self._total_steps)
        return path

    def load_checkpoint(self, path, *, map_location=None) -> dict[str, Any]:
        state = torch.load(Path(path), map_location=map_location, weights_only=False)
        self.model.load_state_dict(state["model"])
        self.optimizer.load_state_dict(state["optimizer"])
        self._total_steps = state["total_steps"]
        self.loss_scale = state["loss_scale"]
        self._steps_since_scale_change = state.get("steps_since_scale_change", 0)
        self._overflow_count = state.get("overflow_count", 0)
        self.warmup_steps = state.get("warmup_steps", self.warmup_steps)
        if self.scheduler is not None and "scheduler" in state:
            self.scheduler.load_state_dict(state["scheduler"])
        if self.amax_ema is not None and "amax_ema" in state:
            self.amax_ema.load_state_dict(state["amax_ema"])
        rng = state.get("rng", {})
        if "python" in rng:
            torch.random.set_rng_state(rng["python"].cpu() if hasattr(rng["python"], "cpu") else rng["python"])
        if rng.get("cuda") is not None and torch.cuda.is_available():
            torch.cuda.set_rng_state(rng["cuda"].cpu())
        if "axs6_philox_offset" in rng:
            ops.reset_philox(int(rng["axs6_philox_offset"]))
        if "axs6_philox_epoch" in rng and torch.cuda.is_available():
            ops.set_philox_epoch(int(rng["axs6_philox_epoch"]))
        logger.info("Loaded checkpoint from %s (step %d)", path, self._total_steps)
        return state.get("extra", {})

    @property
    def stats(self) -> dict[str, Any]:
        recent = self._grad_norms[-100:] if self._grad_norms else [0.0]
        return {"total_steps": self._total_steps, "overflow_count": self._overflow_count,
                "current_loss_scale": self.loss_scale, "is_warmup": self.is_warmup, "warmup_steps": self.warmup_steps,
                "avg_grad_norm_recent": sum(recent) / len(recent), "max_grad_norm_recent": max(recent),
                "amax_ema_active": self.amax_ema is not None, "lr": self._current_lr()}
