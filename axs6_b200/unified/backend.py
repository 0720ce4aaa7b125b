"""The dispatch surface of ``axs/unified/backend.py`` with a single implementation behind it.

The reference selects between eager / compiled / int8 / Triton at run time
(backend.py:79-180) and falls back on any exception (:512-535).  Here there is exactly one
backend -- the sm_100a CUDA library -- and errors surface instead of falling back.  The
function names and arguments are the ones every reference module calls:
``accelerated_fake_quantize`` (backend.py:495-537), ``accelerated_linear`` (:540-618),
``accelerated_matmul`` (:621-671).
"""
from __future__ import annotations

from enum import Enum
from typing import Literal

import torch

from .. import _lib, ops
from ..core import DEFAULT_BLOCK_SIZE
from .quantize_unified import fused_fake_quantize


class BackendType(str, Enum):
    CUDA_SM100 = "cuda_sm100"


def get_backend() -> BackendType:
    return BackendType.CUDA_SM100


def set_backend(backend) -> None:
    """Only one backend exists; anything else is an error (no silent fallback)."""
    name = backend.value if isinstance(backend, BackendType) else str(backend)
    if name != BackendType.CUDA_SM100.value:
        raise ValueError(f"axs6_b200 has a single backend ({BackendType.CUDA_SM100.value!r}); got {name!r}")


def accelerated_fake_quantize(tensor: torch.Tensor, block_size: int = DEFAULT_BLOCK_SIZE,
                              rounding: Literal["nearest", "stochastic"] = "nearest") -> torch.Tensor:
    """NF5 fake-quantise (reference: backend.py:495-537)."""
    return fused_fake_quantize(tensor, block_size, rounding)


def accelerated_linear(input: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None = None,
                       block_size: int = DEFAULT_BLOCK_SIZE, quantize_input: bool = True) -> torch.Tensor:
    """FQ(input) @ FQ(weight)^T + bias, forward only (reference: backend.py:540-618).  fp32
    tensors run the fp32 graph on the TF32 tensor cores and return fp32; bf16 input with bf16
    weight runs on the bf16 tensor cores and returns bf16."""
    if not input.is_cuda:
        raise RuntimeError("accelerated_linear requires CUDA tensors")
    x2 = input.reshape(-1, input.shape[-1])
    if x2.dtype not in (torch.float32, torch.bfloat16):
        x2 = x2.float()
    if x2.stride(-1) != 1 or (x2.shape[0] > 1 and x2.stride(0) < x2.shape[1]):
        x2 = x2.contiguous()
    w = weight if weight.dtype in (torch.float32, torch.bfloat16) else weight.float()
    w = w if w.stride(-1) == 1 else w.contiguous()
    all_bf16 = x2.dtype == torch.bfloat16 and w.dtype == torch.bfloat16
    b32 = bias.float().contiguous() if bias is not None else None
    y, _ = ops.linear_fwd(x2, w, b32, block_size, ops.GRID_NF5, bool(quantize_input),
                          torch.bfloat16 if all_bf16 else torch.float32, tf32=not all_bf16, fp32_accuracy=not all_bf16)
    return y.reshape(*input.shape[:-1], weight.shape[0])


def accelerated_matmul(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """``a (*, K) @ b (K, N)`` on the tensor cores, fp32 result (reference: backend.py:621-671; no
    quantisation step -- the operands are expected to be fake-quantised already).  fp32 operands
    are consumed as TF32, bf16 operands as bf16; ``b`` is read in place (no transpose copy)."""
    if not a.is_cuda:
        raise RuntimeError("accelerated_matmul requires CUDA tensors")
    a2 = a.reshape(-1, a.shape[-1])
    if a2.dtype != b.dtype or a2.dtype not in (torch.float32, torch.bfloat16):
        a2, b = a2.float(), b.float()
    out = ops.gemm_bf16(a2, b.reshape(-1, b.shape[-1]), a_mn=False, b_mn=True, out_dtype=torch.float32)
    return out.reshape(*a.shape[:-1], b.shape[-1])


def detect_best_backend() -> BackendType:
    """The reference probes for Triton / int8 / compiled paths (backend.py:88-125); here the answer is fixed."""
    return BackendType.CUDA_SM100


def clear_int8_weight_cache() -> None:
    """The reference caches int8 re-quantised weights (backend.py:261-280); this package has no such cache.
    Kept so that training loops written for the reference can keep calling it after ``optimizer.step()``."""


def backend_info() -> dict[str, object]:
    """Diagnostics in the spirit of backend.py:678-691."""
    cuda = torch.cuda.is_available()
    return {
        "active_backend": get_backend().value,
        "cuda_available": cuda,
        "library": _lib.LIB_PATH,
        "device_ok": bool(_lib.load().axs6_query(0)) if cuda else False,
        "sm_count": int(_lib.load().axs6_query(1)) if cuda else 0,
        "kernel_launches": _lib.launches() if cuda else 0,
        "gpu_name": torch.cuda.get_device_name() if cuda else None,
        "compute_capability": torch.cuda.get_device_capability() if cuda else None,
    }
