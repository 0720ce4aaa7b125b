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
