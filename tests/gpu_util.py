"""Helpers for the GPU parity tests: numpy <-> CUDA tensors as raw bit patterns."""
from __future__ import annotations

import numpy as np
import torch


def to_cuda(x: np.ndarray) -> torch.Tensor:
    """float32 array -> fp32 tensor; uint16 array -> bf16 tensor (same bits)."""
    if x.dtype == np.uint16:
        return torch.from_numpy(x.view(np.int16).copy()).view(torch.bfloat16).cuda()
    return torch.from_numpy(np.ascontiguousarray(x, dtype=np.float32).copy()).cuda()


def to_bits(t: torch.Tensor) -> np.ndarray:
    t = t.detach().contiguous().cpu()
    if t.dtype == torch.float32:
        return t.view(torch.int32).numpy().view(np.uint32)
    if t.dtype == torch.bfloat16:
        return t.view(torch.int16).numpy().view(np.uint16)
    if t.dtype == torch.bool:
        return t.to(torch.uint8).numpy()
    return t.numpy()


def np_bits(a: np.ndarray) -> np.ndarray:
    a = np.ascontiguousarray(a)
    return a.view(np.uint32) if a.dtype == np.float32 else a


def assert_bits_equal(got: torch.Tensor, want: np.ndarray, what: str = "") -> None:
    g = to_bits(got).reshape(-1)
    w = np_bits(want).reshape(-1)
    assert g.shape == w.shape, (what, g.shape, w.shape)
    if not np.array_equal(g, w):
        bad = np.nonzero(g != w)[0]
        raise AssertionError(f"{what}: {bad.size} of {g.size} differ; first at {bad[0]}: "
                             f"got {g[bad[0]]:#x} want {w[bad[0]]:#x}")
