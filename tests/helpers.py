"""Shared helpers for the parity tests: fixture decoding and seeded input generators."""
from __future__ import annotations

import hashlib

import numpy as np


def sha(a: np.ndarray) -> str:
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def fq_case_names(manifest, stochastic=None, prefix="") -> list[str]:
    out = []
    for name, info in manifest["cases"].items():
        if "block" not in info or not name.startswith(prefix):
            continue
        if stochastic is not None and info["stochastic"] != stochastic:
            continue
        out.append(name)
    return sorted(out)


def case_input(fq_cases, manifest, name):
    """-> (bits array shaped like the input, info).  fp32 inputs come as uint32 bit patterns
    (view as float32), bf16 inputs as uint16."""
    info = manifest["cases"][name]
    x = fq_cases[f"{name}.x"].reshape(info["shape"])
    if info["dtype"] == "float32":
        x = x.view(np.float32)
    noise = fq_cases[f"{name}.noise"] if info["stochastic"] else None
    return x, noise, info


def expect_bits(fq_cases, name, key, like):
    """Golden output as the same representation as `like` (float32 array or uint16 bits)."""
    g = fq_cases[f"{name}.{key}"]
    if g.dtype == np.uint32:
        g = g.view(np.float32)
    return g.reshape(like.shape) if like is not None else g


def bits_equal(a: np.ndarray, b: np.ndarray) -> bool:
    a = np.ascontiguousarray(a)
    b = np.ascontiguousarray(b)
    if a.dtype == np.float32:
        a = a.view(np.uint32)
    if b.dtype == np.float32:
        b = b.view(np.uint32)
    return a.shape == b.shape and np.array_equal(a, b)


# ----------------------------------------------------------------- seeded workload generators
def config1_input():
    """1024x1024 fp32 ~ N(0, 0.02), torch seed 0."""
    import torch
    torch.manual_seed(0)
    return (torch.randn(1024, 1024) * 0.02).numpy()


def config2_input(rows=8192, cols=4096, seed=2):
    """bf16 (as uint16 bits): N(0,1), 0.1 % outliers x10, 1 % exact zeros."""
    g = np.random.default_rng(seed)
    x = g.standard_normal((rows, cols), dtype=np.float32)
    x[g.random((rows, cols)) < 1e-3] *= 10
    x[g.random((rows, cols)) < 1e-2] = 0
    return x


def config3_input(rows, cols, seed=3):
    """fp32 with per-row sigma log-uniform in [1e-4, 10]."""
    g = np.random.default_rng(seed)
    sig = (10.0 ** (g.random((rows, 1)) * 5 - 4)).astype(np.float32)
    return g.standard_normal((rows, cols), dtype=np.float32) * sig
