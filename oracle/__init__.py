"""CPU oracle for the AXS-6 hot path -- TEST INFRASTRUCTURE ONLY.

A restatement of the reference's eager algorithm: the arithmetic lives in
``axs6_oracle.c`` (plain C, one loop per block) and the tables are rebuilt here with
numpy/scipy following ``axs/unified/quantize_unified.py:50-114``.  Nothing in the
product package imports this module; it is used by ``tests/``, by the smoke check and
by the CPU-baseline / reference arm of ``bench.py`` as the checker and the timed CPU
baseline.  Its parity with the reference is pinned by ``tests/golden/`` (vectors made
by importing the reference; generator ``tests/golden/make_golden.py``).

All functions take and return numpy arrays.  bf16 data travels as ``uint16`` bit
patterns (``torch_tensor.view(torch.uint16).numpy()``).
"""
from __future__ import annotations

import ctypes
import math
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "liboracle.so")
_SRC = os.path.join(_HERE, "axs6_oracle.c")

GRID_UNIFORM = 0
GRID_NF5 = 1
LAYOUT_WIRE = 1   # 1 exponent byte + 6-bit payload (25 B per block of 32)
LAYOUT_SPEC = 2   # u16 LE header (exp<<2 | config) + payload (26 B per block of 32)


def build(force: bool = False) -> str:
    """Compile ``axs6_oracle.c`` into ``liboracle.so`` next to it (gcc + OpenMP)."""
    stale = (not os.path.exists(_SO)) or os.path.getmtime(_SO) < os.path.getmtime(_SRC)
    if force or stale:
        subprocess.check_call(
            ["gcc", "-O2", "-fopenmp", "-fPIC", "-shared", "-ffp-contract=off",
             "-o", _SO, _SRC, "-lm"])
    return _SO


_lib = None


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        _lib = ctypes.CDLL(build())
        _lib.orc_log2_bump_scan.restype = ctypes.c_int64
        _lib.orc_floor_log2.restype = ctypes.c_int
        _lib.orc_floor_log2.argtypes = [ctypes.c_float]
    return _lib


# --------------------------------------------------------------------------- tables
def _erfinv(p: float) -> float:
    from scipy.special import erfinv
    return float(erfinv(np.float64(p)))


def build_codebook() -> np.ndarray:
    """32 half-normal quantile levels, normalised (quantize_unified.py:50-58)."""
    lv = np.array([math.sqrt(2.0) * _erfinv((i + 0.5) / 32) for i in range(32)], dtype=np.float64)
    return (lv / lv[-1]).astype(np.float32)


def build_lut(codebook: np.ndarray) -> np.ndarray:
    """1024-entry value LUT (quantize_unified.py:68-92)."""
    cb = codebook.astype(np.float64)
    bounds = np.concatenate([[0.0], (cb[:-1] + cb[1:]) / 2.0, [1.0 + 1e-6]])
    xs = np.linspace(0.0, 1.0, 1024, dtype=np.float64)
    codes = np.clip(np.searchsorted(bounds, xs, side="left") - 1, 0, 31)
    return cb[codes].astype(np.float32)


def build_reverse_lut(codebook: np.ndarray, lut: np.ndarray) -> np.ndarray:
    """LUT index -> code index (quantize_unified.py:105-111)."""
    d = np.abs(lut.astype(np.float64)[:, None] - codebook.astype(np.float64)[None, :])
    return d.argmin(axis=-1).astype(np.uint8)


NF5_CODEBOOK = build_codebook()
FUSED_NF5_LUT = build_lut(NF5_CODEBOOK)
REVERSE_NF5_LUT = build_reverse_lut(NF5_CODEBOOK, FUSED_NF5_LUT)


# --------------------------------------------------------------------------- helpers
def _p(a: np.ndarray):
    return a.ctypes.data_as(ctypes.c_void_p)


def _i64(v) -> ctypes.c_int64:
    return ctypes.c_int64(int(v))


def bf16_to_f32(bits: np.ndarray) -> np.ndarray:
    bits = np.ascontiguousarray(bits, dtype=np.uint16)
    out = np.empty(bits.shape, dtype=np.float32)
    lib().orc_bf16_to_f32(_p(bits), _p(out), _i64(bits.size))
    return out


def f32_to_bf16(x: np.ndarray) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.float32)
    out = np.empty(x.shape, dtype=np.uint16)
    lib().orc_f32_to_bf16(_p(x), _p(out), _i64(x.size))
    return out


def _as2d(x: np.ndarray) -> np.ndarray:
    x = np.asarray(x)
    if x.ndim == 0:
        raise ValueError("need at least one dimension")
    return np.ascontiguousarray(x.reshape(-1, x.shape[-1]))


def _to_f32(x: np.ndarray) -> tuple[np.ndarray, bool]:
    if x.dtype == np.uint16:
        return bf16_to_f32(x), True
    return np.ascontiguousarray(x, dtype=np.float32), False


# --------------------------------------------------------------------------- ops
def fused_fake_quantize(x: np.ndarray, block_size: int = 32, noise: np.ndarray | None = None) -> np.ndarray:
    """NF5 fake-quantise (quantize_unified.py:121-204).  ``x`` fp32 or uint16 (bf16 bits);
    returns the same dtype.  ``noise``: U[0,1) in the padded (rows, nblk, B) layout."""
    assert block_size in (8, 16, 32)
    shape = x.shape
    x2, was_bf16 = _to_f32(_as2d(x))
    rows, cols = x2.shape
    y = np.empty_like(x2)
    if noise is not None:
        noise = np.ascontiguousarray(noise, dtype=np.float32)
        assert noise.size == rows * (-(-cols // block_size)) * block_size
    lib().orc_fq_nf5(_p(x2), _p(y), _i64(rows), _i64(cols), _i64(cols), _i64(cols),
                     ctypes.c_int(block_size), _p(FUSED_NF5_LUT),
                     _p(noise) if noise is not None else None)
    y = y.reshape(shape)
    return f32_to_bf16(y) if was_bf16 else y


def quantize(x: np.ndarray, block_size: int = 32, grid: int = GRID_NF5, noise: np.ndarray | None = None):
    """-> (shared_exponents u8 (rows, nblk), signs u8 (rows, nblk, B), magnitudes u8 (rows, nblk, B)).
    grid NF5: quantize_unified.py:211-282; grid uniform: core.py:294-369."""
    assert block_size in (8, 16, 32)
    x2, _ = _to_f32(_as2d(x))
    rows, cols = x2.shape
    nblk = -(-cols // block_size)
    se = np.empty((rows, nblk), dtype=np.uint8)
    sg = np.empty((rows, nblk, block_size), dtype=np.uint8)
    mg = np.empty((rows, nblk, block_size), dtype=np.uint8)
    if noise is not None:
        noise = np.ascontiguousarray(noise, dtype=np.float32)
        assert noise.size == sg.size
    lib().orc_quantize(_p(x2), _i64(rows), _i64(cols), _i64(cols), ctypes.c_int(block_size),
                       ctypes.c_int(grid), _p(REVERSE_NF5_LUT),
                       _p(noise) if noise is not None else None, _p(se), _p(sg), _p(mg))
    return se, sg, mg


def dequantize(se: np.ndarray, sg: np.ndarray, mg: np.ndarray, cols: int, grid: int = GRID_NF5) -> np.ndarray:
    """-> fp32 (rows, cols).  grid NF5: quantize_unified.py:285-308; uniform: core.py:372-403."""
    rows, nblk, B = mg.shape
    se = np.ascontiguousarray(se, dtype=np.uint8)
    sg = np.ascontiguousarray(sg, dtype=np.uint8)
    mg = np.ascontiguousarray(mg, dtype=np.uint8)
    y = np.empty((rows, cols), dtype=np.float32)
    lib().orc_dequantize(_p(se), _p(sg), _p(mg), _i64(rows), _i64(cols), _i64(cols),
                         ctypes.c_int(B), ctypes.c_int(grid), _p(NF5_CODEBOOK), _p(y))
    return y


def pack_bytes(se: np.ndarray, sg: np.ndarray, mg: np.ndarray, layout: int = LAYOUT_WIRE) -> np.ndarray:
    """Planes -> flat uint8 records (distributed.py:147-198 / core.py:97-118)."""
    rows, nblk, B = mg.shape
    rec = (2 if layout == LAYOUT_SPEC else 1) + B * 6 // 8
    out = np.empty(rows * nblk * rec, dtype=np.uint8)
    lib().orc_pack_bytes(_p(np.ascontiguousarray(se)), _p(np.ascontiguousarray(sg)),
                         _p(np.ascontiguousarray(mg)), _i64(rows * nblk), ctypes.c_int(B),
                         ctypes.c_int(layout), _p(out))
    return out


def unpack_bytes(buf: np.ndarray, rows: int, nblk: int, block_size: int, layout: int = LAYOUT_WIRE):
    """Flat uint8 records -> planes (distributed.py:201-232 / core.py:120-152)."""
    buf = np.ascontiguousarray(buf).view(np.uint8)
    se = np.empty((rows, nblk), dtype=np.uint8)
    sg = np.empty((rows, nblk, block_size), dtype=np.uint8)
    mg = np.empty((rows, nblk, block_size), dtype=np.uint8)
    lib().orc_unpack_bytes(_p(buf), _i64(rows * nblk), ctypes.c_int(block_size),
                           ctypes.c_int(layout), _p(se), _p(sg), _p(mg))
    return se, sg, mg


def fake_quantize_uniform(x: np.ndarray, block_size: int = 32, noise: np.ndarray | None = None) -> np.ndarray:
    """V1 fake-quantise = dequantize(quantize(x)), always fp32 (nn/functional.py:46-53)."""
    shape = x.shape
    x2 = _as2d(x)
    se, sg, mg = quantize(x2, block_size, GRID_UNIFORM, noise)
    return dequantize(se, sg, mg, x2.shape[1], GRID_UNIFORM).reshape(shape)


def gemm_nt(a: np.ndarray, b: np.ndarray) -> np.ndarray:
    """fp32 ``a @ b.T`` with fp64 accumulation (the GEMM tolerance reference)."""
    a = np.ascontiguousarray(a, dtype=np.float32)
    b = np.ascontiguousarray(b, dtype=np.float32)
    M, K = a.shape
    N, K2 = b.shape
    assert K == K2
    c = np.empty((M, N), dtype=np.float32)
    lib().orc_gemm_nt(_p(a), _p(b), _p(c), _i64(M), _i64(N), _i64(K))
    return c


def set_threads(n: int = 0) -> int:
    """Set (n > 0) and return the number of OpenMP threads the oracle's loops use."""
    return int(lib().orc_set_threads(int(n)))


def log2_bump_scan(cap: int = 1 << 16) -> np.ndarray:
    out = np.zeros(cap, dtype=np.uint32)
    n = lib().orc_log2_bump_scan(_p(out), _i64(cap))
    assert n <= cap
    return np.sort(out[:n])
