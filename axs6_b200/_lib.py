"""ctypes binding of ``libaxs6_b200.so`` (see ``include/axs6_b200.h``).

There is no CPU fallback: importing the package works without the library (so that host-side
logic can be tested anywhere), but the first call of any op raises if the library is missing.
"""
from __future__ import annotations

import ctypes
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libaxs6_b200.so")

F32, BF16 = 0, 1
GRID_UNIFORM, GRID_NF5 = 0, 1
ROUND_NEAREST, ROUND_STOCHASTIC = 0, 1
LAYOUT_PLANES, LAYOUT_WIRE, LAYOUT_SPEC, LAYOUT_SPLIT = 0, 1, 2, 3
FLAG_INPUT_VIA_BF16 = 1
FLAG_OUTPUT_TF32 = 2
LINEAR_QUANTIZE_INPUT, LINEAR_QUANTIZE_GRAD, LINEAR_COMPUTE_TF32, LINEAR_BIAS_FROM_QUANTIZED = 1, 2, 4, 8
LINEAR_BIAS_VIA_BF16 = 16
LINEAR_REUSE_WQ, LINEAR_REUSE_GQ = 32, 64
LINEAR_OPERANDS_PACKED = 128
LINEAR_SPLITK_WORKSPACE = 256
LINEAR_FP32_ACCURACY = 512

_i64, _int, _u32, _u64, _ptr = ctypes.c_int64, ctypes.c_int, ctypes.c_uint32, ctypes.c_uint64, ctypes.c_void_p

# name -> (restype, argtypes); mirrors include/axs6_b200.h one to one
SIGNATURES = {
    "axs6_strerror": (ctypes.c_char_p, [_int]),
    "axs6_query": (_i64, [_int]),
    "axs6_record_bytes": (_i64, [_int, _int]),
    "axs6_tune": (_int, [_int, _i64]),
    "axs6_philox_advance": (_int, [_u64, _int, _ptr]),
    "axs6_philox_epoch": (_int, [ctypes.POINTER(_u64)]),
    "axs6_repack": (_int, [_int, _int, _int, _i64, _ptr, _ptr, _ptr, _ptr, _ptr]),
    "axs6_fq": (_int, [_ptr, _ptr, _int, _int, _i64, _i64, _i64, _i64, _int, _int, _int, _u32, _u64, _u64, _ptr]),
    "axs6_fq_with_noise": (_int, [_ptr, _ptr, _int, _int, _i64, _i64, _i64, _i64, _int, _int, _u32, _ptr, _ptr]),
    "axs6_fq_gather": (_int, [_ptr, _i64, _ptr, _ptr, _int, _int, _i64, _i64, _i64, _i64, _int, _int, _int, _u64, _u64, _ptr]),
    "axs6_fq_gather_status": (_int, []),
    "axs6_pack_ef": (_int, [_ptr, _ptr, _i64, _i64, _i64, _int, _int, _int, _u64, _u64, _ptr, _ptr, _ptr, _ptr]),
    "axs6_pack": (_int, [_ptr, _int, _i64, _i64, _i64, _int, _int, _int, _u32, _u64, _u64, _ptr, _int,
                         _ptr, _ptr, _ptr, _ptr]),
    "axs6_unpack": (_int, [_int, _ptr, _ptr, _ptr, _ptr, _int, _i64, _i64, _i64, _int, _int, _ptr]),
    "axs6_unpack_sum": (_int, [_int, _ptr, _i64, _i64, _ptr, _int, _i64, _i64, _i64, _int, _int, ctypes.c_float, _ptr]),
    "axs6_gemm_bf16": (_int, [_ptr, _ptr, _ptr, _ptr, _i64, _i64, _i64, _i64, _i64, _i64, _int, _int, _int, _ptr]),
    "axs6_gemm_bf16_ws": (_int, [_ptr, _ptr, _ptr, _ptr, _i64, _i64, _i64, _i64, _i64, _i64, _int, _int, _int, _ptr, _i64, _ptr]),
    "axs6_gemm_workspace_bytes": (_i64, [_i64, _i64, _i64, _int]),
    "axs6_gemm_packed": (_int, [_ptr, _ptr, _i64, _ptr, _ptr, _i64, _ptr, _ptr, _i64, _i64, _i64, _i64, _int, _int, _int, _ptr]),
    "axs6_gemm_tf32": (_int, [_ptr, _ptr, _ptr, _ptr, _i64, _i64, _i64, _i64, _i64, _i64, _int, _int, _int, _ptr]),
    "axs6_gemm_status": (_int, []),
    "axs6_codec_status": (_int, []),
    "axs6_linear_workspace_bytes": (_i64, [_int, _i64, _i64, _i64]),
    "axs6_bias_grad": (_int, [_ptr, _int, _i64, _i64, _i64, _ptr, _ptr, _ptr]),
    "axs6_bias_grad_static": (_int, [_ptr, _int, _i64, _i64, _i64, _ptr, _ptr]),
    "axs6_linear_fwd": (_int, [_ptr, _int, _i64, _ptr, _int, _i64, _ptr, _ptr, _int, _i64, _i64, _i64, _i64,
                               _int, _int, _u32, _ptr, _ptr, _ptr]),
    "axs6_linear_bwd": (_int, [_ptr, _int, _i64, _ptr, _ptr, _int, _i64, _ptr, _int, _i64, _ptr, _i64, _ptr,
                               _i64, _i64, _i64, _int, _int, _u32, _u64, _u64, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr]),
    "axs6_transpose_f32": (_int, [_ptr, _ptr, _i64, _i64, _i64, _i64, _ptr]),
}

_lib = None


class Axs6Error(RuntimeError):
    """A C-ABI call returned a negative status."""

    def __init__(self, fn: str, status: int, text: str):
        super().__init__(f"{fn} failed with status {status}: {text}")
        self.status = status


def load() -> ctypes.CDLL:
    """Load the library once; raise if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m axs6_b200.build` "
                "(this package has no CPU or PyTorch fallback)")
        lib = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype = res
            fn.argtypes = args
        # experiment knobs from the environment: AXS6_TUNE="key=value,key=value" (see axs6_tune in the header)
        for item in filter(None, os.environ.get("AXS6_TUNE", "").split(",")):
            key, _, value = item.partition("=")
            if lib.axs6_tune(int(key), int(value)) != 0:
                raise ValueError(f"AXS6_TUNE: bad entry {item!r}")
        _lib = lib
    return _lib


def check(fn: str, status: int) -> None:
    if status != 0:
        raise Axs6Error(fn, status, load().axs6_strerror(status).decode())


def launches() -> int:
    """Number of kernels this process has launched through the library."""
    return int(load().axs6_query(3))
