"""``triton_axs_matmul`` of the reference (``axs/triton_kernels/matmul_kernel.py:138-190``): both operands are
quantised on the uniform grid in blocks of ``block_k`` ALONG K (rows of A, columns of B) and multiplied with
fp32 accumulation.  Here: two fake-quantise passes (B through its transpose, which is also the K-major layout
the tensor-core kernel wants) and one TF32 tcgen05 GEMM.  ``block_m`` / ``block_n`` were tile-size knobs of
the reference kernel and are accepted and ignored."""
from __future__ import annotations

import torch

from .. import ops


def triton_axs_matmul(a: torch.Tensor, b: torch.Tensor, quantize_a: bool = True, quantize_b: bool = True,
                      block_m: int = 64, block_n: int = 64, block_k: int = 32) -> torch.Tensor:
    if not (a.is_cuda and b.is_cuda):
        raise RuntimeError("triton_axs_matmul requires CUDA tensors")
    assert a.ndim == 2 and b.ndim == 2
    assert a.shape[1] == b.shape[0], f"Incompatible dimensions: {a.shape} @ {b.shape}"
    if block_k not in ops.VALID_BLOCK_SIZES:
        raise ValueError(f"block_k must be one of {ops.VALID_BLOCK_SIZES}")
    aq = a.float()
    bt = b.float().t().contiguous()                        # (N, K): blocks along K are blocks of its rows
    if quantize_a:
        aq = ops.fake_quantize(aq, block_k, ops.GRID_UNIFORM, "nearest", who="triton_axs_matmul")
    if quantize_b:
        bt = ops.fake_quantize(bt, block_k, ops.GRID_UNIFORM, "nearest", who="triton_axs_matmul")
    return ops.gemm_bf16(aq.contiguous(), bt)
