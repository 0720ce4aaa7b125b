"""Seeded random GEMM shapes through the C ABI: every kernel choice of the launcher (single CTA, CTA pairs with and
without tail split, 256 x 512 tiles, split-K with and without workspace), ragged extents, all operand layouts, bf16 and
fp32 outputs, with and without bias, against an fp32 product (TF32 off).  Tolerances as in test_gpu_linear_config4."""
import random

import pytest
import torch

pytestmark = pytest.mark.gpu

from axs6_b200 import _lib, ops  # noqa: E402
from test_gpu_linear_config4 import check_bf16_output, fp32_matmul, fp32_tol, rel  # noqa: E402


def _cases(n: int, seed: int):
    rng = random.Random(seed)
    out = []
    for i in range(n):
        big = i % 3 == 0
        M = rng.choice([1, 7, 64, 129, 256, 1000]) if not big else rng.randrange(1500, 9000)
        N = rng.randrange(1, 700) * 8 if not big else rng.randrange(100, 640) * 8
        K = rng.choice([8, 40, 64, 520, 1032]) if i % 4 == 1 else rng.randrange(64, 1200) * 8
        out.append((M, N, K, rng.randrange(2), rng.randrange(2), rng.randrange(2), rng.randrange(2)))
    return out


@pytest.mark.parametrize("M,N,K,a_mn,b_mn,f32_out,with_bias", _cases(48, 2024),
                         ids=lambda v: str(v))
def test_gemm_random_shape(M, N, K, a_mn, b_mn, f32_out, with_bias):
    g = torch.Generator(device="cuda").manual_seed(M * 7919 + N * 31 + K)
    a = torch.randn((K, M) if a_mn else (M, K), generator=g, device="cuda").to(torch.bfloat16)
    b = torch.randn((K, N) if b_mn else (N, K), generator=g, device="cuda").to(torch.bfloat16)
    bias = torch.randn(N, generator=g, device="cuda") if with_bias else None
    ref = fp32_matmul(a, b, bool(a_mn), bool(b_mn))
    if bias is not None:
        ref = ref + bias
    out_dtype = torch.float32 if f32_out else torch.bfloat16
    c = ops.gemm_bf16(a, b, bias=bias, a_mn=bool(a_mn), b_mn=bool(b_mn), out_dtype=out_dtype)
    assert _lib.load().axs6_gemm_status() == 0
    assert c.shape == (M, N)
    if f32_out:
        assert rel(c, ref) < fp32_tol(K)
    else:
        check_bf16_output(c, ref)
