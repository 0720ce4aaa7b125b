"""GPU tests of the rounding-strategy wrappers that are host compositions around the pack kernel:
gradient-aware stochastic rounding (axs/quantize.py:203-307) and quantization_error (axs/core.py:411-440),
against outputs recorded from the reference (tests/golden/block_cases.npz)."""
import os

import numpy as np
import pytest
import torch

from gpu_util import to_cuda

pytestmark = pytest.mark.gpu

from axs6_b200 import core, quantize as aq  # noqa: E402

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


@pytest.fixture(scope="module")
def blocks():
    return np.load(os.path.join(GOLDEN, "block_cases.npz"))


@pytest.mark.parametrize("B", [32, 16, 8])
@pytest.mark.parametrize("temp", [1, 3])
def test_gasr_with_recorded_draws(blocks, B, temp):
    """Exponents and signs bit-exact.  Magnitudes: the reference compares `rand < frac ** e`, this library
    `rand ** (1 / e) < frac`; the two fp32 evaluations can disagree only when the draw sits within rounding
    error of the threshold, so at most 0.2 % of the values may differ, each by one level."""
    key = f"gasr.b{B}.t{temp}"
    x = to_cuda(blocks[f"{key}.x"].view(np.float32))
    g = to_cuda(blocks[f"{key}.g"].view(np.float32))
    noise = torch.from_numpy(blocks[f"{key}.noise"]).cuda()
    q = aq.quantize_gasr(x, g, B, float(temp), noise=noise)
    assert np.array_equal(q.shared_exponents.cpu().numpy(), blocks[f"{key}.se"])
    assert np.array_equal(q.signs.cpu().numpy(), blocks[f"{key}.sign"])
    got, want = q.magnitudes.cpu().numpy().astype(np.int32), blocks[f"{key}.mag"].astype(np.int32)
    diff = np.abs(got - want)
    assert diff.max() <= 1
    assert (diff != 0).mean() <= 2e-3
    # the dispatcher reaches it, and asks for the gradient
    q2 = aq.quantize_adaptive(x, aq.RoundingMode.GASR, B, gradient=g, gasr_temperature=float(temp))
    assert q2.magnitudes.shape == q.magnitudes.shape
    with pytest.raises(ValueError, match="requires a gradient"):
        aq.quantize_adaptive(x, aq.RoundingMode.GASR, B)


def test_gasr_bias_follows_the_gradient_weight():
    """What the rule does (quantize.py:291-296): a value between two levels goes up with probability frac ** (2 - w),
    w = sigmoid(T |g| / mean|g|).  Large gradients (w -> 1) give plain stochastic rounding, unbiased; small gradients
    (w -> 0.5) give frac ** 1.5 < frac, i.e. a bias towards the lower level of about 1 / 2.5 - 1 / 2 = -0.1 levels."""
    g = torch.Generator(device="cuda").manual_seed(4)
    x = torch.randn(512, 1024, generator=g, device="cuda")
    grad = torch.randn(512, 1024, generator=g, device="cuda").abs()
    q = aq.quantize_gasr(x, grad, 32, 4.0)
    scale = torch.exp2(q.shared_exponents.float() - 127.0).unsqueeze(-1)
    exact = (x.abs().view(512, 32, 32) / scale) * 31.0                      # position on the magnitude grid
    bias = (q.magnitudes.float() - exact).view(512, 1024)
    hi = grad > grad.median()
    assert abs(float(bias[hi].mean())) < 0.02
    assert float(bias[~hi].mean()) < -0.03


@pytest.mark.parametrize("B", [8, 16, 32])
def test_quantization_error_matches_the_reference(blocks, B):
    x = to_cuda(blocks["qerr.x"].view(np.float32)).reshape(64, 256)
    e = core.quantization_error(x, B, "nearest")
    want = blocks[f"qerr.b{B}"]
    got = np.array([e["mse"], e["rmse"], e["max_abs_error"], e["mean_abs_error"], e["signal_to_noise_db"]])
    assert np.allclose(got, want, rtol=1e-5)


@pytest.mark.parametrize("shape", [(64, 64), (7, 96), (3, 5, 40), (1024, 1000)])
@pytest.mark.parametrize("rounding", ["nearest", "stochastic"])
def test_error_feedback_in_one_kernel_equals_the_four_steps(shape, rounding):
    """quantize_with_error_feedback on a contiguous fp32 CUDA tensor runs as ONE kernel (axs6_pack_ef); its codes and
    its residual buffer equal, bit for bit and step after step, those of add -> quantize -> dequantize -> subtract
    (axs/quantize.py:190-199) with the same draws."""
    from axs6_b200 import ops
    from axs6_b200.core import dequantize, quantize
    from axs6_b200.quantize import ErrorFeedbackState, quantize_with_error_feedback
    g = torch.Generator(device="cuda").manual_seed(sum(shape))
    xs = [torch.randn(*shape, generator=g, device="cuda") * (0.1 + i) for i in range(3)]
    state = ErrorFeedbackState()
    manual = torch.zeros(*shape, device="cuda")
    for step, x in enumerate(xs):
        ops.reset_philox(1000 * step)
        q = quantize_with_error_feedback(x, 32, rounding, "p", state)
        ops.reset_philox(1000 * step)
        corrected = x + manual
        q2 = quantize(corrected, 32, rounding)
        manual = corrected - dequantize(q2)
        assert torch.equal(q.shared_exponents, q2.shared_exponents)
        assert torch.equal(q.signs, q2.signs) and torch.equal(q.magnitudes, q2.magnitudes)
        assert torch.equal(state.get_buffer("p", x).view(torch.int32), manual.view(torch.int32))
    assert ops.pack_error_feedback(xs[0], torch.zeros_like(xs[0])) is not None       # the fused path was the one taken
