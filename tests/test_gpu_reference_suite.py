"""The reference's own GPU acceptance cases for this path, run against the B200 kernels with the CPU
oracle in the role of the reference's eager implementation.  Shapes, scales and thresholds are those of
tests/test_triton_kernels.py, tests/test_triton_fused_linear.py and tests/test_mixed_precision.py of the
reference; where the reference accepts `allclose(atol=1e-6)` the fake-quantise results here must be
bit-identical."""
import importlib

import numpy as np
import pytest
import torch
import torch.nn as nn

import oracle
from gpu_util import assert_bits_equal

pytestmark = pytest.mark.gpu

from axs6_b200 import _lib  # noqa: E402

tk = importlib.import_module("axs6_b200.unified.triton_kernels")
mp = importlib.import_module("axs6_b200.unified.mixed_precision")
um = importlib.import_module("axs6_b200.unified.modules_unified")
fu = importlib.import_module("axs6_b200.unified.functional_unified")
ub = importlib.import_module("axs6_b200.unified.backend")
import axs6_b200.unified as unified  # noqa: E402


# ---------------------------------------------------------------- fake-quantise (test_triton_kernels.py:78-280)
@pytest.mark.parametrize("shape", [(4096, 4096), (256, 256), (100, 50), (7, 13), (1, 32), (4, 16, 64), (3, 100, 17),
                                   (2, 4, 8, 32), (128, 128)], ids=lambda s: "x".join(map(str, s)))
def test_nearest_matches_eager(shape):
    torch.manual_seed(42)
    x = torch.randn(*shape)
    y = tk.triton_fused_fake_quantize(x.cuda(), 32, "nearest")
    assert y.shape == x.shape and y.dtype == torch.float32 and y.is_cuda
    assert_bits_equal(y, oracle.fused_fake_quantize(x.numpy(), 32), str(shape))


@pytest.mark.parametrize("bs", [8, 16, 32])
def test_block_sizes(bs):
    torch.manual_seed(123)
    x = torch.randn(256, 256)
    assert_bits_equal(tk.triton_fused_fake_quantize(x.cuda(), bs), oracle.fused_fake_quantize(x.numpy(), bs), f"bs{bs}")


@pytest.mark.parametrize("scale", [1000.0, 1e-6])
def test_large_and_tiny_values(scale):
    torch.manual_seed(5)
    x = torch.randn(64, 64) * scale
    assert_bits_equal(tk.triton_fused_fake_quantize(x.cuda()), oracle.fused_fake_quantize(x.numpy()), f"x{scale}")


def test_zero_tensor_and_single_block_and_power_of_two_amax():
    z = torch.zeros(128, 128, device="cuda")
    assert bool((tk.triton_fused_fake_quantize(z) == 0).all())
    torch.manual_seed(1)
    one = torch.randn(1, 32)
    assert_bits_equal(tk.triton_fused_fake_quantize(one.cuda()), oracle.fused_fake_quantize(one.numpy()), "single block")
    x = torch.zeros(1, 32)
    for exp in (-2, 0, 1, 3, 5, 8):
        x[0, 0] = 2.0 ** exp
        assert_bits_equal(tk.triton_fused_fake_quantize(x.cuda()), oracle.fused_fake_quantize(x.numpy()), f"amax 2^{exp}")


@pytest.mark.parametrize("n_blocks", [16, 32, 64, 128, 256])
def test_n_blocks_argument_is_accepted(n_blocks):
    torch.manual_seed(9)
    x = torch.randn(512, 512)
    y = tk.triton_fused_fake_quantize(x.cuda(), 32, "nearest", n_blocks=n_blocks)
    assert_bits_equal(y, oracle.fused_fake_quantize(x.numpy()), f"n_blocks {n_blocks}")


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_half_precision_inputs_keep_their_dtype(dtype):
    x = torch.randn(64, 64, device="cuda").to(dtype)
    y = tk.triton_fused_fake_quantize(x)
    assert y.dtype == dtype and y.shape == x.shape


# ---------------------------------------------------------------- fused linear (test_triton_fused_linear.py:70-350)
def _ref_linear(x, w, b, quantize_input=True):
    x2 = x.reshape(-1, x.shape[-1]).numpy()
    xq = oracle.fused_fake_quantize(x2) if quantize_input else x2
    wq = oracle.fused_fake_quantize(w.numpy())
    y = xq.astype(np.float64) @ wq.astype(np.float64).T
    if b is not None:
        y = y + b.numpy().astype(np.float64)
    return torch.from_numpy(y).reshape(*x.shape[:-1], w.shape[0])


def _close(y, ref):
    err = float((y.detach().cpu().double() - ref).norm() / ref.norm())
    assert err < 1e-3, err


@pytest.mark.parametrize("M,N,K", [(32, 64, 128), (64, 128, 256), (128, 256, 512), (1, 64, 128), (17, 33, 64), (256, 256, 256)])
@pytest.mark.parametrize("bias", [True, False])
def test_fused_linear(M, N, K, bias):
    torch.manual_seed(M + N + K)
    x, w = torch.randn(M, K), torch.randn(N, K)
    b = torch.randn(N) if bias else None
    y = tk.triton_fused_linear(x.cuda(), w.cuda(), b.cuda() if bias else None)
    assert y.dtype == torch.float32 and y.shape == (M, N) and y.is_contiguous() and y.is_cuda
    _close(y, _ref_linear(x, w, b))


@pytest.mark.parametrize("K", [33, 50, 100, 127, 255])
def test_fused_linear_non_aligned_k(K):
    torch.manual_seed(K)
    x, w, b = torch.randn(32, K), torch.randn(64, K), torch.randn(64)
    _close(tk.triton_fused_linear(x.cuda(), w.cuda(), b.cuda()), _ref_linear(x, w, b))


@pytest.mark.parametrize("shape", [(4, 8, 128), (2, 3, 4, 128), (1, 1, 128), (16, 128)])
def test_fused_linear_batched(shape):
    torch.manual_seed(len(shape))
    x, w, b = torch.randn(*shape), torch.randn(64, 128), torch.randn(64)
    y = tk.triton_fused_linear(x.cuda(), w.cuda(), b.cuda())
    assert y.shape == (*shape[:-1], 64)
    _close(y, _ref_linear(x, w, b))


def test_fused_linear_without_input_quantisation():
    torch.manual_seed(3)
    x, w = torch.randn(64, 256), torch.randn(128, 256)
    _close(tk.triton_fused_linear(x.cuda(), w.cuda(), None, 32, False), _ref_linear(x, w, None, quantize_input=False))
    _close(ub.accelerated_linear(x.cuda(), w.cuda(), None, 32, False), _ref_linear(x, w, None, quantize_input=False))


def test_gradient_flows_through_the_unified_linear():
    torch.manual_seed(4)
    x = torch.randn(16, 128, device="cuda", requires_grad=True)
    w = torch.randn(64, 128, device="cuda", requires_grad=True)
    b = torch.randn(64, device="cuda", requires_grad=True)
    y = fu.axs_linear_unified(x, w, b)
    y.sum().backward()
    for t in (x, w, b):
        assert t.grad is not None and bool(torch.isfinite(t.grad).all()) and float(t.grad.abs().sum()) > 0
    ref = torch.nn.functional.linear(x.detach(), w.detach(), b.detach())
    assert float((y.detach() - ref).abs().mean()) < 0.5 * float(ref.abs().mean())     # magnitude is reasonable


def test_exports():
    for name in ("triton_fused_fake_quantize", "triton_fused_linear"):
        assert hasattr(tk, name)
    for name in ("fused_fake_quantize", "quantize_unified", "dequantize_unified", "accelerated_fake_quantize",
                 "accelerated_linear", "accelerated_matmul", "axs_linear_unified", "fake_quantize_unified",
                 "axs_linear_mixed_precision", "AXSLinearMixedPrecision", "convert_to_axs_mixed_precision",
                 "estimate_memory_savings", "AXSLinearUnified", "convert_to_axs_unified"):
        assert hasattr(unified, name), name


# ---------------------------------------------------------------- mixed precision (test_mixed_precision.py:86-550)
def _ref_mixed(x, w, b):
    xb = oracle.f32_to_bf16(x.reshape(-1, x.shape[-1]).numpy())
    xq = oracle.bf16_to_f32(oracle.fused_fake_quantize(xb)).astype(np.float64)
    wq = oracle.bf16_to_f32(oracle.fused_fake_quantize(oracle.f32_to_bf16(w.numpy()))).astype(np.float64)
    y = xq @ wq.T
    if b is not None:
        y = y + oracle.bf16_to_f32(oracle.f32_to_bf16(b.numpy())).astype(np.float64)
    return torch.from_numpy(y).reshape(*x.shape[:-1], w.shape[0])


@pytest.mark.parametrize("M,N,K", [(32, 64, 128), (64, 128, 256), (1, 32, 64), (128, 256, 512)])
def test_mixed_precision_shapes_and_values(M, N, K):
    torch.manual_seed(M + K)
    x, w, b = torch.randn(M, K), torch.randn(N, K), torch.randn(N)
    y = mp.axs_linear_mixed_precision(x.cuda(), w.cuda(), b.cuda())
    assert y.dtype == torch.bfloat16 and y.shape == (M, N)
    ref = _ref_mixed(x, w, b)
    assert torch.allclose(y.float().cpu().double(), ref, atol=0.05, rtol=5e-3)       # the reference's own tolerance
    y3 = mp.axs_linear_mixed_precision(x.reshape(1, M, K).cuda(), w.cuda())
    assert y3.shape == (1, M, N)


def test_mixed_precision_dtypes_of_gradients():
    x = torch.randn(16, 64, device="cuda", requires_grad=True)
    w = torch.randn(32, 64, device="cuda", requires_grad=True)
    b = torch.randn(32, device="cuda", requires_grad=True)
    mp.axs_linear_mixed_precision(x, w, b).float().sum().backward()
    assert w.grad.dtype == torch.float32 and b.grad.dtype == torch.float32 and x.grad.dtype == torch.float32


def test_mixed_precision_edge_cases():
    assert mp.axs_linear_mixed_precision(torch.randn(1, 32, device="cuda"), torch.randn(32, 32, device="cuda")).shape == (1, 32)
    out = mp.axs_linear_mixed_precision(torch.randn(1024, 64, device="cuda"), torch.randn(32, 64, device="cuda"))
    assert out.shape == (1024, 32) and bool(torch.isfinite(out).all())
    out = mp.axs_linear_mixed_precision(torch.zeros(8, 64, device="cuda"), torch.randn(32, 64, device="cuda"))
    assert float(out.abs().max()) < 0.01
    layer = mp.AXSLinearMixedPrecision(64, 32).cuda()
    with torch.no_grad():
        assert layer(torch.randn(8, 64, device="cuda")).shape == (8, 32)
    torch.manual_seed(42)
    x, w, b = torch.randn(32, 64, device="cuda"), torch.randn(16, 64, device="cuda"), torch.randn(16, device="cuda")
    torch.testing.assert_close(mp.axs_linear_mixed_precision(x, w, b).float(), fu.axs_linear_unified(x, w, b), atol=1.0, rtol=0.1)


def test_module_behaviour():
    layer = mp.AXSLinearMixedPrecision(64, 32).cuda()
    assert layer.weight.dtype == torch.float32 and layer.bias is not None
    assert mp.AXSLinearMixedPrecision(64, 32, bias=False).bias is None
    assert "mixed_precision=bf16" in layer.extra_repr()
    x = torch.randn(8, 64, device="cuda", requires_grad=True)
    y = layer(x)
    y.float().sum().backward()
    assert layer.weight.grad is not None and bool(torch.isfinite(layer.weight.grad).all())


def test_simple_fit_converges():
    """A two-layer net on a fixed regression target improves by more than 40 % in 200 AdamW steps."""
    torch.manual_seed(0)
    net = nn.Sequential(mp.AXSLinearMixedPrecision(32, 64), nn.ReLU(), mp.AXSLinearMixedPrecision(64, 1)).cuda()
    opt = torch.optim.AdamW(net.parameters(), lr=1e-2)
    x = torch.randn(256, 32, device="cuda")
    y = (x[:, :4].sum(dim=1, keepdim=True) * 0.5).detach()
    first = last = None
    for _ in range(200):
        opt.zero_grad()
        loss = torch.nn.functional.mse_loss(net(x).float(), y)
        loss.backward()
        opt.step()
        last = float(loss.detach())
        first = last if first is None else first
    assert last < 0.6 * first


def test_conversion_variants_and_memory_estimate():
    model = nn.Sequential(nn.Linear(64, 32), nn.ReLU(), nn.Linear(32, 16))
    conv = mp.convert_to_axs_mixed_precision(model)
    assert isinstance(conv[0], mp.AXSLinearMixedPrecision) and isinstance(conv[1], nn.ReLU)
    assert isinstance(model[0], nn.Linear) and not isinstance(model[0], mp.AXSLinearMixedPrecision)
    torch.testing.assert_close(conv[0].weight.data, model[0].weight.data)
    torch.testing.assert_close(conv[0].bias.data, model[0].bias.data)
    inpl = nn.Sequential(nn.Linear(64, 32))
    mp.convert_to_axs_mixed_precision(inpl, inplace=True)
    assert isinstance(inpl[0], mp.AXSLinearMixedPrecision)
    skipped = mp.convert_to_axs_mixed_precision(nn.Sequential(nn.Linear(64, 32), nn.Linear(32, 16)), skip_layers={"0"})
    assert not isinstance(skipped[0], mp.AXSLinearMixedPrecision) and isinstance(skipped[1], mp.AXSLinearMixedPrecision)
    from_unified = mp.convert_to_axs_mixed_precision(nn.Sequential(um.AXSLinearUnified(64, 32)))
    assert isinstance(from_unified[0], mp.AXSLinearMixedPrecision)

    class TwoLayer(nn.Module):
        def __init__(self):
            super().__init__()
            self.net = nn.Sequential(nn.Linear(64, 32), nn.ReLU(), nn.Linear(32, 16))

        def forward(self, t):
            return self.net(t)

    nested = mp.convert_to_axs_mixed_precision(TwoLayer()).cuda()
    assert isinstance(nested.net[0], mp.AXSLinearMixedPrecision) and isinstance(nested.net[2], mp.AXSLinearMixedPrecision)
    out = nested(torch.randn(8, 64, device="cuda"))
    assert out.shape == (8, 16) and out.dtype == torch.bfloat16 and bool(torch.isfinite(out).all())
    est = mp.estimate_memory_savings(nn.Sequential(mp.AXSLinearMixedPrecision(1024, 4096)), batch_size=8, seq_len=128)
    assert est["fp32_mb"] == round((8 * 128 * 1024 + 4096 * 1024) * 4 / 2 ** 20, 2)
    assert est["bf16_recomp_mb"] == round(8 * 128 * 1024 * 2 / 2 ** 20, 2) and est["savings_ratio"] > 2
    assert mp.estimate_memory_savings(nn.Sequential(nn.Linear(4, 4)))["bf16_recomp_mb"] == 0


def test_no_bounded_wait_gave_up_in_this_file():
    assert _lib.load().axs6_gemm_status() == 0


# ---------------------------------------------------------------- first-generation launchers (axs/triton_kernels)
def test_first_generation_launchers():
    """triton_quantize / triton_dequantize / triton_fake_quantize / triton_axs_matmul (uniform grid, 2-D input,
    row length a multiple of the block size): codes, reconstruction and fake-quantise bit for bit against the
    oracle's uniform-grid path, the product within 1e-3 of the product of the oracle-quantised operands."""
    lk = importlib.import_module("axs6_b200.triton_kernels")
    torch.manual_seed(21)
    x = torch.randn(96, 160) * torch.logspace(-2, 2, 96).unsqueeze(1)
    for B in (8, 16, 32):
        se, sg, mg = lk.triton_quantize(x.cuda(), B)
        ose, osg, omg = oracle.quantize(x.numpy(), B, oracle.GRID_UNIFORM)
        assert se.shape == (96, 160 // B) and sg.shape == (96, 160) and sg.dtype == torch.bool and mg.dtype == torch.uint8
        assert_bits_equal(se, ose, "exponents")
        assert_bits_equal(sg, osg.reshape(96, 160), "signs")
        assert_bits_equal(mg, omg.reshape(96, 160), "magnitudes")
        back = lk.triton_dequantize(se, sg, mg, B)
        assert back.dtype == torch.float32
        assert_bits_equal(back, oracle.dequantize(ose, osg, omg, 160, oracle.GRID_UNIFORM), "dequantize")
        assert_bits_equal(lk.triton_fake_quantize(x.cuda(), B), oracle.fake_quantize_uniform(x.numpy(), B), "fake quantize")
    sq = lk.triton_fake_quantize(x.cuda(), 32, stochastic=True)
    assert sq.shape == x.shape and bool(torch.isfinite(sq).all())
    with pytest.raises(AssertionError):
        lk.triton_fake_quantize(torch.randn(4, 33, device="cuda"))
    with pytest.raises(AssertionError):
        lk.triton_quantize(torch.randn(2, 4, 32, device="cuda"))
    a, b = torch.randn(130, 256), torch.randn(256, 72)
    c = lk.triton_axs_matmul(a.cuda(), b.cuda())
    aq = oracle.fake_quantize_uniform(a.numpy(), 32).astype(np.float64)
    bq = oracle.fake_quantize_uniform(np.ascontiguousarray(b.numpy().T), 32).astype(np.float64).T
    ref = torch.from_numpy(aq @ bq)
    assert c.shape == (130, 72) and c.dtype == torch.float32
    _close(c, ref)
    _close(lk.triton_axs_matmul(a.cuda(), b.cuda(), quantize_a=False, quantize_b=False), (a.double() @ b.double()))
