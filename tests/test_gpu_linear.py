"""GPU parity of the tensor-core GEMM and the AXS-6 Linear (forward + backward), through the
C ABI.  Tolerance (stated by the task): relative Frobenius error <= 1e-3 against an fp32 matmul
of the dequantised operands; checked here on the fp32 accumulator output.  bf16 outputs are
compared with the bf16 rounding of that reference (a bf16 rounding alone costs ~1.7e-3
relative Frobenius, so they are held to 4e-3)."""
import importlib

import numpy as np
import pytest
import torch

import oracle
from gpu_util import to_bits, to_cuda

pytestmark = pytest.mark.gpu

from axs6_b200 import _lib, ops  # noqa: E402

mp = importlib.import_module("axs6_b200.unified.mixed_precision")
qu = importlib.import_module("axs6_b200.unified.quantize_unified")

TOL = 1e-3
TOL_BF16_OUT = 4e-3


def rel(a: torch.Tensor, b: torch.Tensor) -> float:
    a, b = a.detach().double(), b.detach().double()
    return float((a - b).norm() / b.norm())


def gemm_status_ok():
    assert _lib.load().axs6_gemm_status() == 0, "a bounded wait inside the GEMM kernel gave up"


@pytest.mark.parametrize("a_mn,b_mn", [(0, 0), (0, 1), (1, 0), (1, 1)])
@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (256, 512, 512), (1000, 776, 520), (1, 8, 8), (130, 40, 72),
                                   (2048, 1024, 4096)])
def test_gemm_against_fp32_matmul(M, N, K, a_mn, b_mn):
    g = torch.Generator().manual_seed(M * 7 + N * 3 + K + a_mn * 2 + b_mn)
    A = torch.randn((K, M) if a_mn else (M, K), generator=g).to(torch.bfloat16)
    B = torch.randn((K, N) if b_mn else (N, K), generator=g).to(torch.bfloat16)
    if (A.shape[1] % 8) or (B.shape[1] % 8):
        pytest.skip("operand rows are not 16-byte multiples; covered through the padded path below")
    C = ops.gemm_bf16(A.cuda(), B.cuda(), a_mn=bool(a_mn), b_mn=bool(b_mn))
    gemm_status_ok()
    Af = A.float().t() if a_mn else A.float()
    Bf = B.float() if b_mn else B.float().t()
    ref = (Af.double() @ Bf.double())
    assert rel(C.cpu(), ref) < 1e-5


def test_gemm_ragged_operands_and_bias_and_bf16_out():
    g = torch.Generator().manual_seed(1)
    A = torch.randn(77, 50, generator=g).to(torch.bfloat16)       # rows of 100 bytes: needs the padded copy
    B = torch.randn(33, 50, generator=g).to(torch.bfloat16)
    bias = torch.randn(33, generator=g)
    C = ops.gemm_bf16(A.cuda(), B.cuda(), bias=bias.cuda())
    gemm_status_ok()
    ref = A.double() @ B.double().t() + bias.double()
    assert rel(C.cpu(), ref) < 1e-5
    Cb = ops.gemm_bf16(A.cuda(), B.cuda(), bias=bias.cuda(), out_dtype=torch.bfloat16)
    assert Cb.dtype == torch.bfloat16
    assert torch.equal(Cb.cpu(), C.cpu().to(torch.bfloat16))      # same accumulator, rounded once


def test_gemm_single_row_operand_with_ragged_length():
    """M = 1 with a contraction length that is not a 16-byte multiple (bf16 K = 100, fp32 K = 50)."""
    g = torch.Generator().manual_seed(3)
    for dtype, K in ((torch.bfloat16, 100), (torch.float32, 50)):
        A = torch.randn(1, K, generator=g).to(dtype)
        B = torch.randn(24, K, generator=g).to(dtype)
        C = ops.gemm_bf16(A.cuda(), B.cuda())
        gemm_status_ok()
        assert C.shape == (1, 24)
        assert rel(C.cpu(), A.double() @ B.double().t()) < (1e-5 if dtype == torch.bfloat16 else TOL)


def test_gemm_rejects_misaligned_operands():
    lib = _lib.load()
    a = torch.zeros(64, 72, dtype=torch.bfloat16, device="cuda")
    c = torch.zeros(64, 64, device="cuda")
    st = torch.cuda.current_stream().cuda_stream
    assert lib.axs6_gemm_bf16(a.data_ptr() + 2, a.data_ptr(), c.data_ptr(), None, 64, 64, 64, 72, 72, 64, 0, 0, 0, st) == -2
    assert lib.axs6_gemm_bf16(a.data_ptr(), a.data_ptr(), c.data_ptr(), None, 64, 64, 64, 68, 72, 64, 0, 0, 0, st) == -2
    assert lib.axs6_gemm_bf16(None, a.data_ptr(), c.data_ptr(), None, 64, 64, 64, 72, 72, 64, 0, 0, 0, st) == -1


def _oracle_linear(x, w, b, g, noise, qin, qgrad, block=32):
    """fp32/fp64 restatement of the mixed-precision graph (mixed_precision.py:96-150) on the CPU
    oracle: returns y, dx, dw, db in float64 computed from the dequantised bf16 operands."""
    xb = oracle.f32_to_bf16(x) if x.dtype == np.float32 else x
    wb = oracle.f32_to_bf16(w)
    xq = oracle.bf16_to_f32(oracle.fused_fake_quantize(xb, block) if qin else xb)
    wq = oracle.bf16_to_f32(oracle.fused_fake_quantize(wb, block))
    y = xq.astype(np.float64) @ wq.astype(np.float64).T
    if b is not None:
        y = y + oracle.bf16_to_f32(oracle.f32_to_bf16(b)).astype(np.float64)
    gb = oracle.f32_to_bf16(g)
    gq = oracle.bf16_to_f32(oracle.fused_fake_quantize(gb, block, noise) if qgrad else gb)
    dx = gq.astype(np.float64) @ wq.astype(np.float64)
    dw = gq.astype(np.float64).T @ xq.astype(np.float64)
    db = g.astype(np.float64).sum(0)
    return y, dx, dw, db


@pytest.mark.parametrize("M,K,N,bias,qin,qgrad", [(256, 128, 96, True, True, True), (40, 96, 64, True, True, False),
                                                 (48, 128, 32, False, False, True), (24, 50, 24, True, True, True),
                                                 (1024, 1024, 1024, True, True, True)])
def test_linear_mixed_precision_vs_oracle(M, K, N, bias, qin, qgrad):
    rng = np.random.default_rng(M + K + N)
    x = rng.standard_normal((M, K), dtype=np.float32)
    w = (rng.standard_normal((N, K), dtype=np.float32) * 0.05)
    b = (rng.standard_normal(N, dtype=np.float32) * 0.1) if bias else None
    g = rng.standard_normal((M, N), dtype=np.float32)
    nblk = -(-N // 32)
    noise = (rng.integers(0, 1 << 24, size=M * nblk * 32).astype(np.float32) * np.float32(2.0 ** -24))
    xt = torch.from_numpy(x).cuda().requires_grad_(True)
    wt = torch.from_numpy(w).cuda().requires_grad_(True)
    bt = torch.from_numpy(b).cuda().requires_grad_(True) if bias else None
    y = mp.axs_linear_mixed_precision(xt, wt, bt, 32, qin, qgrad)
    assert y.dtype == torch.bfloat16 and y.shape == (M, N)
    mp._noise_for_next_backward = torch.from_numpy(noise).cuda() if qgrad else None
    y.backward(torch.from_numpy(g).cuda().to(torch.bfloat16))
    gemm_status_ok()
    # gradient fed to backward is bf16(g): db is the column sum of exactly that tensor
    g_b = oracle.bf16_to_f32(oracle.f32_to_bf16(g))
    ry, rdx, rdw, rdb = _oracle_linear(x, w, b, g_b, noise if qgrad else None, qin, qgrad)
    assert wt.grad.dtype == torch.float32 and xt.grad.dtype == torch.float32
    assert rel(y.float().cpu(), torch.from_numpy(ry)) < TOL_BF16_OUT
    assert rel(xt.grad.cpu(), torch.from_numpy(rdx)) < TOL_BF16_OUT       # dX is produced in bf16
    assert rel(wt.grad.cpu(), torch.from_numpy(rdw)) < TOL                # dW: fp32 accumulator
    if bias:
        assert bt.grad.dtype == torch.float32
        assert rel(bt.grad.cpu(), torch.from_numpy(rdb)) < 1e-5


def test_linear_fp32_accumulator_meets_1e_minus_3():
    """The stated GEMM bar, on the accumulator: y (fp32 out) and dX (fp32 out) against the fp32
    matmul of the dequantised operands."""
    rng = np.random.default_rng(5)
    M, K, N = 512, 1024, 768
    x = rng.standard_normal((M, K), dtype=np.float32)
    w = rng.standard_normal((N, K), dtype=np.float32) * 0.02
    g = rng.standard_normal((M, N), dtype=np.float32)
    xt, wt = torch.from_numpy(x).cuda(), torch.from_numpy(w).cuda()
    y, xq = ops.linear_fwd(xt, wt, None, 32, ops.GRID_NF5, True, torch.float32)
    dx, dw, _ = ops.linear_bwd(torch.from_numpy(g).cuda(), xq, wt, M, N, K, 32, ops.GRID_NF5, False, True, True, False,
                               torch.float32)
    gemm_status_ok()
    ry, rdx, rdw, _ = _oracle_linear(x, w, None, g, None, True, False)
    assert rel(y.cpu(), torch.from_numpy(ry)) < 1e-5
    assert rel(dx.cpu(), torch.from_numpy(rdx)) < 1e-5
    assert rel(dw.cpu(), torch.from_numpy(rdw)) < 1e-5


def test_backward_reusing_the_forward_quantised_weight_is_bit_identical():
    """dX from the forward's quantised weight equals dX from the recomputed one (mixed_precision.py:130), also when
    backward is split into a dW call and a dX call that reuses the rounded gradient; a weight changed in place
    between forward and backward is re-quantised."""
    g = torch.Generator().manual_seed(17)
    M, K, N = 192, 256, 160
    x = torch.randn(M, K, generator=g).cuda()
    w0 = (torch.randn(N, K, generator=g) * 0.05).cuda()
    go = torch.randn(M, N, generator=g).cuda().to(torch.bfloat16)
    noise = torch.rand(M * N, generator=g).cuda()
    grads = {}
    try:
        for keep in (True, False):
            mp.KEEP_QUANTIZED_WEIGHT = keep
            xt, wt = x.clone().requires_grad_(True), w0.clone().requires_grad_(True)
            y = mp.axs_linear_mixed_precision(xt, wt, None, 32, True, True)
            mp._noise_for_next_backward = noise
            y.backward(go)
            grads[keep] = (xt.grad.clone(), wt.grad.clone())
    finally:
        mp.KEEP_QUANTIZED_WEIGHT = True
    assert torch.equal(grads[True][0], grads[False][0]) and torch.equal(grads[True][1], grads[False][1])
    # two calls through the C ABI: dW first, then dX / db reusing the rounded gradient and the forward's weight
    lib = _lib.load()
    st = torch.cuda.current_stream().cuda_stream
    xb = x.to(torch.bfloat16)
    ws = [torch.empty(int(lib.axs6_linear_workspace_bytes(i, M, N, K)), dtype=torch.uint8, device="cuda") for i in range(4)]
    yb = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
    assert lib.axs6_linear_fwd(xb.data_ptr(), 1, K, w0.data_ptr(), 0, K, None, yb.data_ptr(), 1, N, M, N, K, 32, 1, 1,
                               ws[0].data_ptr(), ws[1].data_ptr(), st) == 0
    dx = torch.empty(M, K, dtype=torch.bfloat16, device="cuda")
    dw = torch.empty(N, K, device="cuda")
    db = torch.empty(N, device="cuda")
    args = lambda dxp, dwp, dbp, flags: (go.data_ptr(), 1, N, ws[0].data_ptr(), w0.data_ptr(), 0, K, dxp, 1, K, dwp, K, dbp,
                                         M, N, K, 32, 1, flags, 0, 0, noise.data_ptr(), ws[2].data_ptr(), ws[1].data_ptr(),
                                         ws[3].data_ptr(), None, st)
    assert lib.axs6_linear_bwd(*args(None, dw.data_ptr(), None, 2)) == 0
    assert lib.axs6_linear_bwd(*args(dx.data_ptr(), None, db.data_ptr(), 2 | 32 | 64)) == 0
    gemm_status_ok()
    assert torch.equal(dx.float(), grads[True][0]) and torch.equal(dw, grads[True][1])
    assert torch.allclose(db, go.float().sum(0), rtol=1e-5, atol=1e-4)


def test_linear_golden_from_reference(linear_cases, manifest):
    """Cases recorded by running the reference's mixed-precision Function on the CPU (with the
    same stochastic draws): outputs agree within the bf16-output tolerance, dtypes as the reference."""
    for name in ("lin_mixed_a", "lin_mixed_b", "lin_mixed_c"):
        info = manifest["cases"][name]
        M = int(np.prod(info["M"])); K = info["K"]; N = info["N"]
        xb = linear_cases[f"{name}.x"]
        x = to_cuda(xb.view(np.float32) if xb.dtype == np.uint32 else xb).reshape(*info["M"], K).requires_grad_(True)
        w = to_cuda(linear_cases[f"{name}.w"].view(np.float32)).reshape(N, K).requires_grad_(True)
        b = to_cuda(linear_cases[f"{name}.b"].view(np.float32)).requires_grad_(True) if info["bias"] else None
        g = to_cuda(linear_cases[f"{name}.g"].view(np.float32)).reshape(*info["M"], N)
        y = mp.axs_linear_mixed_precision(x, w, b, 32, info["quantize_input"], info["quantize_grad"])
        assert str(y.dtype).endswith(info["y_dtype"])
        mp._noise_for_next_backward = torch.from_numpy(linear_cases[f"{name}.noise"]).cuda() if info["quantize_grad"] else None
        y.backward(g.to(y.dtype))
        mp._noise_for_next_backward = None
        gemm_status_ok()
        want_y = torch.from_numpy(linear_cases[f"{name}.y"].view(np.float32)).reshape(y.shape)
        want_dx = torch.from_numpy(linear_cases[f"{name}.dx"].view(np.float32)).reshape(x.shape)
        want_dw = torch.from_numpy(linear_cases[f"{name}.dw"].view(np.float32)).reshape(N, K)
        assert rel(y.float().cpu(), want_y) < TOL_BF16_OUT, name
        assert rel(x.grad.float().cpu(), want_dx) < TOL_BF16_OUT, name
        assert rel(w.grad.cpu(), want_dw) < TOL, name
        assert str(w.grad.dtype).endswith(info["dw_dtype"]) and str(x.grad.dtype).endswith(info["dx_dtype"])
        if info["bias"]:
            want_db = torch.from_numpy(linear_cases[f"{name}.db"].view(np.float32))
            assert rel(b.grad.cpu(), want_db) < 1e-5, name


def test_module_and_conversion():
    torch.manual_seed(0)
    lin = mp.AXSLinearMixedPrecision(128, 64).cuda()
    x = torch.randn(4, 10, 128, device="cuda", requires_grad=True)
    y = lin(x)
    assert y.shape == (4, 10, 64) and y.dtype == torch.bfloat16
    y.float().sum().backward()
    assert lin.weight.grad.dtype == torch.float32 and lin.bias.grad.dtype == torch.float32 and x.grad.shape == x.shape
    lin._warmup_active = True
    assert torch.equal(lin(x), torch.nn.functional.linear(x.to(torch.bfloat16), lin.weight.to(torch.bfloat16),
                                                          lin.bias.to(torch.bfloat16)))
    net = torch.nn.Sequential(torch.nn.Linear(32, 64), torch.nn.ReLU(), torch.nn.Linear(64, 8)).cuda()
    conv = mp.convert_to_axs_mixed_precision(net)
    assert isinstance(conv[0], mp.AXSLinearMixedPrecision) and isinstance(conv[2], mp.AXSLinearMixedPrecision)
    assert conv(torch.randn(5, 32, device="cuda")).shape == (5, 8)
    with pytest.raises(RuntimeError, match="requires CUDA tensors"):
        mp.axs_linear_mixed_precision(torch.randn(2, 32), torch.randn(4, 32))


@pytest.mark.parametrize("rows,cols", [(1, 1), (33, 70), (1000, 64), (16384, 4096)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_bias_grad_column_sums(rows, cols, dtype):
    g = torch.randn(rows, cols, generator=torch.Generator().manual_seed(rows + cols)).to(dtype)
    out = ops.bias_grad(g.cuda())
    assert out.dtype == torch.float32 and out.shape == (cols,)
    ref = g.double().sum(0)
    assert float((out.cpu().double() - ref).abs().max()) <= 1e-5 * max(1.0, float(ref.abs().max())) * (rows ** 0.5)
    again = ops.bias_grad(g.cuda())
    assert torch.equal(out, again)          # fixed summation order


@pytest.mark.parametrize("a_mn,b_mn", [(0, 0), (0, 1), (1, 0), (1, 1)])
@pytest.mark.parametrize("M,N,K", [(128, 256, 32), (256, 512, 512), (1000, 776, 516), (2048, 1024, 2048)])
def test_gemm_tf32_against_fp32_matmul(M, N, K, a_mn, b_mn):
    """fp32 operands consumed as TF32: operands pre-rounded to TF32 must give an fp32-exact
    product; raw fp32 operands stay within the 1e-3 bar."""
    g = torch.Generator().manual_seed(M + N + K + a_mn * 2 + b_mn)
    A = torch.randn((K, M) if a_mn else (M, K), generator=g)
    B = torch.randn((K, N) if b_mn else (N, K), generator=g)
    def tf32(t):            # keep 10 mantissa bits, round to nearest (ties away)
        return ((t.view(torch.int32) + 0x1000) & ~0x1FFF).view(torch.float32)
    At, Bt = tf32(A), tf32(B)
    C = ops.gemm_bf16(At.cuda(), Bt.cuda(), a_mn=bool(a_mn), b_mn=bool(b_mn))    # MN-major fp32 operands go through a transposed copy
    gemm_status_ok()
    Af = At.t() if a_mn else At
    Bf = Bt if b_mn else Bt.t()
    assert rel(C.cpu(), Af.double() @ Bf.double()) < 1e-5
    C2 = ops.gemm_bf16(A.cuda(), B.cuda(), a_mn=bool(a_mn), b_mn=bool(b_mn))
    Af = A.t() if a_mn else A
    Bf = B if b_mn else B.t()
    assert rel(C2.cpu(), Af.double() @ Bf.double()) < TOL


def test_fq_tf32_rounded_output():
    x = torch.randn(64, 256, generator=torch.Generator().manual_seed(8)).cuda()
    lib = _lib.load()
    y = torch.empty_like(x)
    st = torch.cuda.current_stream().cuda_stream
    assert lib.axs6_fq(x.data_ptr(), y.data_ptr(), 0, 0, 64, 256, 256, 256, 32, 1, 0, 2, 0, 0, st) == 0
    ref = qu.fused_fake_quantize(x)
    want = ((ref.view(torch.int32) + 0x1000) & ~0x1FFF).view(torch.float32)
    assert torch.equal(y, want)
    assert int((y.view(torch.int32) & 0x1FFF).abs().max()) == 0


# ------------------------------------------------------------------ fp32 graphs (TF32 tensor cores)
fu = importlib.import_module("axs6_b200.unified.functional_unified")
nnf = importlib.import_module("axs6_b200.nn.functional")
ub = importlib.import_module("axs6_b200.unified.backend")
tk = importlib.import_module("axs6_b200.unified.triton_kernels")
_lf = importlib.import_module("axs6_b200._linear_fn")


@pytest.mark.parametrize("family", ["unified", "v1"])
def test_fp32_linear_golden_from_reference(family, linear_cases, manifest):
    """Cases recorded from the reference's fp32 autograd functions on the CPU (same stochastic
    draws): y, dx, dw, db within 1e-3 relative Frobenius; fp32 everywhere."""
    fn = fu.axs_linear_unified if family == "unified" else nnf.axs_linear
    for name in (f"lin_{family}_a", f"lin_{family}_b", f"lin_{family}_c"):
        info = manifest["cases"][name]
        K, N = info["K"], info["N"]
        x = to_cuda(linear_cases[f"{name}.x"].view(np.float32)).reshape(*info["M"], K).requires_grad_(True)
        w = to_cuda(linear_cases[f"{name}.w"].view(np.float32)).reshape(N, K).requires_grad_(True)
        b = to_cuda(linear_cases[f"{name}.b"].view(np.float32)).requires_grad_(True) if info["bias"] else None
        g = to_cuda(linear_cases[f"{name}.g"].view(np.float32)).reshape(*info["M"], N)
        y = fn(x, w, b, 32, info["quantize_input"], info["quantize_grad"])
        assert y.dtype == torch.float32
        _lf._noise_for_next_backward = torch.from_numpy(linear_cases[f"{name}.noise"]).cuda() if info["quantize_grad"] else None
        y.backward(g)
        _lf._noise_for_next_backward = None
        gemm_status_ok()
        for got, key in ((y, "y"), (x.grad, "dx"), (w.grad, "dw")):
            want = torch.from_numpy(linear_cases[f"{name}.{key}"].view(np.float32)).reshape(got.shape)
            assert got.dtype == torch.float32
            assert rel(got.cpu(), want) < TOL, (name, key, rel(got.cpu(), want))
        if info["bias"]:
            want = torch.from_numpy(linear_cases[f"{name}.db"].view(np.float32))
            assert rel(b.grad.cpu(), want) < TOL, name            # column sums of the quantised (TF32-rounded) gradient


def test_accelerated_linear_and_fused_linear_vs_oracle():
    """Forward-only entry points against the fp32 matmul of the oracle's fake-quantised
    operands; shapes as in the reference's fused-linear tests (ragged K, batched input, M = 1)."""
    rng = np.random.default_rng(21)
    for shape, K, N, bias, qin in (((64,), 128, 96, True, True), ((4, 8), 33, 20, False, True), ((2, 3, 5), 50, 17, True, True),
                                   ((1,), 100, 64, True, False), ((7,), 127, 40, False, True), ((16,), 255, 33, True, True)):
        x = rng.standard_normal((*shape, K), dtype=np.float32)
        w = rng.standard_normal((N, K), dtype=np.float32) * 0.1
        b = rng.standard_normal(N, dtype=np.float32) if bias else None
        xq = oracle.fused_fake_quantize(x.reshape(-1, K)) if qin else x.reshape(-1, K)
        wq = oracle.fused_fake_quantize(w)
        ref = xq.astype(np.float64) @ wq.astype(np.float64).T + (b.astype(np.float64) if bias else 0.0)
        ref = torch.from_numpy(ref).reshape(*shape, N)
        xt, wt = torch.from_numpy(x).cuda(), torch.from_numpy(w).cuda()
        bt = torch.from_numpy(b).cuda() if bias else None
        for fn in (ub.accelerated_linear, tk.triton_fused_linear):
            y = fn(xt, wt, bt, 32, qin)
            assert y.dtype == torch.float32 and y.shape == ref.shape and y.is_contiguous()
            assert rel(y.cpu(), ref) < TOL
    gemm_status_ok()
    with pytest.raises(ValueError, match="block_size=32"):
        tk.triton_fused_linear(xt, wt, None, 16)
    with pytest.raises(RuntimeError, match="requires CUDA tensors"):
        tk.triton_fused_linear(torch.randn(2, 32), torch.randn(4, 32))
    yb = tk.triton_fused_linear(xt.to(torch.bfloat16), wt)
    assert yb.dtype == torch.bfloat16


def test_accelerated_matmul():
    g = torch.Generator().manual_seed(2)
    a = torch.randn(3, 40, 96, generator=g)
    b = torch.randn(96, 56, generator=g)
    out = ub.accelerated_matmul(a.cuda(), b.cuda())
    gemm_status_ok()
    assert out.dtype == torch.float32 and out.shape == (3, 40, 56)
    assert rel(out.cpu(), a.double() @ b.double()) < TOL
    outb = ub.accelerated_matmul(a.cuda().to(torch.bfloat16), b.cuda().to(torch.bfloat16))
    assert outb.dtype == torch.float32
    assert rel(outb.cpu(), a.to(torch.bfloat16).double() @ b.to(torch.bfloat16).double()) < 1e-5
    m = fu.axs_matmul_unified(a.cuda(), b.cuda())
    aq = oracle.fused_fake_quantize(a.numpy()); bq = oracle.fused_fake_quantize(b.numpy())
    assert rel(m.cpu(), torch.from_numpy(aq.astype(np.float64) @ bq.astype(np.float64))) < TOL


def test_fp32_modules_train_a_step():
    torch.manual_seed(3)
    um = importlib.import_module("axs6_b200.unified.modules_unified")
    nm = importlib.import_module("axs6_b200.nn.modules")
    for cls in (um.AXSLinearUnified, nm.AXSLinear):
        lin = cls(64, 32).cuda()
        x = torch.randn(10, 64, device="cuda", requires_grad=True)
        y = lin(x)
        assert y.dtype == torch.float32 and y.shape == (10, 32)
        y.sum().backward()
        assert lin.weight.grad.shape == (32, 64) and lin.bias.grad.shape == (32,) and x.grad.shape == x.shape
        # straight-through: with an all-ones upstream gradient db is the row count (quantised ones are exact)
        assert torch.allclose(lin.bias.grad, torch.full((32,), 10.0, device="cuda"), rtol=0.05)
    net = torch.nn.Sequential(torch.nn.Linear(32, 64), torch.nn.ReLU(), torch.nn.Linear(64, 8)).cuda()
    conv = um.convert_to_axs_unified(net)
    assert isinstance(conv[0], um.AXSLinearUnified) and conv(torch.randn(5, 32, device="cuda")).shape == (5, 8)


def test_tf32_entry_rejects_mn_major():
    lib = _lib.load()
    a = torch.zeros(64, 64, device="cuda")
    st = torch.cuda.current_stream().cuda_stream
    assert lib.axs6_gemm_tf32(a.data_ptr(), a.data_ptr(), a.data_ptr(), None, 64, 64, 64, 64, 64, 64, 0, 1, 0, st) == -6
    t = ops.transpose_f32(torch.arange(35 * 50, dtype=torch.float32, device="cuda").reshape(35, 50))
    assert torch.equal(t, torch.arange(35 * 50, dtype=torch.float32, device="cuda").reshape(35, 50).t())


def test_split_k_weight_gradient_product_is_deterministic_and_accurate():
    """The optional split-K mode of the 2-CTA kernel (fp32 output, red.add onto a zeroed buffer):
    two partials commute, so the result is reproducible."""
    lib = _lib.load()
    g = torch.Generator().manual_seed(12)
    M, N, K = 1024, 1024, 4096                       # 16 tile pairs
    A = torch.randn(K, M, generator=g).to(torch.bfloat16).cuda()
    B = torch.randn(K, N, generator=g).to(torch.bfloat16).cuda()
    ref = (A.float().t().double() @ B.float().double()).cpu()
    outs = []
    try:
        lib.axs6_tune(7, 2)                          # pairs
        for mode in (2, 2, 1):                       # split, split again, no split
            lib.axs6_tune(3, mode)
            outs.append(ops.gemm_bf16(A, B, a_mn=True, b_mn=True))
    finally:
        lib.axs6_tune(7, 0); lib.axs6_tune(3, 0)
    gemm_status_ok()
    assert torch.equal(outs[0], outs[1])
    assert rel(outs[0].cpu(), ref) < 1e-5 and rel(outs[2].cpu(), ref) < 1e-5


class _DecoderBlock(torch.nn.Module):
    """Pre-norm decoder block (d_model 256, 4 heads, FFN 1024) with every Linear supplied by `linear`."""
    D, HEADS, FFN = 256, 4, 1024

    def __init__(self, linear):
        super().__init__()
        D = self.D
        self.ln1, self.ln2 = torch.nn.LayerNorm(D), torch.nn.LayerNorm(D)
        self.q, self.k, self.v, self.o = (linear(D, D) for _ in range(4))
        self.fc1, self.fc2 = linear(D, self.FFN), linear(self.FFN, D)

    def forward(self, x):
        B, T, D = x.shape
        F = torch.nn.functional
        h = self.ln1(x.float()).to(torch.bfloat16)
        q, k, v = (m(h).view(B, T, self.HEADS, -1).transpose(1, 2) for m in (self.q, self.k, self.v))
        a = F.scaled_dot_product_attention(q, k, v, is_causal=True).transpose(1, 2).reshape(B, T, D)
        x = x + self.o(a)
        h = self.ln2(x.float()).to(torch.bfloat16)
        return x + self.fc2(F.gelu(self.fc1(h)))


@pytest.mark.parametrize("M,N,K,bias", [(1024, 1024, 8192, False), (512, 1000, 4096, True), (256, 256, 16384, False)])
def test_split_k_with_workspace_is_reproducible(M, N, K, bias):
    """Few output tiles, long contraction (a small layer's weight gradient): with a workspace the product is split more
    than two ways, the partials are added in index order, and two runs agree bit for bit; without one at most two
    partials are formed.  Both within 1e-5 of the fp32 product."""
    lib = _lib.load()
    g = torch.Generator().manual_seed(M + N + K)
    A = torch.randn(K, M, generator=g).to(torch.bfloat16).cuda()
    B = torch.randn(K, N, generator=g).to(torch.bfloat16).cuda()
    bv = torch.randn(N, generator=g).cuda() if bias else None
    ref = A.float().t().double() @ B.float().double() + (bv.double() if bias else 0.0)
    need = int(lib.axs6_gemm_workspace_bytes(M, N, K, 0))
    assert need > 0 and int(lib.axs6_gemm_workspace_bytes(M, N, K, 1)) == 0
    ws = torch.empty(need, dtype=torch.uint8, device="cuda")
    st = torch.cuda.current_stream().cuda_stream
    outs = []
    for _ in range(3):
        c = torch.full((M, N), float("nan"), device="cuda")
        assert lib.axs6_gemm_bf16_ws(A.data_ptr(), B.data_ptr(), c.data_ptr(), bv.data_ptr() if bias else None, M, N, K, M,
                                     ops._row_pitch(B), N, 1, 1, 0, ws.data_ptr(), need, st) == 0
        outs.append(c)
    gemm_status_ok()
    assert torch.equal(outs[0], outs[1]) and torch.equal(outs[0], outs[2])
    assert rel(outs[0], ref.cuda()) < 1e-5
    plain = torch.empty(M, N, device="cuda")
    assert lib.axs6_gemm_bf16(A.data_ptr(), B.data_ptr(), plain.data_ptr(), bv.data_ptr() if bias else None, M, N, K, M,
                              ops._row_pitch(B), N, 1, 1, 0, st) == 0
    assert rel(plain, ref.cuda()) < 1e-5
    small = torch.empty(M, N, device="cuda")          # a workspace that is too small is ignored
    assert lib.axs6_gemm_bf16_ws(A.data_ptr(), B.data_ptr(), small.data_ptr(), bv.data_ptr() if bias else None, M, N, K, M,
                                 ops._row_pitch(B), N, 1, 1, 0, ws.data_ptr(), 1024, st) == 0
    assert torch.equal(small, plain)


def test_minigpt_block_trains_with_axs6_linears():
    """A decoder block built on AXSLinearMixedPrecision: forward/backward run, gradients reach every
    parameter, a few AdamW steps reduce the loss (convergence smoke test in the spirit of
    tests/test_mixed_precision.py:286-348 of the reference)."""
    torch.manual_seed(0)
    blk = _DecoderBlock(lambda i, o, bias=True: mp.AXSLinearMixedPrecision(i, o, bias=bias)).cuda()
    head = mp.AXSLinearMixedPrecision(_DecoderBlock.D, 64).cuda()
    params = list(blk.parameters()) + list(head.parameters())
    opt = torch.optim.AdamW(params, lr=1e-3)
    x = torch.randn(2, 128, _DecoderBlock.D, device="cuda").to(torch.bfloat16)
    y = torch.randint(0, 64, (2 * 128,), device="cuda")
    losses = []
    for _ in range(12):
        opt.zero_grad()
        loss = torch.nn.functional.cross_entropy(head(blk(x)).float().view(-1, 64), y)
        loss.backward()
        opt.step()
        losses.append(float(loss))
    assert all(p.grad is not None for p in params)
    assert losses[-1] < losses[0] * 0.9
    gemm_status_ok()


@pytest.mark.parametrize("M,K,N", [(512, 1024, 768), (300, 96, 200)])
def test_saved_activation_as_records_gives_the_same_gradients(M, K, N):
    """SAVE_PACKED_INPUT keeps the activation for backward as 25-byte wire records (25/64 of the bf16 bytes).  The
    records decode to the fake-quantised input wherever the input is not exactly zero, so on an input without
    zeros y, dX, dW and db are bit-identical to the default path (same draws for the gradient's rounding)."""
    g = torch.Generator(device="cuda").manual_seed(M + K + N)
    x = torch.randn(M, K, generator=g, device="cuda").to(torch.bfloat16)
    x = torch.where(x == 0, torch.full_like(x, 0.5), x)
    w = (torch.randn(N, K, generator=g, device="cuda") * 0.05)
    b = torch.randn(N, generator=g, device="cuda")
    go = torch.randn(M, N, generator=g, device="cuda").to(torch.bfloat16)
    nblk = -(-N // 32)
    noise = torch.rand(M, nblk, 32, generator=g, device="cuda")
    res = {}
    saved_bytes = {}
    for flag in (False, True):
        mp.SAVE_PACKED_INPUT = flag
        try:
            xi = x.clone().requires_grad_(True)
            wi = w.clone().requires_grad_(True)
            bi = b.clone().requires_grad_(True)
            y = mp.axs_linear_mixed_precision(xi, wi, bi, 32, True, True)
            saved = y.grad_fn.saved_tensors[0]
            saved_bytes[flag] = saved.numel() * saved.element_size()
            mp._noise_for_next_backward = noise
            y.backward(go)
            res[flag] = (y.detach(), xi.grad, wi.grad, bi.grad)
        finally:
            mp.SAVE_PACKED_INPUT = False
    assert saved_bytes[True] == M * (K // 32) * 25 and saved_bytes[False] == M * K * 2
    for got, want, name in zip(res[True], res[False], ("y", "dx", "dw", "db")):
        assert torch.equal(got, want), name
