"""GPU parity of the GEMM and the AXS-6 Linear at the size the benchmark times
(M = 16384, K = N = 4096) and on multi-wave shapes, through the C ABI.

At this size every product runs the CTA-pair kernel over many waves of tiles (1024 / 1024 / 256
tile pairs on 74 clusters), Y and dX leave as bf16, and the fp32 weight gradient takes the
tail-split branch (its last, partly filled wave is computed as two K halves).  None of that is
reached by the small cases of test_gpu_linear.py.

References: the same operands multiplied by ``torch.matmul`` in fp32 on the GPU (TF32 off), and a
sample of output rows recomputed by the CPU oracle in double precision.  Tolerances (relative
Frobenius; the stated GEMM bar is 1e-3): fp32 accumulator output 1e-5 up to K = 2048, growing as
sqrt(K) to 5e-5 at K = 16384, because both sides accumulate in fp32; bf16 output is that accumulator
rounded once: every element within half a bf16 ulp of the fp32 reference (plus the accumulation noise).
"""
import importlib

import numpy as np
import pytest
import torch

import oracle
from gpu_util import to_cuda

pytestmark = pytest.mark.gpu

from axs6_b200 import _lib, ops  # noqa: E402

mp = importlib.import_module("axs6_b200.unified.mixed_precision")


def rel(a: torch.Tensor, b: torch.Tensor) -> float:
    a, b = a.double(), b.double()
    return float((a - b).norm() / b.norm())


def gemm_status_ok():
    assert _lib.load().axs6_gemm_status() == 0, "a bounded wait inside the GEMM kernel gave up"


def fp32_matmul(a: torch.Tensor, b: torch.Tensor, a_mn: bool, b_mn: bool) -> torch.Tensor:
    prev = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    try:
        af = a.float().t() if a_mn else a.float()
        bf = b.float() if b_mn else b.float().t()
        return af @ bf
    finally:
        torch.backends.cuda.matmul.allow_tf32 = prev


def fp32_tol(K: int) -> float:
    """Two fp32 accumulations of K products in different orders differ by about sqrt(K) * 2^-24 relative to the
    result's typical magnitude; 1e-5 up to K = 2048, 5e-5 at K = 16384 (the stated GEMM bar is 1e-3)."""
    return max(1e-5, 4e-7 * K ** 0.5)


def check_bf16_output(c_bf16: torch.Tensor, ref_f32: torch.Tensor) -> None:
    """bf16 output = the fp32 accumulator rounded once: every element within half a bf16 ulp (2^-8 relative) of the fp32
    reference, plus the fp32 accumulation-order noise (absolute, 2e-4 of the output's rms: sums that cancel to almost
    zero have no meaningful relative error)."""
    err = (c_bf16.float() - ref_f32).abs()
    allowed = ref_f32.abs() * (2.0 ** -8) * 1.01 + 2e-4 * float(ref_f32.double().pow(2).mean().sqrt())
    bad = int((err > allowed).sum())
    assert bad == 0, f"{bad} of {c_bf16.numel()} bf16 outputs are further than half an ulp from the fp32 product"
    assert rel(c_bf16.float(), ref_f32) < 2.5e-3


def check_sampled_rows(c: torch.Tensor, a: torch.Tensor, b: torch.Tensor, a_mn: bool, b_mn: bool, nrows: int, tol: float,
                       seed: int) -> None:
    """`nrows` random output rows against the CPU oracle's product in double precision."""
    M = c.shape[0]
    idx = np.sort(np.random.default_rng(seed).choice(M, size=min(nrows, M), replace=False))
    it = torch.from_numpy(idx).cuda()
    a_rows = (a[:, it].t() if a_mn else a[it]).float().cpu().numpy()            # (nrows, K)
    b_nk = (b.t() if b_mn else b).float().cpu().numpy()                         # (N, K)
    want = oracle.gemm_nt(np.ascontiguousarray(a_rows), np.ascontiguousarray(b_nk))
    got = c[it].float().cpu()
    assert rel(got, torch.from_numpy(want)) < tol


CONFIG4 = [  # name, M, N, K, a_mn, b_mn, out dtype
    ("fwd", 16384, 4096, 4096, 0, 0, torch.bfloat16),
    ("dx", 16384, 4096, 4096, 0, 1, torch.bfloat16),
    ("dw", 4096, 4096, 16384, 1, 1, torch.float32),
]


@pytest.mark.parametrize("name,M,N,K,a_mn,b_mn,odt", CONFIG4, ids=[c[0] for c in CONFIG4])
def test_gemm_at_benchmark_size(name, M, N, K, a_mn, b_mn, odt):
    g = torch.Generator(device="cuda").manual_seed(M + 3 * N + 7 * K + a_mn + 2 * b_mn)
    a = torch.randn((K, M) if a_mn else (M, K), generator=g, device="cuda").to(torch.bfloat16)
    b = torch.randn((K, N) if b_mn else (N, K), generator=g, device="cuda").to(torch.bfloat16)
    ref = fp32_matmul(a, b, bool(a_mn), bool(b_mn))
    c = ops.gemm_bf16(a, b, a_mn=bool(a_mn), b_mn=bool(b_mn), out_dtype=odt)
    gemm_status_ok()
    if odt == torch.float32:
        assert rel(c, ref) < fp32_tol(K)
        check_sampled_rows(c, a, b, bool(a_mn), bool(b_mn), 256, fp32_tol(K), 11)
    else:
        check_bf16_output(c, ref)
        check_sampled_rows(c, a, b, bool(a_mn), bool(b_mn), 256, 2.5e-3, 12)
        # the fp32 accumulator of the same product
        c32 = ops.gemm_bf16(a, b, a_mn=bool(a_mn), b_mn=bool(b_mn), out_dtype=torch.float32)
        gemm_status_ok()
        assert rel(c32, ref) < fp32_tol(K)


def test_weight_gradient_product_with_and_without_tail_split():
    """4096 x 4096 from 16384 rows: 256 tile pairs on 74 clusters.  Default = last wave split in two K halves;
    tune key 3 = 1 = no split.  Both within 1e-5 of the fp32 product, each reproducible run to run."""
    lib = _lib.load()
    g = torch.Generator(device="cuda").manual_seed(99)
    a = torch.randn(16384, 4096, generator=g, device="cuda").to(torch.bfloat16)
    b = torch.randn(16384, 4096, generator=g, device="cuda").to(torch.bfloat16)
    ref = fp32_matmul(a, b, True, True)
    outs = {}
    try:
        for mode in (0, 1):
            lib.axs6_tune(3, mode)
            outs[mode] = [ops.gemm_bf16(a, b, a_mn=True, b_mn=True) for _ in range(2)]
    finally:
        lib.axs6_tune(3, 0)
    gemm_status_ok()
    for mode in (0, 1):
        assert torch.equal(outs[mode][0], outs[mode][1]), f"mode {mode}: not reproducible"
        assert rel(outs[mode][0], ref) < fp32_tol(16384)
    assert rel(outs[0][0], outs[1][0]) < 1e-5


# Multi-wave shapes whose partial tiles land in later waves and at the tail-split boundaries (74 clusters):
# 75 tile pairs (remainder 1), 111 (2 x remainder = clusters), 149 (two full waves + 1), ragged M and N,
# K not a multiple of 64.
WAVES = [
    ("75_pairs", 15 * 256, 5 * 256, 2048),
    ("111_pairs", 37 * 256, 3 * 256, 2048),
    ("149_pairs", 149 * 256, 256, 2048),
    ("75_pairs_ragged", 15 * 256 - 56, 5 * 256 - 24, 2056),
    ("ragged_19208x4104", 19208, 4104, 520),
    ("148_pairs_exact", 37 * 256, 4 * 256, 1032),
]


@pytest.mark.parametrize("a_mn,b_mn", [(0, 0), (0, 1), (1, 1)])
@pytest.mark.parametrize("name,M,N,K", WAVES, ids=[w[0] for w in WAVES])
def test_gemm_multi_wave_shapes(name, M, N, K, a_mn, b_mn):
    g = torch.Generator(device="cuda").manual_seed(M + N + K + a_mn + 2 * b_mn)
    a = torch.randn((K, M) if a_mn else (M, K), generator=g, device="cuda").to(torch.bfloat16)
    b = torch.randn((K, N) if b_mn else (N, K), generator=g, device="cuda").to(torch.bfloat16)
    ref = fp32_matmul(a, b, bool(a_mn), bool(b_mn))
    c32 = ops.gemm_bf16(a, b, a_mn=bool(a_mn), b_mn=bool(b_mn), out_dtype=torch.float32)
    gemm_status_ok()
    assert c32.shape == (M, N)
    assert rel(c32, ref) < fp32_tol(K)
    c16 = ops.gemm_bf16(a, b, a_mn=bool(a_mn), b_mn=bool(b_mn), out_dtype=torch.bfloat16)
    gemm_status_ok()
    check_bf16_output(c16, ref)
    check_sampled_rows(c32, a, b, bool(a_mn), bool(b_mn), 64, fp32_tol(K), 5)


WIDE = [(512, 512, 256), (1000, 776, 520), (4096, 4096, 1024), (256, 520, 4096), (19208, 4104, 520), (37 * 256, 1024 + 8, 1032)]


@pytest.mark.parametrize("a_mn,b_mn", [(0, 0), (0, 1), (1, 1)])
@pytest.mark.parametrize("M,N,K", WIDE)
def test_gemm_wide_tiles_forced(M, N, K, a_mn, b_mn):
    """The 256 x 512 tile kernel (one A tile feeds two 256-column products, two accumulators with their own epilogue
    groups) on every operand layout, forced with tune key 7 = 3: few and many tiles, a second product that is partly or
    wholly outside the matrix, ragged M, K not a multiple of 64; bf16 and fp32 outputs."""
    lib = _lib.load()
    g = torch.Generator(device="cuda").manual_seed(M + N + K + 3 * a_mn + b_mn)
    a = torch.randn((K, M) if a_mn else (M, K), generator=g, device="cuda").to(torch.bfloat16)
    b = torch.randn((K, N) if b_mn else (N, K), generator=g, device="cuda").to(torch.bfloat16)
    bias = torch.randn(N, generator=g, device="cuda")
    ref = fp32_matmul(a, b, bool(a_mn), bool(b_mn)) + bias
    try:
        lib.axs6_tune(7, 3)
        c32 = ops.gemm_bf16(a, b, bias=bias, a_mn=bool(a_mn), b_mn=bool(b_mn), out_dtype=torch.float32)
        c16 = ops.gemm_bf16(a, b, bias=bias, a_mn=bool(a_mn), b_mn=bool(b_mn), out_dtype=torch.bfloat16)
        again = ops.gemm_bf16(a, b, bias=bias, a_mn=bool(a_mn), b_mn=bool(b_mn), out_dtype=torch.float32)
    finally:
        lib.axs6_tune(7, 0)
    gemm_status_ok()
    assert rel(c32, ref) < fp32_tol(K)
    check_bf16_output(c16, ref)
    assert torch.equal(c32, again)
    lib.axs6_tune(7, 2)                      # the 256 x 256 kernel on the same operands
    try:
        narrow = ops.gemm_bf16(a, b, bias=bias, a_mn=bool(a_mn), b_mn=bool(b_mn), out_dtype=torch.float32)
    finally:
        lib.axs6_tune(7, 0)
    if K < 2048:                             # no K split in either kernel: the same fp32 sums in the same order
        assert torch.equal(c32, narrow)
    assert rel(c32, narrow) < 1e-6


def test_linear_forward_backward_at_benchmark_size():
    """axs_linear_mixed_precision at M = 16384, K = N = 4096 with supplied rounding draws: y, dX (bf16) and dW (fp32
    accumulator), db against products of the CPU oracle's fake-quantised operands (mixed_precision.py:86-155)."""
    M, K, N = 16384, 4096, 4096
    rng = np.random.default_rng(404)
    x = rng.standard_normal((M, K), dtype=np.float32)
    w = rng.standard_normal((N, K), dtype=np.float32) * np.float32(0.02)
    bias = rng.standard_normal(N, dtype=np.float32) * np.float32(0.1)
    g = rng.standard_normal((M, N), dtype=np.float32)
    noise = rng.integers(0, 1 << 24, size=M * N, dtype=np.int64).astype(np.float32) * np.float32(2.0 ** -24)
    xb, gb = oracle.f32_to_bf16(x), oracle.f32_to_bf16(g)
    # the oracle's operands (bf16 bit patterns), uploaded as they are
    xq = to_cuda(oracle.fused_fake_quantize(xb, 32))
    wq = to_cuda(oracle.fused_fake_quantize(oracle.f32_to_bf16(w), 32))
    gq = to_cuda(oracle.fused_fake_quantize(gb, 32, noise))
    xt = to_cuda(xb).requires_grad_(True)
    wt = torch.from_numpy(w).cuda().requires_grad_(True)
    bt = torch.from_numpy(bias).cuda().requires_grad_(True)
    y = mp.axs_linear_mixed_precision(xt, wt, bt, 32, True, True)
    assert y.dtype == torch.bfloat16 and y.shape == (M, N)
    mp._noise_for_next_backward = torch.from_numpy(noise).cuda()
    y.backward(to_cuda(gb))
    gemm_status_ok()
    ref_y = fp32_matmul(xq, wq, False, False) + bt.detach().to(torch.bfloat16).float()
    assert rel(y.float(), ref_y) < 4e-3
    check_bf16_output(y.detach(), ref_y)
    ref_dx = fp32_matmul(gq, wq, False, True)
    assert xt.grad.dtype == torch.bfloat16
    assert rel(xt.grad.float(), ref_dx) < 4e-3
    check_bf16_output(xt.grad, ref_dx)
    ref_dw = fp32_matmul(gq, xq, True, True)
    assert wt.grad.dtype == torch.float32
    assert rel(wt.grad, ref_dw) < 1e-3
    assert rel(wt.grad, ref_dw) < fp32_tol(M)   # what the fp32 accumulator actually achieves
    ref_db = to_cuda(gb).double().sum(0)
    assert float((bt.grad.double() - ref_db).abs().max()) <= 1e-5 * float(ref_db.abs().max()) * (M ** 0.5)
    # a sample of rows of every product recomputed by the oracle in double precision
    check_sampled_rows(wt.grad, gq, xq, True, True, 64, fp32_tol(M), 21)
    check_sampled_rows(y.detach().float() - bt.detach().to(torch.bfloat16).float(), xq, wq, False, False, 64, 4e-3, 22)
    check_sampled_rows(xt.grad, gq, wq, False, True, 64, 4e-3, 23)


EPILOGUES = [  # name, M, N, K, a_mn, b_mn: store, reduce-add (tail split) and workspace-partial pieces, full and ragged
    ("ragged_store", 15 * 256 - 56, 5 * 256 - 24, 2056, 0, 0),
    ("tail_split_dw", 4096, 4096, 16384, 1, 1),
    ("workspace_split_dw", 1024, 1024, 8192, 1, 1),
    ("workspace_split_ragged", 1000, 776, 8200, 1, 1),
]


@pytest.mark.parametrize("name,M,N,K,a_mn,b_mn", EPILOGUES, ids=[e[0] for e in EPILOGUES])
def test_tensor_map_epilogue_equals_per_thread_stores(name, M, N, K, a_mn, b_mn):
    """The CTA-pair kernel's outputs leave through shared memory and tensor-map stores (tune key 5 = 0) or through
    per-thread stores (key 5 = 1); with and without programmatic dependent launch (key 15); MN-major operands arrive as
    one 4-D box per stage (key 4 = 0) or as two 2-D boxes (key 4 = 1); work units assigned to clusters up front (key 6 = 0)
    or taken over through cluster launch control (key 6 = 1).  Same accumulators, same rounding, same order of the (at
    most two, or workspace-ordered) partials: the results are bit-identical."""
    lib = _lib.load()
    g = torch.Generator(device="cuda").manual_seed(M + N + K)
    a = torch.randn((K, M) if a_mn else (M, K), generator=g, device="cuda").to(torch.bfloat16)
    b = torch.randn((K, N) if b_mn else (N, K), generator=g, device="cuda").to(torch.bfloat16)
    outs = {}
    knobs = ((0, 0, 0, 0), (0, 1, 0, 0), (0, 0, 1, 0), (1, 0, 0, 0), (0, 0, 0, 1))
    try:
        lib.axs6_tune(7, 2)
        for k4, k5, k15, k6 in knobs:
            lib.axs6_tune(4, k4)
            lib.axs6_tune(5, k5)
            lib.axs6_tune(15, k15)
            lib.axs6_tune(6, k6)
            outs[(k4, k5, k15, k6)] = (ops.gemm_bf16(a, b, a_mn=bool(a_mn), b_mn=bool(b_mn), out_dtype=torch.float32),
                                   ops.gemm_bf16(a, b, a_mn=bool(a_mn), b_mn=bool(b_mn), out_dtype=torch.bfloat16))
    finally:
        for key in (4, 5, 6, 15, 7):
            lib.axs6_tune(key, 0)
    gemm_status_ok()
    ref = fp32_matmul(a, b, bool(a_mn), bool(b_mn))
    assert rel(outs[knobs[0]][0], ref) < fp32_tol(K)
    for key in knobs[1:]:
        assert torch.equal(outs[key][0], outs[knobs[0]][0]), f"fp32 output differs with knobs {key}"
        assert torch.equal(outs[key][1], outs[knobs[0]][1]), f"bf16 output differs with knobs {key}"


@pytest.mark.parametrize("M,N,K", [(4096, 2048, 1024), (3000, 1544, 1032), (9472, 1024, 520)])
def test_tf32_gemm_on_cta_pairs(M, N, K):
    """fp32 operands at sizes where the TF32 instantiation of the CTA-pair kernel runs (at least 37 tile pairs):
    operands pre-rounded to TF32 give the fp32 product up to accumulation order; the single-CTA kernel on the same
    operands (tune key 7 = 1) agrees to the same bound."""
    lib = _lib.load()
    g = torch.Generator(device="cuda").manual_seed(M + N + K)
    a = torch.randn(M, K, generator=g, device="cuda")
    b = torch.randn(N, K, generator=g, device="cuda")
    tf32 = lambda t: ((t.view(torch.int32) + 0x1000) & ~0x1FFF).view(torch.float32)
    a, b = tf32(a), tf32(b)
    ref = a.double() @ b.double().t()
    c = ops.gemm_bf16(a, b)
    gemm_status_ok()
    assert rel(c, ref) < fp32_tol(K)
    try:
        lib.axs6_tune(7, 1)
        c1 = ops.gemm_bf16(a, b)
    finally:
        lib.axs6_tune(7, 0)
    gemm_status_ok()
    assert rel(c1, ref) < fp32_tol(K)
    assert rel(c, c1.double()) < fp32_tol(K)


def test_fp32_graph_linear_at_a_pair_kernel_size():
    """axs_linear_unified (fp32 in / out) at 4096 x 1024 -> 2048: forward within 1e-5 of the fp64 product of the
    fake-quantised operands (three TF32 products), gradients within the TF32 bar of 1e-3."""
    fu = importlib.import_module("axs6_b200.unified.functional_unified")
    qu = importlib.import_module("axs6_b200.unified.quantize_unified")
    M, K, N = 4096, 1024, 2048
    g = torch.Generator(device="cuda").manual_seed(77)
    x = torch.randn(M, K, generator=g, device="cuda").requires_grad_(True)
    w = (torch.randn(N, K, generator=g, device="cuda") * 0.05).requires_grad_(True)
    bias = torch.randn(N, generator=g, device="cuda").requires_grad_(True)
    go = torch.randn(M, N, generator=g, device="cuda")
    y = fu.axs_linear_unified(x, w, bias, quantize_grad=False)
    y.backward(go)
    gemm_status_ok()
    xq, wq = qu.fused_fake_quantize(x.detach()).double(), qu.fused_fake_quantize(w.detach()).double()
    assert rel(y.detach(), xq @ wq.t() + bias.detach().double()) < 1e-5
    assert rel(x.grad, go.double() @ wq) < 1e-3
    assert rel(w.grad, go.double().t() @ xq) < 1e-3
    assert rel(bias.grad, go.double().sum(0)) < 1e-5
