"""GPU parity of the split code layout and of the decode-on-load GEMM (operands held as AXS-6 codes),
through the C ABI.

* split layout = the bytes of the 25-byte wire record in two planes: checked bit for bit against the CPU
  oracle's codes and exponents, and unpack(split) against unpack(wire);
* axs6_gemm_packed: the operands the kernel decodes are bit-identical to axs6_unpack(..., bf16) of the same
  codes, so the product must agree with axs6_gemm_bf16 on those unpacked operands to fp32 accumulation-order
  noise (1e-5 relative Frobenius) and with the fp32 matmul of the oracle's dequantised operands to 1e-5
  (the stated GEMM bar is 1e-3).  All three products of the Linear (K-major / MN-major operands), one or both
  operands packed, ragged M and N, multi-wave tile counts, all-zero and extreme-exponent blocks.
"""
import numpy as np
import pytest
import torch

import oracle
from gpu_util import to_cuda

pytestmark = pytest.mark.gpu

from axs6_b200 import _lib, ops  # noqa: E402


def rel(a, b) -> float:
    a, b = a.double(), b.double()
    return float((a - b).norm() / b.norm())


def assert_half_ulp(c_bf16, ref_f32):
    """bf16 output within half a bf16 ulp of the fp32 result (plus fp32 accumulation-order noise, absolute)."""
    err = (c_bf16.float() - ref_f32).abs()
    allowed = ref_f32.abs() * (2.0 ** -8) * 1.01 + 2e-4 * float(ref_f32.double().pow(2).mean().sqrt())
    assert int((err > allowed).sum()) == 0


def gemm_status_ok():
    assert _lib.load().axs6_gemm_status() == 0, "a bounded wait inside the GEMM kernel gave up"


@pytest.mark.parametrize("rows,cols", [(4, 64), (33, 192), (256, 4096)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_split_layout_matches_oracle_and_wire(rows, cols, dtype):
    rng = np.random.default_rng(rows + cols)
    x = rng.standard_normal((rows, cols), dtype=np.float32) * (10.0 ** rng.uniform(-3, 2, size=(rows, 1))).astype(np.float32)
    x[0, :32] = 0.0                                            # an all-zero block
    x[1, 5] = 0.0
    xt = torch.from_numpy(x).cuda().to(dtype)
    pk = ops.pack_split(xt)
    xo = xt.float().cpu().numpy()
    se, sg, mg = oracle.quantize(xo, 32, oracle.GRID_NF5)
    wire = oracle.pack_bytes(se, sg, mg, oracle.LAYOUT_WIRE).reshape(rows, cols // 32, 25)
    assert pk.exps.shape == (cols // 64, rows, 2)            # exponents by pairs of blocks: [b // 2, row, b % 2]
    assert np.array_equal(pk.exps.permute(1, 0, 2).reshape(rows, cols // 32).cpu().numpy(), wire[:, :, 0])
    assert np.array_equal(pk.codes.cpu().numpy(), wire[:, :, 1:])
    for odt in (torch.float32, torch.bfloat16):
        back = ops.unpack_split(pk, odt)
        ref = ops.unpack(ops.LAYOUT_WIRE, torch.from_numpy(wire.reshape(-1).copy()).cuda(), rows, cols, 32, ops.GRID_NF5, odt)
        assert torch.equal(back, ref)


def test_split_layout_stochastic_with_supplied_draws():
    rng = np.random.default_rng(3)
    x = rng.standard_normal((64, 256), dtype=np.float32)
    u = rng.random((64, 256), dtype=np.float32)
    pk = ops.pack_split(torch.from_numpy(x).cuda(), rounding="stochastic", noise=torch.from_numpy(u).cuda())
    se, sg, mg = oracle.quantize(x, 32, oracle.GRID_NF5, u.reshape(-1))
    wire = oracle.pack_bytes(se, sg, mg, oracle.LAYOUT_WIRE).reshape(64, 8, 25)
    assert np.array_equal(pk.exps.permute(1, 0, 2).reshape(64, 8).cpu().numpy(), wire[:, :, 0])
    assert np.array_equal(pk.codes.cpu().numpy(), wire[:, :, 1:])


def _operands(M, N, K, a_mn, b_mn, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    sa = 10 ** (torch.rand((K if a_mn else M), 1, generator=g, device="cuda") * 4 - 2)
    a = torch.randn((K, M) if a_mn else (M, K), generator=g, device="cuda") * sa
    b = torch.randn((K, N) if b_mn else (N, K), generator=g, device="cuda") * 0.05
    return a.to(torch.bfloat16), b.to(torch.bfloat16)


SHAPES = [(128, 256, 64), (256, 256, 512), (200, 328, 192), (1000, 776, 1024), (8, 64, 64), (2048, 1024, 2048),
          (37 * 256, 3 * 256, 1024)]


@pytest.mark.parametrize("which", ["a", "b", "ab"])
@pytest.mark.parametrize("a_mn,b_mn", [(0, 0), (0, 1), (1, 1)])
@pytest.mark.parametrize("M,N,K", SHAPES)
def test_gemm_packed_against_unpacked_operands(M, N, K, a_mn, b_mn, which):
    if (a_mn and M % 64) or (b_mn and N % 64):
        pytest.skip("an MN-major packed operand needs a contiguous extent that is a multiple of 64")
    a, b = _operands(M, N, K, a_mn, b_mn, M + N + K + 2 * a_mn + b_mn)
    pa, pb = ops.pack_split(a), ops.pack_split(b)
    ua, ub = ops.unpack_split(pa, torch.bfloat16), ops.unpack_split(pb, torch.bfloat16)
    A = pa if "a" in which else ua
    B = pb if "b" in which else ub
    for odt in (torch.float32, torch.bfloat16):
        c = ops.gemm_packed(A, B, a_mn=bool(a_mn), b_mn=bool(b_mn), out_dtype=odt)
        gemm_status_ok()
        ref = ops.gemm_bf16(ua, ub, a_mn=bool(a_mn), b_mn=bool(b_mn), out_dtype=torch.float32)
        if odt == torch.float32:
            assert rel(c, ref) < 1e-5
        else:
            assert rel(c.float(), ref) < 2.5e-3
            assert_half_ulp(c, ref)
    # and against the oracle's dequantised operands in double precision (sampled rows keep the CPU work small)
    af = oracle.dequantize(*oracle.quantize(a.float().cpu().numpy(), 32, oracle.GRID_NF5), a.shape[1], oracle.GRID_NF5)
    bf = oracle.dequantize(*oracle.quantize(b.float().cpu().numpy(), 32, oracle.GRID_NF5), b.shape[1], oracle.GRID_NF5)
    af = oracle.bf16_to_f32(oracle.f32_to_bf16(af)).reshape(a.shape)
    bf = oracle.bf16_to_f32(oracle.f32_to_bf16(bf)).reshape(b.shape)
    Am = af.T if a_mn else af
    Bm = bf.T if b_mn else bf
    idx = np.sort(np.random.default_rng(1).choice(M, size=min(M, 48), replace=False))
    want = oracle.gemm_nt(np.ascontiguousarray(Am[idx]), np.ascontiguousarray(Bm))
    c32 = ops.gemm_packed(A, B, a_mn=bool(a_mn), b_mn=bool(b_mn))
    assert rel(c32[torch.from_numpy(idx).cuda()].cpu(), torch.from_numpy(want)) < 1e-5


@pytest.mark.parametrize("a_mn,b_mn", [(0, 0), (0, 1), (1, 1)])
def test_gemm_packed_per_warp_arrivals_give_the_same_bits(a_mn, b_mn):
    """axs6_tune(9, 1): every decode warp signals the stage barrier itself instead of the last warp of its group for
    all four.  Same decoded stages, same products: the outputs must be identical, multi-wave shape included."""
    lib = _lib.load()
    M, N, K = 37 * 256, 3 * 256, 1024
    a, b = _operands(M, N, K, a_mn, b_mn, 77 + 2 * a_mn + b_mn)
    pa, pb = ops.pack_split(a), ops.pack_split(b)
    want = ops.gemm_packed(pa, pb, a_mn=bool(a_mn), b_mn=bool(b_mn), out_dtype=torch.bfloat16)
    want_w = ops.gemm_packed(ops.unpack_split(pa, torch.bfloat16), pb, a_mn=bool(a_mn), b_mn=bool(b_mn), out_dtype=torch.bfloat16)
    gemm_status_ok()
    assert lib.axs6_tune(9, 1) == 0
    try:
        got = ops.gemm_packed(pa, pb, a_mn=bool(a_mn), b_mn=bool(b_mn), out_dtype=torch.bfloat16)
        got_w = ops.gemm_packed(ops.unpack_split(pa, torch.bfloat16), pb, a_mn=bool(a_mn), b_mn=bool(b_mn), out_dtype=torch.bfloat16)
        torch.cuda.synchronize()
    finally:
        lib.axs6_tune(9, 0)
    gemm_status_ok()
    assert torch.equal(got, want) and torch.equal(got_w, want_w)


def test_gemm_packed_zero_and_extreme_blocks_and_bias():
    """All-zero blocks (exponent byte 0: the smallest level times 2^-127, a bf16 denormal), tiny and huge block scales,
    and the bias epilogue."""
    M, N, K = 256, 256, 256
    g = torch.Generator(device="cuda").manual_seed(5)
    a = torch.randn(M, K, generator=g, device="cuda")
    a[:, :32] = 0.0
    a[:, 32:64] *= 1e-36
    a[:, 64:96] *= 1e30
    b = torch.randn(N, K, generator=g, device="cuda") * 0.1
    b[:, 64:96] *= 1e-30                       # keeps the products of the huge block finite
    bias = torch.randn(N, generator=g, device="cuda")
    pa, pb = ops.pack_split(a.to(torch.bfloat16)), ops.pack_split(b.to(torch.bfloat16))
    ua, ub = ops.unpack_split(pa, torch.bfloat16), ops.unpack_split(pb, torch.bfloat16)
    c = ops.gemm_packed(pa, pb, bias=bias)
    gemm_status_ok()
    ref = ops.gemm_bf16(ua, ub, bias=bias)
    assert torch.isfinite(c).all()
    assert rel(c, ref) < 1e-5


def test_gemm_packed_argument_checks():
    lib = _lib.load()
    st = torch.cuda.current_stream().cuda_stream
    z = torch.zeros(1 << 16, dtype=torch.uint8, device="cuda")
    c = torch.zeros(64, 64, device="cuda")
    p = z.data_ptr()
    # nothing packed
    assert lib.axs6_gemm_packed(p, None, 64, p, None, 64, c.data_ptr(), None, 64, 64, 64, 64, 0, 0, 0, st) == -1
    # contraction length of a K-major packed operand not a multiple of 64; row count not a multiple of 8
    assert lib.axs6_gemm_packed(p, p, 0, p, p, 0, c.data_ptr(), None, 64, 64, 96, 64, 0, 0, 0, st) == -6
    assert lib.axs6_gemm_packed(p, p, 0, p, p, 0, c.data_ptr(), None, 60, 64, 64, 64, 0, 0, 0, st) == -6
    # misaligned payload plane
    assert lib.axs6_gemm_packed(p + 8, p, 0, p, p, 0, c.data_ptr(), None, 64, 64, 64, 64, 0, 0, 0, st) == -2


@pytest.mark.parametrize("M,K,N", [(256, 256, 192), (1000, 512, 320), (4096, 1024, 1024)])
def test_linear_with_packed_operands_matches_the_two_pass_linear(M, K, N):
    """AXS6_LINEAR_OPERANDS_PACKED against the bf16-workspace path on the same inputs and rounding draws: the
    decoded operands are the same bf16 values (no exact zeros in the data), so y and dX (bf16) agree to rounding
    of accumulation-order noise and dW (fp32) to 1e-6."""
    import importlib
    mp = importlib.import_module("axs6_b200.unified.mixed_precision")
    g = torch.Generator().manual_seed(M + K + N)
    x = torch.randn(M, K, generator=g).cuda()
    w = (torch.randn(N, K, generator=g) * 0.05).cuda()
    b = torch.randn(N, generator=g).cuda()
    go = torch.randn(M, N, generator=g).cuda().to(torch.bfloat16)
    noise = torch.rand(M * N, generator=g).cuda()
    res = {}
    try:
        for packed in (False, True):
            mp.PACKED_OPERANDS = packed
            xt, wt, bt = x.clone().requires_grad_(True), w.clone().requires_grad_(True), b.clone().requires_grad_(True)
            y = mp.axs_linear_mixed_precision(xt, wt, bt, 32, True, True)
            mp._noise_for_next_backward = noise
            y.backward(go)
            res[packed] = (y.detach().float(), xt.grad.clone(), wt.grad.clone(), bt.grad.clone())
    finally:
        mp.PACKED_OPERANDS = False
    gemm_status_ok()
    y0, dx0, dw0, db0 = res[False]
    y1, dx1, dw1, db1 = res[True]
    assert rel(dw1, dw0) < 1e-5
    assert torch.equal(db1, db0)
    for got, want in ((y1, y0), (dx1, dx0)):
        # both are bf16 roundings of fp32 sums that differ in the last bits: a few elements land on the other side of a
        # rounding boundary, each one bf16 ulp (2^-7 relative) away
        assert rel(got, want) < 1e-3
        err = (got - want).abs()
        assert int((err > want.abs() * 2.0 ** -7 * 1.01 + 2e-4 * float(want.pow(2).mean().sqrt())).sum()) == 0
        assert int((err != 0).sum()) <= 0.01 * got.numel()
