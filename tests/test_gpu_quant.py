"""GPU parity of the fake-quantise and codec kernels, called through the C ABI
(axs6_b200.ops -> ctypes -> libaxs6_b200.so), against the golden vectors recorded from the
reference and against the CPU oracle on seeded inputs.  Integer/byte results and fp32/bf16
fake-quant outputs must be BIT-EXACT."""
import json
import os

import numpy as np
import pytest
import torch

import oracle
from gpu_util import assert_bits_equal, to_bits, to_cuda
from helpers import (case_input, config1_input, config2_input, config3_input, expect_bits, fq_case_names, sha)

pytestmark = pytest.mark.gpu

from axs6_b200 import _lib, core, ops  # noqa: E402
from axs6_b200.nn import functional as nnf  # noqa: E402
from axs6_b200.unified import distributed as udist  # noqa: E402
import importlib  # noqa: E402
qu = importlib.import_module("axs6_b200.unified.quantize_unified")  # the package re-exports a function of the same name
from axs6_b200.unified.triton_kernels import triton_fused_fake_quantize  # noqa: E402

with open(os.path.join(os.path.dirname(__file__), "golden", "manifest.json")) as _f:
    _MANIFEST = json.load(_f)
_NEAREST = fq_case_names(_MANIFEST, stochastic=False)
_STOCH = fq_case_names(_MANIFEST, stochastic=True)


def test_library_reports_b200():
    assert _lib.load().axs6_query(0) == 1
    assert _lib.load().axs6_query(1) >= 100


# ------------------------------------------------------------------ golden vectors, nearest
@pytest.mark.parametrize("case", _NEAREST)
def test_golden_nearest(case, fq_cases, manifest):
    x, _, info = case_input(fq_cases, manifest, case)
    B = info["block"]
    xt = to_cuda(x)
    before = _lib.launches()
    y = qu.fused_fake_quantize(xt, B)
    assert _lib.launches() == before + 1
    assert y.dtype == xt.dtype and y.shape == xt.shape
    assert_bits_equal(y, fq_cases[f"{case}.fq_nf5"], "fq_nf5")
    # V1 fake-quantise: always fp32
    y1 = nnf.fake_quantize(xt, B)
    assert y1.dtype == torch.float32
    assert_bits_equal(y1, fq_cases[f"{case}.deq_uni"], "fq_uniform")
    for tag, qfn, dfn in (("nf5", qu.quantize_unified, qu.dequantize_unified), ("uni", core.quantize, core.dequantize)):
        q = qfn(xt, B)
        assert q.signs.dtype == torch.bool and q.magnitudes.dtype == torch.uint8
        assert_bits_equal(q.shared_exponents, fq_cases[f"{case}.{tag}.se"], tag + ".se")
        assert_bits_equal(q.magnitudes, fq_cases[f"{case}.{tag}.mag"], tag + ".mag")
        assert_bits_equal(q.signs, fq_cases[f"{case}.{tag}.sign"], tag + ".sign")
        d = dfn(q)
        assert d.dtype == torch.float32 and d.shape == xt.shape
        assert_bits_equal(d, fq_cases[f"{case}.deq_{tag}"], tag + ".deq")
    if f"{case}.nf5.wire" in fq_cases.files:
        w = udist.pack_wire(xt, B)
        assert w.dtype == torch.int8
        assert_bits_equal(w.view(torch.uint8), fq_cases[f"{case}.nf5.wire"], "wire")
        back = udist.unpack_wire(w, xt.shape, B)
        assert_bits_equal(back, fq_cases[f"{case}.deq_nf5"], "wire roundtrip")
    if f"{case}.nf5.spec" in fq_cases.files:
        s = core.tensor_to_bytes(xt, B, nf5=True)
        assert_bits_equal(s, fq_cases[f"{case}.nf5.spec"], "spec")
        back = core.tensor_from_bytes(s, xt.shape, B, nf5=True)
        assert_bits_equal(back, fq_cases[f"{case}.deq_nf5"], "spec roundtrip")


# ------------------------------------------------------------------ golden vectors, stochastic with given noise
@pytest.mark.parametrize("case", _STOCH)
def test_golden_stochastic_with_noise(case, fq_cases, manifest):
    x, noise, info = case_input(fq_cases, manifest, case)
    B = info["block"]
    xt = to_cuda(x)
    nz = torch.from_numpy(noise).cuda()
    y = ops.fake_quantize(xt, B, ops.GRID_NF5, "stochastic", noise=nz)
    assert_bits_equal(y, fq_cases[f"{case}.fq_nf5"], "fq_nf5 stochastic")
    for tag, grid in (("nf5", ops.GRID_NF5), ("uni", ops.GRID_UNIFORM)):
        se, sg, mg = ops.pack(xt, B, grid, "stochastic", ops.LAYOUT_PLANES, noise=nz)
        assert_bits_equal(se, fq_cases[f"{case}.{tag}.se"], tag + ".se")
        assert_bits_equal(mg, fq_cases[f"{case}.{tag}.mag"], tag + ".mag")
        assert_bits_equal(sg, fq_cases[f"{case}.{tag}.sign"], tag + ".sign")
    y1 = ops.fake_quantize(xt, B, ops.GRID_UNIFORM, "stochastic", out_dtype=torch.float32, noise=nz)
    assert_bits_equal(y1, fq_cases[f"{case}.deq_uni"], "fq_uniform stochastic")


# ------------------------------------------------------------------ BASELINE configs vs manifest hashes and oracle
def test_config1(manifest):
    x = config1_input()
    y = qu.fused_fake_quantize(torch.from_numpy(x).cuda())
    assert_bits_equal(y, oracle.fused_fake_quantize(x), "config1 vs oracle")
    if sha(x) == manifest["hashes"]["config1.input"]:
        assert sha(to_bits(y)) == manifest["hashes"]["config1.fq_nf5"]
        y1 = nnf.fake_quantize(torch.from_numpy(x).cuda())
        assert sha(to_bits(y1)) == manifest["hashes"]["config1.fq_uniform"]


def test_config2_quarter_hashes(manifest):
    xb = oracle.f32_to_bf16(config2_input(2048, 4096))
    assert sha(xb) == manifest["hashes"]["config2_quarter.input"]
    xt = to_cuda(xb)
    w = udist.pack_wire(xt)
    assert sha(to_bits(w.view(torch.uint8))) == manifest["hashes"]["config2_quarter.wire"]
    back = udist.unpack_wire(w, xt.shape)
    assert sha(to_bits(back)) == manifest["hashes"]["config2_quarter.roundtrip"]
    assert sha(to_bits(qu.fused_fake_quantize(xt))) == manifest["hashes"]["config2_quarter.fq_nf5"]


def test_config2_full_roundtrip_properties():
    """8192x4096 bf16: fake-quant == unpack(pack) except at exact zeros, where the codec returns
    +codebook[0]*scale (the reference's behaviour: sign bit clear, code 0 is not zero)."""
    x = config2_input(8192, 4096)
    xt = torch.from_numpy(x).cuda().to(torch.bfloat16)
    w = udist.pack_wire(xt)
    assert w.numel() == 8192 * 128 * 25
    back = udist.unpack_wire(w, xt.shape)
    fq = qu.fused_fake_quantize(xt.float())
    zero = xt == 0
    assert int(zero.sum()) > 100000
    assert torch.equal(back[~zero], fq[~zero])
    assert bool((back[zero] > 0).all())
    # sampled rows against the oracle, bit for bit
    rows = np.random.default_rng(0).choice(8192, 256, replace=False)
    xs = to_bits(xt[torch.from_numpy(rows).cuda()])
    se, sg, mg = oracle.quantize(xs, 32, oracle.GRID_NF5)
    want = oracle.dequantize(se, sg, mg, 4096, oracle.GRID_NF5)
    assert_bits_equal(back[torch.from_numpy(rows).cuda()], want, "sampled rows")


def test_config3_4096(manifest):
    x = config3_input(4096, 4096)
    assert sha(x) == manifest["hashes"]["config3_4096.input"]
    xt = torch.from_numpy(x).cuda()
    assert sha(to_bits(qu.fused_fake_quantize(xt))) == manifest["hashes"]["config3_4096.fq_nf5_f32"]
    assert sha(to_bits(qu.fused_fake_quantize(xt.to(torch.bfloat16)))) == manifest["hashes"]["config3_4096.fq_nf5_bf16"]


@pytest.mark.parametrize("shape", [(256, 256), (8192, 4096)])
@pytest.mark.parametrize("dtype", ["f32", "bf16"])
def test_config3_vs_oracle(shape, dtype):
    x = config3_input(*shape, seed=11)
    xin = oracle.f32_to_bf16(x) if dtype == "bf16" else x
    y = qu.fused_fake_quantize(to_cuda(xin))
    assert_bits_equal(y, oracle.fused_fake_quantize(xin), f"{shape} {dtype}")
    y1 = nnf.fake_quantize(to_cuda(xin))
    assert_bits_equal(y1, oracle.fake_quantize_uniform(xin), f"uniform {shape} {dtype}")


def test_config3_largest_properties():
    """32768x8192 fp32 (1 GiB): size-independent properties plus sampled rows against the oracle."""
    g = torch.Generator(device="cuda").manual_seed(5)
    sig = 10 ** (torch.rand(32768, 1, generator=g, device="cuda") * 5 - 4)
    x = torch.randn(32768, 8192, generator=g, device="cuda") * sig
    y = qu.fused_fake_quantize(x)
    # row-shard invariance: the result of a row range does not depend on the rest of the tensor
    for lo, hi in ((0, 4096), (12288, 16384), (32768 - 4096, 32768)):
        assert torch.equal(qu.fused_fake_quantize(x[lo:hi]), y[lo:hi])
    # signs preserved, |y| <= block scale, zeros stay zeros
    assert bool(((y == 0) | (torch.sign(y) == torch.sign(x))).all())
    # sampled rows, bit-exact against the oracle
    rows = torch.from_numpy(np.random.default_rng(1).choice(32768, 128, replace=False)).cuda()
    assert_bits_equal(y[rows], oracle.fused_fake_quantize(x[rows].cpu().numpy()), "sampled rows")
    del y
    # power-of-two scaling commutes with the quantiser on bf16-representable data
    xb = x[:8192].to(torch.bfloat16).float()
    a = qu.fused_fake_quantize(xb * 8.0)
    b = qu.fused_fake_quantize(xb) * 8.0
    assert torch.equal(a, b)


# ------------------------------------------------------------------ alignment / view handling
@pytest.mark.parametrize("B", [8, 16, 32])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_unaligned_and_strided_views(B, dtype):
    g = torch.Generator().manual_seed(B)
    base = torch.randn(37, 200, generator=g).to(dtype)
    bc = base.cuda()
    for view in (lambda t: t[:, 1:129], lambda t: t[:, 8:136], lambda t: t[3:, :64], lambda t: t[:, 3:36],
                 lambda t: t[::2, 16:144], lambda t: t.t()[:64, :32]):
        v = view(bc)
        want_in = to_bits(view(base).contiguous())
        if dtype == torch.float32:
            want_in = want_in.view(np.float32)
        y = qu.fused_fake_quantize(v, B)
        assert_bits_equal(y, oracle.fused_fake_quantize(want_in, B), "fq view")
        se, sg, mg = ops.pack(v, B, ops.GRID_NF5, "nearest", ops.LAYOUT_PLANES)
        ose, osg, omg = oracle.quantize(want_in, B, oracle.GRID_NF5)
        assert_bits_equal(se, ose, "se view"); assert_bits_equal(mg, omg, "mag view"); assert_bits_equal(sg, osg, "sign view")
        w = ops.pack(v, B, ops.GRID_NF5, "nearest", ops.LAYOUT_WIRE)
        assert_bits_equal(w, oracle.pack_bytes(ose, osg, omg, oracle.LAYOUT_WIRE), "wire view")
        s = ops.pack(v, B, ops.GRID_UNIFORM, "nearest", ops.LAYOUT_SPEC)
        use, usg, umg = oracle.quantize(want_in, B, oracle.GRID_UNIFORM)
        assert_bits_equal(s, oracle.pack_bytes(use, usg, umg, oracle.LAYOUT_SPEC), "spec view")


def test_unaligned_byte_buffers():
    """Byte records at an odd device address take the any-alignment kernels."""
    x = torch.randn(19, 96, generator=torch.Generator().manual_seed(3))
    xc = x.cuda()
    ose, osg, omg = oracle.quantize(x.numpy(), 32, oracle.GRID_NF5)
    want = oracle.pack_bytes(ose, osg, omg, oracle.LAYOUT_WIRE)
    lib = _lib.load()
    buf = torch.zeros(want.size + 64, dtype=torch.uint8, device="cuda")
    st = lib.axs6_pack(xc.data_ptr(), 0, 19, 96, 96, 32, 1, 0, 0, 0, 0, None, 1, buf.data_ptr() + 3, None, None,
                       torch.cuda.current_stream().cuda_stream)
    assert st == 0
    assert_bits_equal(buf[3:3 + want.size], want, "unaligned wire")
    assert int(buf[:3].sum()) == 0 and int(buf[3 + want.size:].sum()) == 0      # nothing written outside
    y = torch.empty(19, 96, device="cuda")
    st = lib.axs6_unpack(1, buf.data_ptr() + 3, None, None, y.data_ptr(), 0, 19, 96, 96, 32, 1,
                         torch.cuda.current_stream().cuda_stream)
    assert st == 0
    assert_bits_equal(y, oracle.dequantize(ose, osg, omg, 96, oracle.GRID_NF5), "unaligned unpack")


def test_canary_no_out_of_bounds_writes():
    """Outputs sit between guard regions that must stay untouched (ragged and aligned shapes)."""
    for rows, cols in ((7, 100), (64, 256), (3, 8), (1, 1), (513, 40)):
        for B in (8, 16, 32):
            x = torch.randn(rows, cols, device="cuda")
            n = rows * cols
            buf = torch.full((n + 512,), 7.0, device="cuda")
            y = buf[256:256 + n].view(rows, cols)
            st = _lib.load().axs6_fq(x.data_ptr(), y.data_ptr(), 0, 0, rows, cols, cols, cols, B, 1, 0, 0, 0, 0,
                                     torch.cuda.current_stream().cuda_stream)
            assert st == 0
            assert bool((buf[:256] == 7.0).all()) and bool((buf[256 + n:] == 7.0).all())
            assert_bits_equal(y, oracle.fused_fake_quantize(x.cpu().numpy(), B), "canary result")


def test_via_bf16_flag_equals_cast_then_quantise():
    w = torch.randn(256, 512, generator=torch.Generator().manual_seed(9)) * 0.02
    wc = w.cuda()
    a = ops.fake_quantize(wc, 32, ops.GRID_NF5, "nearest", out_dtype=torch.bfloat16, via_bf16=True)
    b = qu.fused_fake_quantize(wc.to(torch.bfloat16))
    assert a.dtype == torch.bfloat16 and torch.equal(a, b)
    assert_bits_equal(a, oracle.fused_fake_quantize(oracle.f32_to_bf16(w.numpy())), "via bf16 vs oracle")


# ------------------------------------------------------------------ stochastic rounding statistics (Philox)
def test_stochastic_statistics():
    """Same checks as the reference's GPU tests (tests/test_triton_kernels.py:205-241)."""
    torch.manual_seed(0)
    x = torch.randn(512, 512, device="cuda")
    near = qu.fused_fake_quantize(x, 32, "nearest")
    st1 = qu.fused_fake_quantize(x, 32, "stochastic")
    st2 = qu.fused_fake_quantize(x, 32, "stochastic")
    assert not torch.equal(st1, near) and not torch.equal(st1, st2)
    frac = float((st1 != near).float().mean())
    assert 0.002 < frac < 0.05
    mse_n = float(((near - x) ** 2).mean()); mse_s = float(((st1 - x) ** 2).mean())
    assert 0.5 < mse_s / mse_n < 2.0
    acc = torch.zeros_like(x)
    for _ in range(20):
        acc += qu.fused_fake_quantize(x, 32, "stochastic")
    assert abs(float((acc / 20 - x).mean())) < 0.01
    # every stochastic output is one of the two neighbouring levels of the nearest result's block grid
    assert bool((torch.sign(st1) * torch.sign(x) >= 0).all())


def test_stochastic_uniform_unbiased():
    """V1 stochastic rounding is unbiased (reference: tests/test_quantize.py:53-62)."""
    torch.manual_seed(1)
    x = torch.randn(64, 256, device="cuda")
    acc = torch.zeros_like(x)
    for _ in range(200):
        acc += core.dequantize(core.quantize(x, 32, "stochastic"))
    assert abs(float((acc / 200 - x).mean())) < 0.005


def test_stochastic_reproducible_under_seed():
    x = torch.randn(128, 256, device="cuda")
    torch.manual_seed(77); ops.reset_philox()
    a = qu.fused_fake_quantize(x, 32, "stochastic")
    torch.manual_seed(77); ops.reset_philox()
    b = qu.fused_fake_quantize(x, 32, "stochastic")
    assert torch.equal(a, b)


def test_vector_and_generic_kernels_draw_same_philox_stream():
    """The same (seed, offset) gives the same draws whichever kernel variant runs."""
    x = torch.randn(64, 96, device="cuda")
    lib = _lib.load()
    st = torch.cuda.current_stream().cuda_stream
    y1 = torch.empty_like(x)
    assert lib.axs6_fq(x.data_ptr(), y1.data_ptr(), 0, 0, 64, 96, 96, 96, 32, 1, 1, 0, 1234, 10, st) == 0
    big = torch.empty(64 * 96 + 1, device="cuda")
    xu = big[1:].view(64, 96); xu.copy_(x)                       # 4-byte aligned only -> generic kernel
    y2 = torch.empty_like(big)[1:].view(64, 96)
    assert lib.axs6_fq(xu.data_ptr(), y2.data_ptr(), 0, 0, 64, 96, 96, 96, 32, 1, 1, 0, 1234, 10, st) == 0
    assert torch.equal(y1, y2)


# ------------------------------------------------------------------ error conventions and edge sizes
def test_error_conventions():
    x = torch.randn(4, 32, device="cuda")
    with pytest.raises(AssertionError):
        qu.fused_fake_quantize(x, block_size=7)
    with pytest.raises(AssertionError):
        triton_fused_fake_quantize(x, block_size=64)
    with pytest.raises(RuntimeError, match="requires a CUDA tensor"):
        triton_fused_fake_quantize(torch.randn(4, 32))
    with pytest.raises(RuntimeError, match="requires a CUDA tensor"):
        qu.fused_fake_quantize(torch.randn(4, 32))
    with pytest.raises(ValueError):
        qu.fused_fake_quantize(x, 32, "banana")
    lib = _lib.load()
    st = torch.cuda.current_stream().cuda_stream
    assert lib.axs6_fq(None, x.data_ptr(), 0, 0, 4, 32, 32, 32, 32, 1, 0, 0, 0, 0, st) == -1
    assert lib.axs6_fq(x.data_ptr(), x.data_ptr(), 0, 0, 4, 32, 16, 32, 32, 1, 0, 0, 0, 0, st) == -1
    assert lib.axs6_fq(x.data_ptr(), x.data_ptr(), 5, 0, 4, 32, 32, 32, 32, 1, 0, 0, 0, 0, st) == -1
    assert lib.axs6_strerror(-1).decode().startswith("invalid argument")


def test_empty_and_tiny():
    e = torch.empty(0, 32, device="cuda")
    assert qu.fused_fake_quantize(e).shape == (0, 32)
    e2 = torch.empty(4, 0, device="cuda")
    assert qu.fused_fake_quantize(e2).shape == (4, 0)
    one = torch.tensor([0.3], device="cuda")
    assert_bits_equal(qu.fused_fake_quantize(one), oracle.fused_fake_quantize(np.array([0.3], dtype=np.float32)), "1 value")
    z = torch.zeros(5, 64, device="cuda")
    assert bool((qu.fused_fake_quantize(z) == 0).all())
    assert not bool(torch.signbit(qu.fused_fake_quantize(-z)).any())      # -0.0 -> +0.0


def test_4d_and_fp16_inputs():
    x = torch.randn(2, 3, 5, 48, generator=torch.Generator().manual_seed(4))
    y = qu.fused_fake_quantize(x.cuda(), 16)
    assert y.shape == x.shape
    assert_bits_equal(y, oracle.fused_fake_quantize(x.numpy(), 16), "4-D")


def test_gradient_hooks_on_one_gpu_rank():
    """The DDP hooks with the CUDA codec in a world of one NCCL rank: the result is this rank's own
    AXS-6 reconstruction, bit for bit what the oracle's pack -> unpack gives (incl. the non-zero
    reconstruction of exact zeros)."""
    import torch.distributed as dist
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", str(29400 + os.getpid() % 500))
    dist.init_process_group("nccl", rank=0, world_size=1, device_id=torch.device("cuda", 0))
    try:
        class Bucket:
            def __init__(self, t): self.t = t
            def buffer(self): return self.t
        rng = np.random.default_rng(4)
        g = rng.standard_normal(100003, dtype=np.float32) * 1e-3
        g[::97] = 0.0
        se, sg, mg = oracle.quantize(g.reshape(1, -1), 32, oracle.GRID_NF5)
        want = oracle.dequantize(se, sg, mg, g.size, oracle.GRID_NF5).reshape(-1)
        for hook in (udist.axs6_gradient_hook, udist.axs6_gradient_hook_packed):
            out = hook(None, Bucket(torch.from_numpy(g).cuda())).wait()
            assert out.shape == (g.size,) and out.dtype == torch.float32
            assert_bits_equal(out, want, hook.__name__)
        c = udist.AXS6GradCompressor(packed=True)
        out = c.compress_and_allreduce(torch.from_numpy(g[:7000]).cuda().reshape(1000, 7))
        assert out.shape == (1000, 7)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("B", [8, 16, 32])
def test_planes_to_records_and_back(B):
    """The reference-named helpers for data already held as planes."""
    x = torch.randn(21, 96, generator=torch.Generator().manual_seed(B))
    se, sg, mg, shape = udist._pack_gradient(x.cuda(), B)
    buf = udist._pack_to_flat_buffer(se, sg, mg)
    ose, osg, omg = oracle.quantize(x.numpy(), B, oracle.GRID_NF5)
    assert buf.dtype == torch.int8
    assert_bits_equal(buf.view(torch.uint8), oracle.pack_bytes(ose, osg, omg, oracle.LAYOUT_WIRE), "records from planes")
    se2, sg2, mg2 = udist._unpack_from_flat_buffer(buf, 21, 96 // B, B)
    assert torch.equal(se2, se) and torch.equal(sg2, sg) and torch.equal(mg2, mg) and sg2.dtype == torch.bool
    back = udist._unpack_gradient(se2, sg2, mg2, shape, B)
    assert_bits_equal(back, oracle.dequantize(ose, osg, omg, 96, oracle.GRID_NF5), "values from planes")


def test_philox_epoch_changes_draws_and_reset_restores_them():
    """`axs6_philox_advance` moves a device-resident addend of the Philox counter: the same host-side
    (seed, offset) then gives other draws (what a replayed CUDA graph needs); reset brings them back."""
    x = torch.randn(256, 512, device="cuda")
    lib = _lib.load()
    st = torch.cuda.current_stream().cuda_stream

    def run():
        y = torch.empty_like(x)
        assert lib.axs6_fq(x.data_ptr(), y.data_ptr(), 0, 0, 256, 512, 512, 512, 32, 1, 1, 0, 99, 5, st) == 0
        return y

    try:
        a = run()
        ops.philox_advance(1 << 40)
        b = run()
        ops.philox_advance(0, reset=True)
        c = run()
    finally:
        ops.philox_advance(0, reset=True)
    assert torch.equal(a, c) and not torch.equal(a, b)


def test_philox_epoch_can_be_read_and_restored():
    """What a checkpoint does: read the device-resident epoch, later put it back; the draws continue where they were."""
    x = torch.randn(64, 256, device="cuda")
    lib = _lib.load()
    st = torch.cuda.current_stream().cuda_stream

    def run():
        y = torch.empty_like(x)
        assert lib.axs6_fq(x.data_ptr(), y.data_ptr(), 0, 0, 64, 256, 256, 256, 32, 1, 1, 0, 7, 0, st) == 0
        return y

    try:
        assert ops.philox_epoch() == 0
        ops.philox_advance(12345)
        ops.philox_advance(1 << 40)
        saved = ops.philox_epoch()
        assert saved == 12345 + (1 << 40)
        want = run()
        ops.philox_advance(0, reset=True)
        assert ops.philox_epoch() == 0
        ops.set_philox_epoch(saved)
        assert ops.philox_epoch() == saved
        assert torch.equal(run(), want)
    finally:
        ops.philox_advance(0, reset=True)


@pytest.mark.parametrize("layout", [ops.LAYOUT_WIRE, ops.LAYOUT_SPEC])
@pytest.mark.parametrize("dtype", ["bf16", "f32"])
@pytest.mark.parametrize("shape", [(1, 32), (255, 32), (257, 32), (3, 96), (777, 1056), (2048, 4096)])
def test_record_pack_kernels_agree_with_the_oracle(shape, dtype, layout):
    """NF5, nearest, block 32, byte records: the TMA-fed kernels (default; one for bf16 and one for fp32
    input), the bf16 kernel with per-thread loads (tune key 2 = 2) and the general kernel (tune key
    2 = 1) all give the oracle's bytes, for whole and ragged groups of 256 blocks and for blocks that
    leave the fast paths (all-zero, negative zeros, denormal-range and near-overflow maxima, maxima at
    the top of a binade where the block exponent is bumped)."""
    from axs6_b200 import _lib
    lib = _lib.load()
    g = torch.Generator().manual_seed(shape[0] * 131 + shape[1] + layout)
    x = torch.randn(*shape, generator=g)
    x[torch.rand(*shape, generator=g) < 0.02] = 0.0
    x[torch.rand(*shape, generator=g) < 0.01] = -0.0
    x[torch.rand(*shape, generator=g) < 0.002] *= 1e-30
    if shape[0] > 2:
        x[1] *= 1e-38
        x[2] *= 3e37
        x[0, :32] = 0.0
    x.view(-1)[::97] = float.fromhex("0x1.fffffep+3")
    xb = oracle.f32_to_bf16(x.numpy()) if dtype == "bf16" else x.numpy()
    se, sg, mg = oracle.quantize(xb, 32, oracle.GRID_NF5)
    want = oracle.pack_bytes(se, sg, mg, layout)
    xt = to_cuda(xb)
    try:
        for mode in (0, 2, 1):
            lib.axs6_tune(2, mode)
            got = ops.pack(xt, 32, ops.GRID_NF5, "nearest", layout)
            torch.cuda.synchronize()
            assert_bits_equal(got, want, f"tune(2)={mode} {shape} layout {layout}")
    finally:
        lib.axs6_tune(2, 0)
    assert lib.axs6_codec_status() == 0


@pytest.mark.parametrize("layout", [ops.LAYOUT_WIRE, ops.LAYOUT_SPEC])
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rows,cols", [(1, 32), (255, 32), (257, 32), (3, 96), (777, 1056), (1024, 4096)])
def test_record_unpack_kernels_agree_with_the_oracle(rows, cols, out_dtype, layout):
    """Byte records -> values (NF5, block 32): the TMA-fed kernel (default) and the general kernel
    (tune key 11 = 1) both reproduce the oracle bit for bit on RANDOM records, i.e. for every code and
    every exponent byte, including the blocks outside the integer fast path (se < 8 and se = 255)."""
    lib = _lib.load()
    rng = np.random.default_rng(rows * 7 + cols + layout)
    nblk = cols // 32
    rec = 24 + (2 if layout == ops.LAYOUT_SPEC else 1)
    raw = rng.integers(0, 256, size=(rows * nblk, rec), dtype=np.uint8)
    if layout == ops.LAYOUT_SPEC:
        raw[:, 0] &= 0xFC                                  # config bits 0 = dense block
    raw[rng.random(rows * nblk) < 0.05] = 0                # all-zero records
    if layout == ops.LAYOUT_WIRE:
        raw[rng.random(rows * nblk) < 0.05, 0] = rng.integers(0, 8)    # tiny exponents
    se, sg, mg = oracle.unpack_bytes(raw.reshape(-1), rows, nblk, 32, layout)
    want = oracle.dequantize(se, sg, mg, cols, oracle.GRID_NF5)
    finite = np.isfinite(want)                            # se = 255 decodes to inf: out of contract
    if out_dtype == torch.bfloat16:
        want = oracle.f32_to_bf16(want)
    buf = torch.from_numpy(raw.reshape(-1).copy()).cuda()
    try:
        for mode in (0, 1):
            lib.axs6_tune(11, mode)
            got = ops.unpack(layout, buf, rows, cols, 32, ops.GRID_NF5, out_dtype)
            torch.cuda.synchronize()
            g = to_bits(got).reshape(-1)[finite.reshape(-1)]
            w = (want.view(np.uint32) if want.dtype == np.float32 else want).reshape(-1)[finite.reshape(-1)]
            assert np.array_equal(g, w), f"tune(11)={mode}: {(g != w).sum()} of {g.size} differ"
    finally:
        lib.axs6_tune(11, 0)
    assert lib.axs6_codec_status() == 0


@pytest.mark.parametrize("layout", [ops.LAYOUT_WIRE, ops.LAYOUT_SPEC])
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nsrc,rows,cols", [(1, 255, 32), (2, 257, 32), (3, 1, 32), (3, 777, 1056), (8, 512, 4096), (5, 100, 96)])
def test_fused_unpack_and_average_matches_the_oracle(nsrc, rows, cols, out_dtype, layout):
    """axs6_unpack_sum (the receiving side of the packed gradient exchange) on RANDOM records of nsrc
    sources: bit-identical to summing the oracle's reconstructions in fp32 in source order and dividing by
    nsrc, for the producer/consumer TMA kernel (default) and the one-thread-per-value kernel (tune key 11)."""
    lib = _lib.load()
    rng = np.random.default_rng(nsrc * 1000 + rows + cols + layout)
    nblk = cols // 32
    rec = 24 + (2 if layout == ops.LAYOUT_SPEC else 1)
    per = rows * nblk * rec
    stride = (per + 15) // 16 * 16 + 16 * (nsrc % 2)          # padded, and not always the minimum
    raw = np.zeros(nsrc * stride, dtype=np.uint8)
    acc = None
    for s in range(nsrc):
        r = rng.integers(0, 256, size=(rows * nblk, rec), dtype=np.uint8)
        se_in = rng.integers(0, 250, size=rows * nblk).astype(np.uint32)      # sums of up to 8 sources stay finite
        se_in[rng.random(rows * nblk) < 0.05] = rng.integers(0, 8)           # blocks outside the integer fast path
        if layout == ops.LAYOUT_SPEC:
            r[:, 0] = (se_in << 2) & 0xFF
            r[:, 1] = se_in >> 6
        else:
            r[:, 0] = se_in
        r[rng.random(rows * nblk) < 0.05] = 0
        raw[s * stride:s * stride + per] = r.reshape(-1)
        se, sg, mg = oracle.unpack_bytes(r.reshape(-1), rows, nblk, 32, layout)
        part = oracle.dequantize(se, sg, mg, cols, oracle.GRID_NF5)
        acc = part if acc is None else (acc + part).astype(np.float32)
    assert np.isfinite(acc).all()
    want = (acc / np.float32(nsrc)).astype(np.float32)
    if out_dtype == torch.bfloat16:
        want = oracle.f32_to_bf16(want)
    buf = torch.from_numpy(raw).cuda()
    try:
        for mode in (0, 1):
            lib.axs6_tune(11, mode)
            got = ops.unpack_sum(layout, buf, nsrc, stride, rows, cols, 32, ops.GRID_NF5, out_dtype, float(nsrc))
            torch.cuda.synchronize()
            assert_bits_equal(got, want, f"tune(11)={mode} nsrc={nsrc} {rows}x{cols}")
    finally:
        lib.axs6_tune(11, 0)
    assert lib.axs6_codec_status() == 0


@pytest.mark.parametrize("shape", [(1, 32), (255, 32), (257, 32), (513, 32), (3, 96), (777, 1056), (2048, 4096)])
def test_bf16_fake_quantise_kernels_agree_with_the_oracle(shape):
    """bf16 -> bf16, NF5, nearest, block 32: the TMA-fed in-place kernel (default) and the general kernel
    (tune key 12 = 1) both give the oracle's bits, including +-0 values, all-zero blocks and blocks whose
    maximum lies in the denormal range or next to overflow."""
    lib = _lib.load()
    g = torch.Generator().manual_seed(shape[0] * 17 + shape[1])
    x = torch.randn(*shape, generator=g)
    x[torch.rand(*shape, generator=g) < 0.02] = 0.0
    x[torch.rand(*shape, generator=g) < 0.02] = -0.0
    x[torch.rand(*shape, generator=g) < 0.002] *= 1e-30
    if shape[0] > 2:
        x[1] *= 1e-38
        x[2] *= 3e37
        x[0, :32] = 0.0
    xb = oracle.f32_to_bf16(x.numpy())
    want = oracle.fused_fake_quantize(xb, 32)
    xt = to_cuda(xb)
    try:
        for mode in (0, 1):
            lib.axs6_tune(12, mode)
            got = qu.fused_fake_quantize(xt, 32)
            torch.cuda.synchronize()
            assert got.dtype == torch.bfloat16
            assert_bits_equal(got, want, f"tune(12)={mode} {shape}")
    finally:
        lib.axs6_tune(12, 0)
    assert lib.axs6_codec_status() == 0


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_host_buffer_fake_quantise_is_the_device_result(dtype):
    """fused_fake_quantize_host: pinned host tensors through a ring of device buffers (more chunks than ring
    slots, a ragged last chunk, a second call that reuses the ring) gives the bits of the device operator."""
    g = torch.Generator().manual_seed(5)
    x = (torch.randn(1000, 416, generator=g) * torch.logspace(-3, 1, 1000).unsqueeze(1)).to(dtype)
    hx = x.pin_memory()
    want = qu.fused_fake_quantize(x.cuda(), 32).cpu()
    got = ops.fake_quantize_host(hx, None, 32, chunk_bytes=64 * 416 * x.element_size(), depth=3)     # 16 chunks, last one short
    torch.cuda.synchronize()
    assert got.is_pinned() and got.dtype == dtype and got.shape == x.shape
    assert torch.equal(got.view(torch.int32 if dtype == torch.float32 else torch.int16),
                       want.view(torch.int32 if dtype == torch.float32 else torch.int16))
    hy = torch.empty_like(hx).pin_memory()
    out = qu.fused_fake_quantize_host(hx.view(10, 100, 416), hy.view(10, 100, 416), 32)
    torch.cuda.current_stream().synchronize()
    assert out.data_ptr() == hy.data_ptr() and torch.equal(hy.view(-1).view(torch.uint8), want.reshape(-1).view(torch.uint8))
    with pytest.raises(ValueError):
        ops.fake_quantize_host(x)                       # not pinned
    with pytest.raises(TypeError):
        ops.fake_quantize_host(x.cuda())


def test_bf16_integer_paths_on_every_exponent_and_mantissa():
    """The TMA-fed bf16 kernels replace the fp32 formulas by integer arithmetic on the bit patterns.  Sweep:
    block maxima with every exponent field 1..253 (maxima of 2^127 and above make the scale overflow: outside the
    contract) and four mantissas; under each maximum, values with every
    mantissa at 14 exponent distances, both signs, plus +-0 and bf16 denormals.  Fake-quantise output and packed
    records must equal the oracle's bit for bit."""
    mant = np.arange(128, dtype=np.uint32)
    blocks = []
    for E in range(1, 254):
        for ma in (0, 1, 63, 127):
            amax = (E << 7) | ma
            vals = [np.array([0x0000, 0x8000, 0x0001, 0x8001, 0x007F, 0x807F], dtype=np.uint32)]
            for j in range(14):
                e = E - j
                if e < 1:
                    break
                v = (e << 7) | mant
                v = v[v <= amax]
                vals.append(v)
                vals.append(v | 0x8000)
            v = np.concatenate(vals)
            pad = (-len(v)) % 31
            v = np.concatenate([v, np.zeros(pad, dtype=np.uint32)]).reshape(-1, 31)
            sign = 0x8000 if (E + ma) % 2 else 0
            blk = np.concatenate([np.full((v.shape[0], 1), amax | sign, dtype=np.uint32), v], axis=1)
            blocks.append(blk)
    x = np.concatenate(blocks).astype(np.uint16)                          # (nblocks, 32)
    assert x.shape[0] > 100000
    xt = to_cuda(x)
    fq = qu.fused_fake_quantize(xt, 32)
    assert_bits_equal(fq, oracle.fused_fake_quantize(x, 32), "fake-quantise bf16, all exponents")
    se, sg, mg = oracle.quantize(x, 32, oracle.GRID_NF5)
    for layout in (ops.LAYOUT_WIRE, ops.LAYOUT_SPEC):
        rec = ops.pack(xt, 32, ops.GRID_NF5, "nearest", layout)
        assert_bits_equal(rec, oracle.pack_bytes(se, sg, mg, layout), f"pack bf16 layout {layout}, all exponents")
        back = ops.unpack(layout, rec, x.shape[0], 32, 32, ops.GRID_NF5, torch.bfloat16)
        assert_bits_equal(back, oracle.f32_to_bf16(oracle.dequantize(se, sg, mg, 32, oracle.GRID_NF5)), "unpack to bf16")
    assert _lib.load().axs6_codec_status() == 0


@pytest.mark.parametrize("shape", [(255, 32), (257, 32), (3, 96), (777, 1056), (2048, 4096)])
def test_stochastic_bf16_kernels_give_the_same_bits(shape):
    """Stochastic rounding with the library's draws, bf16 -> bf16: the TMA-fed kernel (default) forms the
    dithered index and the value exactly as the general kernel (tune key 12 = 1) does, so for one seed and
    offset both give the same bits -- including +-0 values, all-zero blocks and blocks outside the fast range."""
    lib = _lib.load()
    g = torch.Generator().manual_seed(shape[0] + shape[1])
    x = torch.randn(*shape, generator=g)
    x[torch.rand(*shape, generator=g) < 0.02] = 0.0
    x[torch.rand(*shape, generator=g) < 0.02] = -0.0
    if shape[0] > 2:
        x[1] *= 1e-38
        x[2] *= 3e37
        x[0, :32] = 0.0
    xt = x.to(torch.bfloat16).cuda()
    outs = []
    try:
        for mode in (0, 1):
            lib.axs6_tune(12, mode)
            torch.manual_seed(5)
            ops.reset_philox(1000)
            outs.append(qu.fused_fake_quantize(xt, 32, "stochastic"))
    finally:
        lib.axs6_tune(12, 0)
    torch.cuda.synchronize()
    assert torch.equal(outs[0].view(torch.int16), outs[1].view(torch.int16))
    nearest = qu.fused_fake_quantize(xt, 32)
    frac = float((outs[0] != nearest).float().mean())
    assert 0.0 < frac < 0.05                              # the dither moves about 1 % of the values
    assert lib.axs6_codec_status() == 0
