"""The bias-gradient entry point that allocates nothing (`axs6_bias_grad_static`).

Some hosts of this library cannot give a kernel scratch memory: a plugin that only ever receives
input and output pointers, or a server that has already handed every free byte of HBM to its own
pool.  For them the column-sum kernel keeps its partial sums in a fixed array inside the library.
This test calls that entry point through the C ABI twice in a row -- the second time with a
different, wider tensor, so that stale partial sums from the first call would show -- and
requires the same fp32 result, bit for bit, as the ordinary entry point that takes a
caller-owned scratch buffer.  The file sorts last so that a run stopping at the first failure
has already executed every other test.
"""
import pytest
import torch

pytestmark = pytest.mark.gpu

from axs6_b200 import _lib  # noqa: E402


def _both(lib, g: torch.Tensor):
    rows, cols = g.shape
    code = 0 if g.dtype == torch.float32 else 1
    st = torch.cuda.current_stream().cuda_stream
    want = torch.empty(cols, device="cuda")
    part = torch.empty(int(lib.axs6_linear_workspace_bytes(3, 0, cols, 0)), dtype=torch.uint8, device="cuda")
    assert lib.axs6_bias_grad(g.data_ptr(), code, cols, rows, cols, want.data_ptr(), part.data_ptr(), st) == 0
    got = torch.full((cols,), float("nan"), device="cuda")
    assert lib.axs6_bias_grad_static(g.data_ptr(), code, cols, rows, cols, got.data_ptr(), st) == 0
    torch.cuda.synchronize()
    return got, want


def test_static_scratch_matches_caller_scratch_on_two_calls_in_a_row():
    lib = _lib.load()
    gen = torch.Generator(device="cuda").manual_seed(11)
    first = torch.randn(4096, 1000, generator=gen, device="cuda") * 3.0
    second = torch.randn(777, 4096, generator=gen, device="cuda").to(torch.bfloat16)
    for g in (first, second):
        got, want = _both(lib, g)
        assert torch.equal(got, want)
        ref = g.double().sum(0)
        assert float((got.double() - ref).abs().max()) <= 1e-5 * (g.shape[0] ** 0.5) * max(1.0, float(ref.abs().max()))


def test_static_scratch_rejects_oversize_and_bad_arguments():
    lib = _lib.load()
    st = torch.cuda.current_stream().cuda_stream
    g = torch.zeros(2, 16392, device="cuda")
    out = torch.zeros(16392, device="cuda")
    rc = lib.axs6_bias_grad_static(g.data_ptr(), 0, 16392, 2, 16392, out.data_ptr(), st)
    assert rc == -7
    assert b"fixed capacity" in lib.axs6_strerror(rc)
    assert lib.axs6_bias_grad_static(None, 0, 8, 2, 8, out.data_ptr(), st) == -1
    assert lib.axs6_bias_grad_static(g.data_ptr(), 0, 16384, 2, 16384, out.data_ptr(), st) == 0   # the maximum itself
    torch.cuda.synchronize()
