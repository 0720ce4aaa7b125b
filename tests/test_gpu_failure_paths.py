"""The give-up path of a bounded device-side wait, exercised without faulting or hanging anything.

`axs6_unpack_sum`'s fast kernel has a producer warp that streams records into shared memory and consumer
warps that wait for them on mbarriers.  Every such wait polls a bounded number of times.  Tune key 14 makes
the producer issue NOTHING (no asynchronous copy is ever in flight) and tune key 13 shortens the poll limit, so
the consumers' first wait runs out: the kernel must return by itself, report status 11 through
`axs6_codec_status()`, leave the output and its guard regions untouched, and the next ordinary call must be
correct.  No trap, no bad address, no endless loop is involved.
"""
import pytest
import torch

pytestmark = pytest.mark.gpu

from axs6_b200 import _lib, ops  # noqa: E402


def test_consumer_wait_runs_out_and_the_library_stays_usable():
    lib = _lib.load()
    rows, cols, nsrc = 512, 1024, 3
    g = torch.Generator(device="cuda").manual_seed(1)
    srcs = [torch.randn(rows, cols, generator=g, device="cuda") for _ in range(nsrc)]
    recs = [ops.pack(s, 32, ops.GRID_NF5, "nearest", ops.LAYOUT_WIRE) for s in srcs]
    per = recs[0].numel()
    stride = (per + 15) // 16 * 16
    buf = torch.zeros(nsrc * stride, dtype=torch.uint8, device="cuda")
    for i, r in enumerate(recs):
        buf[i * stride:i * stride + per] = r
    want = ops.unpack_sum(ops.LAYOUT_WIRE, buf, nsrc, stride, rows, cols, divisor=float(nsrc))
    assert lib.axs6_codec_status() == 0

    guard = 4096
    canvas = torch.full((rows * cols + 2 * guard,), 7.25, device="cuda")
    out = canvas[guard:guard + rows * cols]
    try:
        lib.axs6_tune(13, 2048)          # poll limit of the kernel's waits
        lib.axs6_tune(14, 1)             # the producer issues no load: nothing asynchronous is in flight
        ops.unpack_sum(ops.LAYOUT_WIRE, buf, nsrc, stride, rows, cols, divisor=float(nsrc), out=out)
        torch.cuda.synchronize()         # the kernel came back by itself
        assert lib.axs6_codec_status() == 11, "the consumers' give-up code was not reported"
        assert lib.axs6_codec_status() == 0, "reading the status clears it"
    finally:
        lib.axs6_tune(13, 0)
        lib.axs6_tune(14, 0)
    assert bool((canvas == 7.25).all()), "a kernel that gave up wrote output or touched the guard regions"
    # the context and the library are intact: the same call now gives the right answer
    ops.unpack_sum(ops.LAYOUT_WIRE, buf, nsrc, stride, rows, cols, divisor=float(nsrc), out=out)
    torch.cuda.synchronize()
    assert lib.axs6_codec_status() == 0
    assert torch.equal(out.view(rows, cols), want)
    assert bool((canvas[:guard] == 7.25).all()) and bool((canvas[guard + rows * cols:] == 7.25).all())
