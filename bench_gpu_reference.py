"""Same-GPU comparator: the UNMODIFIED reference, run on the device the library is measured on.

The copy under ``baseline/_ref`` (put there by baseline/install_reference.py) is imported as it is and
its own CUDA code paths are timed with CUDA events on the benchmark's tensors:

* ``fused_fake_quantize`` (axs/unified/quantize_unified.py:121-204): eager torch ops on the device,
* ``triton_fused_fake_quantize`` (axs/unified/triton_kernels.py:295-382): the reference's Triton kernel, when
  Triton can compile for this GPU,
* ``AXSLinearMixedPrecision`` (axs/unified/mixed_precision.py:193-275) forward + backward at the Linear
  benchmark's size: the reference's fake-quantise passes around ``F.linear`` (cuBLAS),
* ``axs_linear_unified`` (axs/unified/functional_unified.py:173-201), the fp32 graph of the same layer.

Each result is also compared with this library's output on the same input (bit for bit for nearest rounding),
which is a full-size parity check against the reference itself.  Nothing of this library runs inside the
timed regions of this module; a failure of any arm is reported in its entry and never stops the benchmark.
"""
from __future__ import annotations

import importlib
import os
import sys

ROOT = os.path.dirname(os.path.abspath(__file__))
REF_DIR = os.path.join(ROOT, "baseline", "_ref")


def _time(torch, fn, warm: int, steps: int) -> float:
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / steps


def run(dev, x, ours_ms: float, linear_ms: float | None = None) -> dict:
    """x: the headline fp32 tensor on `dev`; ours_ms: this library's time for one pass over it."""
    import torch
    if not os.path.isdir(os.path.join(REF_DIR, "axs")):
        return {"unavailable": "no copy of the reference under baseline/_ref (run baseline/install_reference.py)"}
    if REF_DIR not in sys.path:
        sys.path.insert(0, REF_DIR)
    ours_qu = importlib.import_module("axs6_b200.unified.quantize_unified")
    out: dict = {"source": "unmodified reference package under baseline/_ref, its own CUDA code paths, same GPU, same "
                           "tensors, CUDA events; this library's figures beside them"}
    nbytes = x.numel() * 8
    mine = ours_qu.fused_fake_quantize(x)

    def entry(ms: float, y) -> dict:
        same = bool(torch.equal(y.view(torch.int32), mine.view(torch.int32)))
        return {"ms": ms, "GBps": nbytes / (ms * 1e-3) / 1e9, "this_library_ms": ours_ms, "speedup": ms / ours_ms,
                "bit_identical_to_this_library": same}

    try:
        ref_fq = importlib.import_module("axs.unified.quantize_unified").fused_fake_quantize
        with torch.no_grad():
            y = ref_fq(x, 32, "nearest")
            ms = _time(torch, lambda: ref_fq(x, 32, "nearest"), 2, 5)
        out["fused_fake_quantize_eager"] = entry(ms, y)
        del y
    except Exception as e:
        out["fused_fake_quantize_eager"] = {"error": repr(e)[:300]}
    torch.cuda.empty_cache()
    try:
        tk = importlib.import_module("axs.unified.triton_kernels")
        if not tk.has_triton():
            out["fused_fake_quantize_triton"] = {"unavailable": "the reference reports has_triton() == False"}
        else:
            with torch.no_grad():
                y = tk.triton_fused_fake_quantize(x, 32, "nearest")
                ms = _time(torch, lambda: tk.triton_fused_fake_quantize(x, 32, "nearest"), 3, 10)
            out["fused_fake_quantize_triton"] = entry(ms, y)
            del y
    except Exception as e:
        out["fused_fake_quantize_triton"] = {"error": repr(e)[:300]}
    del mine
    torch.cuda.empty_cache()
    try:
        mp = importlib.import_module("axs.unified.mixed_precision")
        M, K, N = 16384, 4096, 4096
        torch.manual_seed(11)
        layer = mp.AXSLinearMixedPrecision(K, N, bias=True).to(dev)
        g = torch.Generator(device=dev).manual_seed(12)
        xin = torch.randn(M, K, generator=g, device=dev).to(torch.bfloat16).requires_grad_(True)
        go = torch.randn(M, N, generator=g, device=dev).to(torch.bfloat16)

        def step():
            layer.zero_grad(set_to_none=True)
            xin.grad = None
            layer(xin).backward(go)

        ms = _time(torch, step, 3, 10)
        ent = {"ms_per_step": ms, "TFLOPs": 6.0 * M * N * K / (ms * 1e-3) / 1e12,
               "workload": f"AXSLinearMixedPrecision forward + backward, M={M}, K={K}, N={N}, bf16 activations"}
        if linear_ms:
            ent["this_library_ms_per_step"] = linear_ms
            ent["speedup"] = ms / linear_ms
        out["linear_step"] = ent
        del layer, xin, go
    except Exception as e:
        out["linear_step"] = {"error": repr(e)[:300]}
    torch.cuda.empty_cache()
    try:
        fu = importlib.import_module("axs.unified.functional_unified")
        M, K, N = 16384, 4096, 4096
        g = torch.Generator(device=dev).manual_seed(13)
        xin = torch.randn(M, K, generator=g, device=dev).requires_grad_(True)
        w = (torch.randn(N, K, generator=g, device=dev) * 0.02).requires_grad_(True)
        b = torch.zeros(N, device=dev, requires_grad=True)
        go = torch.randn(M, N, generator=g, device=dev)

        def step32():
            xin.grad = w.grad = b.grad = None
            fu.axs_linear_unified(xin, w, b).backward(go)

        ms = _time(torch, step32, 2, 5)
        out["linear_step_fp32_graph"] = {
            "ms_per_step": ms, "TFLOPs": 6.0 * M * N * K / (ms * 1e-3) / 1e12,
            "workload": f"axs_linear_unified forward + backward, M={M}, K={K}, N={N}, fp32 tensors (compare linear.fp32_graph)"}
        del xin, w, b, go
    except Exception as e:
        out["linear_step_fp32_graph"] = {"error": repr(e)[:300]}
    torch.cuda.empty_cache()
    return out
