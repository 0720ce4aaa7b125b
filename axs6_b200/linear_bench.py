"""Timing of the AXS-6 Linear forward + backward (bf16 activations (M, K), fp32 master weights
(N, K), block 32 along K) for ``bench.py``: M = 16384 rows per GPU, K = N = 4096.

One step = `axs6_linear_fwd` + `axs6_linear_bwd` (four fake-quantise passes, three tcgen05
GEMMs, the bias-gradient column sums) through the C ABI with caller-owned buffers.  With more
than one rank the batch is sharded (every rank owns M rows) and the fp32 weight gradient is
all-reduced over NCCL on a side stream, overlapped with the next step.
"""
from __future__ import annotations

import torch

from . import _lib

M_PER_GPU, K, N, BLOCK = 16384, 4096, 4096, 32


def run(args, rank: int, world: int, dev, pk: dict, steps: int | None = None) -> dict:
    import torch.distributed as dist
    lib = _lib.load()
    steps = steps or max(5, min(args.steps, 20))
    M = M_PER_GPU
    g = torch.Generator(device=dev).manual_seed(4000 + rank)
    x = torch.randn(M, K, generator=g, device=dev).to(torch.bfloat16)
    w = torch.randn(N, K, generator=g, device=dev) * 0.02
    bias = torch.zeros(N, device=dev)
    go = torch.randn(M, N, generator=g, device=dev).to(torch.bfloat16)
    y = torch.empty(M, N, dtype=torch.bfloat16, device=dev)
    dx = torch.empty(M, K, dtype=torch.bfloat16, device=dev)
    dws = [torch.empty(N, K, dtype=torch.float32, device=dev) for _ in range(2)]
    db = torch.empty(N, dtype=torch.float32, device=dev)
    ws = [torch.empty(int(lib.axs6_linear_workspace_bytes(i, M, N, K)), dtype=torch.uint8, device=dev) for i in range(4)]
    xq, wq, gq, part = ws
    stream = torch.cuda.current_stream().cuda_stream

    def fwd():
        st = lib.axs6_linear_fwd(x.data_ptr(), 1, K, w.data_ptr(), 0, K, bias.data_ptr(), y.data_ptr(), 1, N, M, N, K,
                                 BLOCK, 1, 1, xq.data_ptr(), wq.data_ptr(), stream)
        assert st == 0, st

    def bwd(i):
        st = lib.axs6_linear_bwd(go.data_ptr(), 1, N, xq.data_ptr(), w.data_ptr(), 0, K, dx.data_ptr(), 1, K,
                                 dws[i % 2].data_ptr(), K, db.data_ptr(), M, N, K, BLOCK, 1, 2, 1234, i * (M * N // 8),
                                 None, gq.data_ptr(), wq.data_ptr(), part.data_ptr(), None, stream)
        assert st == 0, st

    pending = [None, None]

    def step(i):
        fwd()
        if pending[i % 2] is not None:
            pending[i % 2].wait()
            pending[i % 2] = None
        bwd(i)
        if world > 1:
            pending[i % 2] = dist.all_reduce(dws[i % 2], async_op=True)

    def drain():
        for j in range(2):
            if pending[j] is not None:
                pending[j].wait()
                pending[j] = None

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for i in range(3):
        step(i)
    drain()
    barrier()
    l0 = _lib.launches()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(steps):
        step(i)
    drain()
    e1.record()
    barrier()
    ms = e0.elapsed_time(e1)
    launches = _lib.launches() - l0
    t = torch.tensor([ms], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_step = float(t.item()) / steps
    flops = 6.0 * M * N * K
    tflops = world * flops / (ms_step * 1e-3) / 1e12
    status = int(lib.axs6_gemm_status())

    # the three GEMMs alone (operands already quantised), for the tensor-pipe roofline
    parts = {}
    if rank == 0:
        def t_of(fn, n=10):
            for _ in range(2):
                fn()
            torch.cuda.synchronize()
            e0.record()
            for _ in range(n):
                fn()
            e1.record()
            torch.cuda.synchronize()
            return e0.elapsed_time(e1) / n
        gf = lambda: lib.axs6_gemm_bf16(xq.data_ptr(), wq.data_ptr(), y.data_ptr(), None, M, N, K, K, K, N, 0, 0, 1, stream)
        gdx = lambda: lib.axs6_gemm_bf16(gq.data_ptr(), wq.data_ptr(), dx.data_ptr(), None, M, K, N, N, K, K, 0, 1, 1, stream)
        gdw = lambda: lib.axs6_gemm_bf16(gq.data_ptr(), xq.data_ptr(), dws[0].data_ptr(), None, N, K, M, N, K, K, 1, 1, 0, stream)
        fqx = lambda: lib.axs6_fq(x.data_ptr(), xq.data_ptr(), 1, 1, M, K, K, K, BLOCK, 1, 0, 1, 0, 0, stream)
        fqw = lambda: lib.axs6_fq(w.data_ptr(), wq.data_ptr(), 0, 1, N, K, K, K, BLOCK, 1, 0, 1, 0, 0, stream)
        fqg = lambda: lib.axs6_fq(go.data_ptr(), gq.data_ptr(), 1, 1, M, N, N, N, BLOCK, 1, 1, 1, 7, 0, stream)
        for name, fn, fl in (("gemm_fwd", gf, 2.0 * M * N * K), ("gemm_dx", gdx, 2.0 * M * N * K), ("gemm_dw", gdw, 2.0 * M * N * K)):
            m = t_of(fn)
            parts[name] = {"ms": m, "TFLOPs": fl / (m * 1e-3) / 1e12}
        for name, fn, nb in (("fq_x", fqx, M * K * 4), ("fq_w", fqw, N * K * 6), ("fq_g_stochastic", fqg, M * N * 4)):
            m = t_of(fn)
            parts[name] = {"ms": m, "GBps": nb / (m * 1e-3) / 1e9}
    best = max((v["TFLOPs"] for k, v in parts.items() if k.startswith("gemm")), default=0.0)
    return {
        "metric": "axs6_linear_fwd_bwd_TFLOPs", "value": tflops, "unit": "TFLOP/s", "ms_per_step": ms_step,
        "steps": steps, "n_gpus": world, "gpu_launches": launches, "gemm_status": status,
        "workload": f"AXS-6 Linear fwd+bwd, M={M} rows per GPU, K={K}, N={N}, bf16 activations, fp32 master weights, "
                    f"block {BLOCK} along K, stochastic gradient rounding, dW all-reduced over NCCL" if world > 1 else
                    f"AXS-6 Linear fwd+bwd, M={M}, K={K}, N={N}, bf16 activations, fp32 master weights, block {BLOCK} along K, "
                    "stochastic gradient rounding",
        "algorithmic_flops_per_step": flops,
        "roofline": {"bound": "tensor", "achieved": tflops / world, "peak": pk["bf16_tflops_sustained"], "unit": "TFLOP/s",
                     "frac": tflops / world / pk["bf16_tflops_sustained"], "peak_burst": pk["bf16_tflops"],
                     "frac_of_burst": tflops / world / pk["bf16_tflops"], "peak_source": pk["source"],
                     "note": "whole step (4 fake-quantise passes + 3 GEMMs + column sums) over 6*M*N*K flops, against the "
                             "sustained cuBLAS bf16 figure; per-kernel figures in `parts`"},
        "best_gemm_TFLOPs": best,
        "parts": parts,
    }
