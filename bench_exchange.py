"""Timing of the gradient exchange for ``bench.py`` (more than one GPU): one 64 Mi-value fp32 bucket
(256 MiB) per rank, three ways.

* ``allreduce_fp32``       plain NCCL all-reduce of the fp32 bucket (no compression), for scale
* ``hook``                 ``axs6_gradient_hook``: local pack -> unpack, all-reduce of the reconstruction
* ``hook_packed``          ``axs6_gradient_hook_packed``: pack to 25-byte records, all-gather of the records
                           (6.25 bits per value on the wire), fused unpack-and-average; as a DDP hook it goes
                           through torch futures, whose callback machinery dominates when timed in isolation
* ``compressor_packed``    the same three steps issued back to back on the current stream
                           (``AXS6GradCompressor(packed=True).compress_and_allreduce``)

The two hooks give the same mean up to fp32 summation order (checked here); times are CUDA events, max
over ranks.
"""
from __future__ import annotations

import torch

NUMEL = 1 << 26


class _Bucket:
    def __init__(self, t):
        self._t = t

    def buffer(self):
        return self._t


def run(rank: int, world: int, dev, steps: int = 10) -> dict:
    import torch.distributed as dist
    from axs6_b200.unified import distributed as udist
    g = torch.Generator(device=dev).manual_seed(900 + rank)
    grad = torch.randn(NUMEL, generator=g, device=dev) * 1e-3
    state = udist.HookState()

    def plain():
        t = grad.clone()
        dist.all_reduce(t)
        return t.div_(world)

    def hook():
        return udist.axs6_gradient_hook(state, _Bucket(grad.clone())).wait()

    def packed():
        return udist.axs6_gradient_hook_packed(state, _Bucket(grad.clone())).wait()

    compressor = udist.AXS6GradCompressor(packed=True)

    def direct():
        return compressor.compress_and_allreduce(grad.clone())

    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    out = {}
    results = {}
    for name, fn in (("allreduce_fp32", plain), ("hook", hook), ("hook_packed", packed), ("compressor_packed", direct)):
        for _ in range(2):
            r = fn()
        results[name] = r
        dist.barrier()
        torch.cuda.synchronize()
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        dist.barrier()
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) / steps], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        out[name] = {"ms": float(t.item())}
    # the three phases of the packed exchange, timed one by one (each followed by a synchronisation)
    codec = udist.CudaCodec()
    flat = grad.clone()
    phases = {}

    def timed(name, fn):
        fn()
        dist.barrier()
        torch.cuda.synchronize()
        e0.record()
        for _ in range(steps):
            r = fn()
        e1.record()
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) / steps], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        phases[name] = float(t.item())
        return r

    mine = timed("pack_ms", lambda: codec.pack_padded16(flat))
    gathered = torch.empty(world * mine.numel(), dtype=torch.uint8, device=dev)
    timed("all_gather_ms", lambda: dist.all_gather_into_tensor(gathered, mine))
    timed("unpack_average_ms", lambda: codec.unpack_mean(gathered, world, mine.numel(), NUMEL, torch.float32))
    out["hook_packed_phases"] = phases
    a, b = results["hook"], results["hook_packed"]
    rel = float(((a - b).norm() / a.norm()).item())
    exact = float(((results["allreduce_fp32"] - a).norm() / results["allreduce_fp32"].norm()).item())
    out["hook_vs_packed_rel_diff"] = rel
    out["hook_vs_compressor_rel_diff"] = float(((a - results["compressor_packed"]).norm() / a.norm()).item())
    out["quantisation_rel_error_of_the_mean"] = exact
    out["wire_bytes_per_rank"] = {"allreduce_fp32": NUMEL * 4, "hook": NUMEL * 4, "hook_packed": NUMEL // 32 * 25}
    out["workload"] = f"one fp32 bucket of {NUMEL} values per rank, {world} ranks, NCCL; each time includes the clone of the bucket"
    return out
