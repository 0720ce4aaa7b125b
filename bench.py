#!/usr/bin/env python
"""Benchmark of the AXS-6 hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--scaling weak|strong]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

Headline workload (one "step" = one pass of the NF5 fake-quantise kernel over the rank's shard):
the largest tensor of the fake-quantise sweep, 32768 x 8192 fp32, per-row sigma log-uniform in
[1e-4, 10], block 32, nearest rounding.  With `--scaling weak` (default) every rank owns a
32768 x 8192 shard of a (N*32768) x 8192 tensor; with `--scaling strong` the one 32768 x 8192
tensor is split by rows over the ranks.  No collective is involved: blocks never cross rows.

Prints ONE JSON line on rank 0:
  value      fake-quant GB/s (algorithmic bytes = numel * (4 + 4)), inputs resident in HBM,
             CUDA-event time of K back-to-back launches, max over ranks
  e2e        same metric through the Python operator for host tensors (`fused_fake_quantize_host`) with
             pinned HOST buffers: H2D copy + kernel + D2H copy of every step inside the timed region
             (the operator pipelines them over chunks of rows, so both PCIe directions run at once)
  roofline   achieved / measured HBM peak for the dominant kernel
  cpu_baseline  the CPU oracle (a port of the reference's eager algorithm, C + OpenMP) on a
             bounded row sample of the same tensor, on this box's host cores
  codec, linear   the two other metrics of the path (pack->unpack GB/s, fused-linear TFLOP/s)
  fq_sweep, minigpt   the fake-quantise sweep (fp32 + bf16) and the MiniGPT-style training step
`--impl reference` times the CPU oracle alone (the reference is pure Python/torch and does not
travel to the GPU box; the oracle is its pinned C restatement) and prints the same line shape.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

ROWS, COLS, BLOCK = 32768, 8192, 32
METRIC = "axs6_fake_quant_GBps"
UNIT = "GB/s"
FALLBACK_HBM_GBS = 6650.0
FALLBACK_BF16_TFLOPS = 1590.0


def peaks() -> dict:
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            d = json.load(f)
        return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]),
                "bf16_tflops_sustained": float(d.get("bf16_tflops_sustained", d["bf16_tflops"])), "source": "measured"}
    return {"hbm_gbs": FALLBACK_HBM_GBS, "bf16_tflops": FALLBACK_BF16_TFLOPS,
            "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons of one GPU through NVML (read-only) while a timed
    region runs."""

    def __init__(self, index: int, period_s: float = 0.05):
        super().__init__(daemon=True)
        self.index, self.period = index, period_s
        self.samples: list[int] = []
        self.reasons: set[str] = set()
        self.max_mhz = None
        self._stop_evt = threading.Event()
        self.ok = False
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = int(pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM))
            self.ok = True
        except Exception:
            self.ok = False

    def run(self):
        if not self.ok:
            return
        nv = self.nv
        names = {
            getattr(nv, "nvmlClocksThrottleReasonHwSlowdown", 0x8): "hw_slowdown",
            getattr(nv, "nvmlClocksThrottleReasonHwThermalSlowdown", 0x40): "hw_thermal_slowdown",
            getattr(nv, "nvmlClocksThrottleReasonSwThermalSlowdown", 0x20): "sw_thermal_slowdown",
            getattr(nv, "nvmlClocksThrottleReasonSwPowerCap", 0x4): "sw_power_cap",
        }
        while not self._stop_evt.is_set():
            try:
                self.samples.append(int(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM)))
                r = int(nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h))
                for bit, name in names.items():
                    if r & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            self._stop_evt.wait(self.period)

    def finish(self) -> dict:
        self._stop_evt.set()
        if self.is_alive():
            self.join(timeout=2)
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons), "samples": 0}
        return {"sm_mhz": statistics.median(self.samples), "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(self.samples)}


def physical_gpu_index(local: int) -> int:
    vis = os.environ.get("CUDA_VISIBLE_DEVICES")
    if vis:
        try:
            return int(vis.split(",")[local])
        except Exception:
            return local
    return local


def make_input(rows: int, cols: int, seed: int, device):
    import torch
    g = torch.Generator(device=device).manual_seed(seed)
    sig = 10 ** (torch.rand(rows, 1, generator=g, device=device) * 5 - 4)
    return torch.randn(rows, cols, generator=g, device=device) * sig


# --------------------------------------------------------------------------------------- reference arm
def run_reference(args, rank: int, world: int) -> None:
    """CPU arm: the oracle (C + OpenMP port of the reference's eager algorithm) on host cores."""
    if rank != 0:
        return
    import numpy as np
    import oracle
    oracle.build()
    cores = os.cpu_count() or 1
    sample_rows = 2048
    rng = np.random.default_rng(0)
    sig = (10.0 ** (rng.random((sample_rows, 1)) * 5 - 4)).astype(np.float32)
    x = rng.standard_normal((sample_rows, COLS), dtype=np.float32) * sig
    for _ in range(max(1, min(args.warmup, 3))):
        oracle.fused_fake_quantize(x, BLOCK)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        oracle.fused_fake_quantize(x, BLOCK)
    dt = (time.perf_counter() - t0) / args.steps
    gbs = x.size * 8 / dt / 1e9
    sample = f"{sample_rows}x{COLS} fp32 rows of the {ROWS}x{COLS} workload per step"
    line = {
        "impl": "reference", "metric": METRIC, "value": gbs, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": args.scaling,
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"NF5 fake-quantize {ROWS}x{COLS} fp32, block {BLOCK}, nearest (fake-quantize sweep, largest size)",
                   "sample": sample, "l2": "n/a (CPU)"},
        "cpu_baseline": {"value": gbs, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": gbs, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# --------------------------------------------------------------------------------------- our arm
def run_ours(args, rank: int, local_rank: int, world: int) -> None:
    import numpy as np
    import torch
    import torch.distributed as dist

    from axs6_b200 import _lib
    import importlib
    qu = importlib.import_module("axs6_b200.unified.quantize_unified")
    udist = importlib.import_module("axs6_b200.unified.distributed")

    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    lib = _lib.load()
    if lib.axs6_query(0) != 1:
        raise RuntimeError("bench.py needs a compute-capability 10.x device; there is no fallback path")
    pk = peaks()

    rows = ROWS if args.scaling == "weak" else ROWS // world
    x = make_input(rows, COLS, 1000 + rank, dev)
    y = torch.empty_like(x)
    numel = x.numel()
    bytes_per_step = numel * 8
    stream = torch.cuda.current_stream().cuda_stream

    def step():
        st = lib.axs6_fq(x.data_ptr(), y.data_ptr(), 0, 0, rows, COLS, COLS, COLS, BLOCK, 1, 0, 0, 0, 0, stream)
        if st != 0:
            raise RuntimeError(f"axs6_fq -> {st}")

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(args.warmup, 3)):
        step()
    barrier()
    sampler = ClockSampler(physical_gpu_index(local_rank))
    sampler.start()
    l0 = _lib.launches()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    barrier()
    ms = e0.elapsed_time(e1)
    launches = _lib.launches() - l0
    # keep the sampler running over a few more launches if the timed region was very short
    t_end = time.perf_counter() + 0.6
    while time.perf_counter() < t_end and len(sampler.samples) < 6:
        step()
        torch.cuda.synchronize()
    clocks = sampler.finish()
    t = torch.tensor([ms], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_max = float(t.item())
    ms_per_step = ms_max / args.steps
    value = world * bytes_per_step / (ms_per_step * 1e-3) / 1e9
    achieved = bytes_per_step / (ms / args.steps * 1e-3) / 1e9          # this rank's kernel

    # ---------------- end to end: host buffers through the Python operator
    e2e_steps = max(1, min(args.steps, 3))
    hx = torch.empty((rows, COLS), dtype=torch.float32, pin_memory=True)
    hy = torch.empty((rows, COLS), dtype=torch.float32, pin_memory=True)
    hx.copy_(x)
    def e2e_step():
        # host buffers in, host buffers out: chunks of rows pipelined over H2D copy, kernel and D2H copy
        qu.fused_fake_quantize_host(hx, hy, BLOCK)
    e2e_step()
    barrier()
    e0.record()
    for _ in range(e2e_steps):
        e2e_step()
    e1.record()
    barrier()
    t = torch.tensor([e0.elapsed_time(e1)], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    e2e_ms = float(t.item()) / e2e_steps
    e2e_val = world * bytes_per_step / (e2e_ms * 1e-3) / 1e9
    del hx, hy

    extra = {}
    cpu = None
    sections = {t for t in args.sections.split(",") if t}
    if rank == 0:
        if "codec" in sections:
            extra["codec"] = bench_codec(torch, lib, udist, dev, pk)
        if "fq_sweep" in sections:
            extra["fq_sweep"] = bench_sweep(torch, lib, dev, pk, x)
        if world == 1:
            cpu = cpu_baseline(x)
    del x, y
    torch.cuda.empty_cache()
    try:
        extra_linear = bench_linear(args, rank, world, dev, pk) if "linear" in sections else None
        if extra_linear is not None and rank == 0:
            extra["linear"] = extra_linear
    except Exception as e:          # the linear metric is reported separately; never hide the headline
        if rank == 0:
            extra["linear"] = {"error": repr(e)}

    if world > 1 and "grad_exchange" in sections:
        try:
            from axs6_b200 import exchange_bench
            ex = exchange_bench.run(rank, world, dev)
            if rank == 0:
                extra["grad_exchange"] = ex
        except Exception as e:
            if rank == 0:
                extra["grad_exchange"] = {"error": repr(e)}

    if "minigpt" in sections:
        try:
            from axs6_b200 import minigpt_bench
            mg = minigpt_bench.run(args, rank, world, dev)
            if rank == 0:
                extra["minigpt"] = mg
        except Exception as e:
            if rank == 0:
                extra["minigpt"] = {"error": repr(e)}

    if rank == 0:
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": True,
            "scaling": args.scaling, "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": f"NF5 fake-quantize {ROWS}x{COLS} fp32, block {BLOCK}, nearest (fake-quantize sweep, largest size)",
                       "per_gpu_shard": f"{rows}x{COLS}", "parallelism": f"rows sharded over {world} GPU(s), no collective",
                       "l2": f"input {numel * 4 / 2**20:.0f} MiB + output {numel * 4 / 2**20:.0f} MiB per launch, larger than the 126 MB L2"},
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": pk["hbm_gbs"], "unit": "GB/s",
                         "frac": achieved / pk["hbm_gbs"], "traffic": TRAFFIC_BYTES_PER_LAUNCH.get(rows),
                         "peak_source": pk["source"], "kernel": "fq_vec_kernel<float,float,NF5,nearest>",
                         "algorithmic_bytes_per_launch": bytes_per_step},
            "e2e": {"value": e2e_val, "unit": UNIT, "h2d_bytes_per_step": numel * 4 * world,
                    "d2h_bytes_per_step": numel * 4 * world, "steps": e2e_steps},
            "gpu_launches": launches,
            "clocks": clocks,
        }
        if cpu is not None:
            line["cpu_baseline"] = cpu
        line.update(extra)
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


# DRAM bytes (read + write) of one launch of the headline kernel from the ncu capture summarised
# under profiles/ (captured on a 4096 x 8192 case and scaled by rows; traffic grows with rows).
TRAFFIC_BYTES_PER_LAUNCH: dict[int, float] = {32768: 4 * 486.1e6, 16384: 2 * 486.1e6, 8192: 486.1e6, 4096: 243.05e6}


def cpu_baseline(x) -> dict:
    """CPU oracle on a bounded row sample of the same tensor, all host threads."""
    import oracle
    oracle.build()
    sample_rows = 4096
    xs = x[:sample_rows].cpu().numpy()
    oracle.fused_fake_quantize(xs[:256], BLOCK)
    reps = 0
    t0 = time.perf_counter()
    while True:
        oracle.fused_fake_quantize(xs, BLOCK)
        reps += 1
        if time.perf_counter() - t0 > 10 or reps >= 20:
            break
    dt = (time.perf_counter() - t0) / reps
    return {"value": xs.size * 8 / dt / 1e9, "unit": UNIT, "cores": os.cpu_count() or 1, "kind": "port",
            "sample": f"first {sample_rows} rows ({sample_rows}x{COLS} fp32) of the workload, {reps} reps"}


def bench_codec(torch, lib, udist, dev, pk) -> dict:
    """Encode + decode round trip on bf16 8192 x 4096 (N(0,1), 0.1 % outliers, 1 % zeros): pack to
    the 25-byte wire records, unpack to fp32.  Buffers are rotated through a pool larger than L2."""
    rows, cols = 8192, 4096
    g = torch.Generator(device=dev).manual_seed(2)
    pool = []
    for i in range(4):
        x = torch.randn(rows, cols, generator=g, device=dev)
        x = torch.where(torch.rand(rows, cols, generator=g, device=dev) < 1e-3, x * 10, x)
        x = torch.where(torch.rand(rows, cols, generator=g, device=dev) < 1e-2, torch.zeros_like(x), x)
        xb = x.to(torch.bfloat16)
        wire = torch.empty(rows * (cols // 32) * 25, dtype=torch.uint8, device=dev)
        out = torch.empty(rows, cols, dtype=torch.float32, device=dev)
        planes = (torch.empty(rows * cols // 32, dtype=torch.uint8, device=dev), torch.empty(rows * cols, dtype=torch.uint8, device=dev),
                  torch.empty(rows * cols, dtype=torch.uint8, device=dev)) if i < 2 else None
        pool.append((xb, wire, out, x, planes))
    stream = torch.cuda.current_stream().cuda_stream

    def pack(i):
        xb, wire = pool[i % 4][:2]
        assert lib.axs6_pack(xb.data_ptr(), 1, rows, cols, cols, 32, 1, 0, 0, 0, 0, None, 1, wire.data_ptr(), None, None, stream) == 0

    def pack_f32(i):
        _, wire, _, x = pool[i % 4][:4]
        assert lib.axs6_pack(x.data_ptr(), 0, rows, cols, cols, 32, 1, 0, 0, 0, 0, None, 1, wire.data_ptr(), None, None, stream) == 0

    def pack_planes(i):
        x, pl = pool[i % 2][3], pool[i % 2][4]
        assert lib.axs6_pack(x.data_ptr(), 0, rows, cols, cols, 32, 1, 0, 0, 0, 0, None, 0, pl[0].data_ptr(), pl[1].data_ptr(),
                             pl[2].data_ptr(), stream) == 0

    def unpack_planes(i):
        out, pl = pool[i % 2][2], pool[i % 2][4]
        assert lib.axs6_unpack(0, pl[0].data_ptr(), pl[1].data_ptr(), pl[2].data_ptr(), out.data_ptr(), 0, rows, cols, cols, 32, 1, stream) == 0

    def unpack(i):
        _, wire, out = pool[i % 4][:3]
        assert lib.axs6_unpack(1, wire.data_ptr(), None, None, out.data_ptr(), 0, rows, cols, cols, 32, 1, stream) == 0

    def unpack_bf16(i):
        _, wire, out = pool[i % 4][:3]
        assert lib.axs6_unpack(1, wire.data_ptr(), None, None, out.data_ptr(), 1, rows, cols, cols, 32, 1, stream) == 0

    res = {}
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    n = 40
    rec = rows * cols // 32 * 25
    for name, fn, nbytes in (("pack_f32", pack_f32, rows * cols * 4 + rec), ("pack", pack, rows * cols * 2 + rec),
                             ("unpack", unpack, rows * cols * 4 + rec), ("unpack_bf16", unpack_bf16, rows * cols * 2 + rec),
                             ("pack_planes", pack_planes, rows * cols * 6 + rows * cols // 32),
                             ("unpack_planes", unpack_planes, rows * cols * 6 + rows * cols // 32)):
        for i in range(8):
            fn(i)
        torch.cuda.synchronize()
        e0.record()
        for i in range(n):
            fn(i)
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / n
        gbs = nbytes / (ms * 1e-3) / 1e9
        res[name] = {"ms": ms, "GBps": gbs, "frac_of_hbm_peak": gbs / pk["hbm_gbs"], "algorithmic_bytes": nbytes}
    res["roundtrip_bf16_GBps"] = 2 * (rows * cols * 2 + rec) / ((res["pack"]["ms"] + res["unpack_bf16"]["ms"]) * 1e-3) / 1e9
    res["stream_status"] = int(lib.axs6_codec_status())
    res["workload"] = ("8192x4096, block 32, 25-byte wire records: pack = bf16 -> records, pack_f32 = fp32 -> records, unpack = records "
                       "-> fp32, unpack_bf16 = records -> bf16 (4 rotating buffer sets, 4 x 355 MiB > L2); pack_planes / unpack_planes = fp32 <-> "
                       "AXSTensor planes (exponent, sign and magnitude bytes: quantize_unified / dequantize_unified), 2 buffer sets")
    return res


def bench_sweep(torch, lib, dev, pk, x_big) -> list:
    """Fake-quantise sweep (fp32 and bf16; 256^2, 4096^2, 8192x4096, 32768x8192).  Shapes smaller
    than L2 rotate through slices of the 1 GiB tensor so that every launch reads cold data."""
    stream = torch.cuda.current_stream().cuda_stream
    out = []
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for dt_name, dt_code, esz in (("f32", 0, 4), ("bf16", 1, 2)):
        src = x_big if dt_code == 0 else x_big.view(-1)[: x_big.numel() // 2].to(torch.bfloat16)
        flat = src.view(-1)
        dst = torch.empty_like(flat)
        for rows, cols in ((256, 256), (4096, 4096), (8192, 4096), (32768, 8192)):
            n = rows * cols
            if n > flat.numel():
                continue
            slots = max(1, min(flat.numel() // n, 64))
            iters = 30 if n >= (1 << 24) else 200

            def run(i):
                off = (i % slots) * n * esz
                st = lib.axs6_fq(flat.data_ptr() + off, dst.data_ptr() + off, dt_code, dt_code, rows, cols, cols, cols,
                                 BLOCK, 1, 0, 0, 0, 0, stream)
                assert st == 0
            for i in range(5):
                run(i)
            torch.cuda.synchronize()
            e0.record()
            for i in range(iters):
                run(i)
            e1.record()
            torch.cuda.synchronize()
            ms = e0.elapsed_time(e1) / iters
            gbs = n * esz * 2 / (ms * 1e-3) / 1e9
            out.append({"shape": f"{rows}x{cols}", "dtype": dt_name, "us": ms * 1e3, "GBps": gbs,
                        "frac_of_hbm_peak": gbs / pk["hbm_gbs"], "rotating_slots": slots})
        del dst
    return out


def bench_linear(args, rank, world, dev, pk):
    """AXS-6 Linear forward + backward (M=16384, K=N=4096); filled in by the linear module."""
    try:
        from axs6_b200 import linear_bench
    except Exception:
        return None
    return linear_bench.run(args, rank, world, dev, pk)


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--scaling", default="weak", choices=["weak", "strong"])
    ap.add_argument("--sections", default="codec,fq_sweep,linear,grad_exchange,minigpt",
                    help="extra sections of the JSON line to measure after the headline (comma list; empty = none)")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world != args.gpus and world > 1:
        args.gpus = world
    if args.impl == "reference":
        if args.steps > 20:
            args.steps = 20
        run_reference(args, rank, world)
        return
    if args.gpus > 1 and world == 1:
        # launched without torchrun: re-launch ourselves under it
        import subprocess
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={args.gpus}",
               "--master-addr", "127.0.0.1", "--master-port", os.environ.get("MASTER_PORT", "29541"),
               os.path.abspath(__file__), "--gpus", str(args.gpus), "--steps", str(args.steps),
               "--warmup", str(args.warmup), "--scaling", args.scaling]
        sys.exit(subprocess.call(cmd))
    run_ours(args, rank, local_rank, world)


if __name__ == "__main__":
    main()
