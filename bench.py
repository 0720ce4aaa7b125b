#!/usr/bin/env python
"""Benchmark of the AXS-6 hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--scaling strong|weak]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...
    python bench.py --case NAME [--launches n]        # one kernel on a small case, for profilers

Headline workload (one "step" = one pass of the NF5 fake-quantise kernel over the rank's shard):
the largest tensor of the fake-quantise sweep, 32768 x 8192 fp32, per-row sigma log-uniform in
[1e-4, 10], block 32, nearest rounding.  With N ranks the default (`--scaling strong`) splits that
ONE tensor by rows, 32768 / N rows per rank; `--scaling weak` gives every rank a 32768 x 8192 tensor
of its own.  The reading that is not the headline is measured too and reported under
`other_scaling`.  No collective is involved: blocks never cross rows.

Prints ONE JSON line on rank 0:
  value      fake-quant GB/s (algorithmic bytes = numel * (4 + 4)), inputs resident in HBM,
             CUDA-event time of K back-to-back launches, max over ranks
  e2e        same metric through the Python operator for host tensors (`fused_fake_quantize_host`) with
             pinned HOST buffers: H2D copy + kernel + D2H copy of every step inside the timed region
             (the operator pipelines them over chunks of rows, so both PCIe directions run at once)
  roofline   achieved / measured HBM peak for the dominant kernel
  cpu_baseline  the reference's CPU implementation of the same pass on a bounded row sample of the same
             tensor, on this box's host cores, thread count set explicitly and reported: kind
             "reference" = the reference's own eager function from baseline/_ref, "port" = the C
             restatement under oracle/ when that copy is absent
  codec, linear   the two other metrics of the path (pack->unpack GB/s, fused-linear TFLOP/s)
  fq_sweep, minigpt   the fake-quantise sweep (fp32 + bf16) and the MiniGPT-style training step
  embedding_gather   the embedding lookup: gather + fake-quantise in one kernel against the two-step form
  gpu_reference   the unmodified reference (baseline/_ref) run on the SAME GPU on the same tensors: its eager
             and Triton fake-quantise and its mixed-precision Linear step, each beside this library's time and with
             a bit-for-bit comparison of the fake-quantise outputs (N = 1 only; see bench_gpu_reference.py)
`--impl reference` times that CPU arm alone, on the first 4096 rows of the same seeded tensor, and
prints the same line shape (rank 0 only under torchrun).
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


def host_cores() -> int:
    try:
        return len(os.sched_getaffinity(0))
    except Exception:
        return os.cpu_count() or 1


# --------------------------------------------------------------------------------------- CPU arm
class CpuReference:
    """The reference's CPU implementation of the headline path, with every host thread it can use.

    kind "reference": the reference's own eager ``fused_fake_quantize`` (axs/unified/quantize_unified.py:121-204),
    imported unmodified from ``baseline/_ref`` (put there by baseline/install_reference.py; it travels with the
    repository snapshot but is not part of its history).  kind "port": the C + OpenMP restatement under
    ``oracle/`` when that copy is absent.  Thread counts are set explicitly (a launcher such as torchrun exports
    OMP_NUM_THREADS=1) and the count in effect is what ``cores`` reports."""

    def __init__(self):
        import torch
        self.torch = torch
        want = host_cores()
        ref_dir = os.path.join(ROOT, "baseline", "_ref")
        self.kind = "port"
        if os.path.isdir(os.path.join(ref_dir, "axs")):
            try:
                if ref_dir not in sys.path:
                    sys.path.insert(0, ref_dir)
                import importlib
                self.ref_fq = importlib.import_module("axs.unified.quantize_unified").fused_fake_quantize
                torch.set_num_threads(want)
                self.cores = int(torch.get_num_threads())
                self.kind = "reference"
            except Exception:
                self.kind = "port"
        if self.kind == "port":
            import oracle
            oracle.build()
            self.oracle = oracle
            self.cores = oracle.set_threads(want)

    def run(self, x_cpu) -> None:
        """One pass over a CPU fp32 tensor."""
        if self.kind == "reference":
            with self.torch.no_grad():
                self.ref_fq(x_cpu, BLOCK, "nearest")
        else:
            self.oracle.fused_fake_quantize(x_cpu.numpy(), BLOCK)

    def describe(self) -> str:
        return ("reference eager fused_fake_quantize (torch CPU ops, unmodified copy under baseline/_ref)" if self.kind == "reference"
                else "C + OpenMP port of the reference's eager algorithm (oracle/)")


def reference_sample(sample_rows: int):
    """The first `sample_rows` rows of the 32768 x 8192 workload tensor: the rows rank 0 of the GPU arm holds."""
    import torch
    if torch.cuda.is_available():
        dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
        x = make_input(ROWS, COLS, 1000, dev)[:sample_rows].cpu()
        torch.cuda.empty_cache()
        return x, True
    return make_input(sample_rows, COLS, 1000, torch.device("cpu")), False


def run_reference(args, rank: int, world: int) -> None:
    """CPU arm: the reference's own implementation of the path on the box's host cores (rank 0 only)."""
    if rank != 0:
        return
    sample_rows = 4096
    x, same = reference_sample(sample_rows)
    cpu = CpuReference()
    for _ in range(max(1, min(args.warmup, 3))):
        cpu.run(x)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        cpu.run(x)
    dt = (time.perf_counter() - t0) / args.steps
    gbs = x.numel() * 8 / dt / 1e9
    sample = (f"first {sample_rows} rows ({sample_rows}x{COLS} fp32) of the {ROWS}x{COLS} workload tensor per step"
              + ("" if same else " (generated on the CPU: no CUDA device for the GPU arm's generator)"))
    line = {
        "impl": "reference", "metric": METRIC, "value": gbs, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": args.scaling,
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD, "sample": sample, "l2": "n/a (CPU)", "what": cpu.describe()},
        "cpu_baseline": {"value": gbs, "unit": UNIT, "cores": cpu.cores, "kind": cpu.kind, "sample": sample},
        "e2e": {"value": gbs, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def cpu_baseline(x) -> dict:
    """The CPU arm on a bounded row sample of the same tensor (about 10 s), all host threads."""
    sample_rows = 4096
    xs = x[:sample_rows].cpu()
    cpu = CpuReference()
    cpu.run(xs[:256])
    reps = 0
    t0 = time.perf_counter()
    while True:
        cpu.run(xs)
        reps += 1
        if time.perf_counter() - t0 > 10 or reps >= 20:
            break
    dt = (time.perf_counter() - t0) / reps
    return {"value": xs.numel() * 8 / dt / 1e9, "unit": UNIT, "cores": cpu.cores, "kind": cpu.kind,
            "sample": f"first {sample_rows} rows ({sample_rows}x{COLS} fp32) of the workload, {reps} reps", "what": cpu.describe()}


# --------------------------------------------------------------------------------------- our arm
WORKLOAD = f"NF5 fake-quantize {ROWS}x{COLS} fp32, block {BLOCK}, nearest (fake-quantize sweep, largest size)"

# DRAM bytes (read + write) of ONE launch of the headline kernel, by shard rows, each from an ncu capture of a launch of
# exactly that size with the two DRAM byte counters only (profiles/fq_vec_kernel_f32_32768x8192.md); None where no
# capture of that shard size exists.
TRAFFIC_BYTES_PER_LAUNCH: dict[int, float] = {32768: 2.09e9, 8192: 485.5e6}
TRAFFIC_CAPTURED = {"rows": 32768, "cols": 8192, "dram_bytes_read": 1.07e9, "dram_bytes_write": 1.02e9,
                    "algorithmic_bytes": 32768 * 8192 * 8, "passes": 1,
                    "source": "profiles/fq_vec_kernel_f32_32768x8192.md"}


def run_ours(args, rank: int, local_rank: int, world: int) -> None:
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
    stream = torch.cuda.current_stream().cuda_stream

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(v: float) -> float:
        t = torch.tensor([v], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def shard(scaling: str):
        """This rank's rows: strong = its contiguous row range of THE 32768 x 8192 tensor (seed 1000);
        weak = a 32768 x 8192 tensor of its own (seed 1000 + rank)."""
        if scaling == "weak" or world == 1:
            return make_input(ROWS, COLS, 1000 + rank, dev)
        per = ROWS // world
        full = make_input(ROWS, COLS, 1000, dev)
        part = full[rank * per:(rank + 1) * per].clone()
        del full
        torch.cuda.empty_cache()
        return part

    def time_fq(x, steps: int, warmup: int):
        """CUDA-event time of `steps` back-to-back launches over this rank's shard.  A shard whose input +
        output are below 1 GiB rotates through several output buffers and input copies so that every launch
        reads data that is not in L2."""
        rows = x.shape[0]
        nbytes = x.numel() * 8
        sets = max(1, min(8, -(-(1 << 30) // nbytes)))
        xs = [x] + [x.clone() for _ in range(sets - 1)]
        ys = [torch.empty_like(x) for _ in range(sets)]

        def step(i):
            xi, yi = xs[i % sets], ys[i % sets]
            st = lib.axs6_fq(xi.data_ptr(), yi.data_ptr(), 0, 0, rows, COLS, COLS, COLS, BLOCK, 1, 0, 0, 0, 0, stream)
            if st != 0:
                raise RuntimeError(f"axs6_fq -> {st}")

        for i in range(max(warmup, 3)):
            step(i)
        barrier()
        l0 = _lib.launches()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        e0.record()
        for i in range(steps):
            step(i)
        e1.record()
        barrier()
        ms = e0.elapsed_time(e1)
        return ms, _lib.launches() - l0, step, sets

    primary = args.scaling if world > 1 else "weak"          # one GPU: the two readings coincide
    x = shard(primary)
    rows = x.shape[0]
    numel = x.numel()
    bytes_per_step = numel * 8
    sampler = ClockSampler(physical_gpu_index(local_rank))
    sampler.start()
    ms, launches, step, sets = time_fq(x, args.steps, args.warmup)
    # keep the sampler running over a few more launches if the timed region was very short
    t_end = time.perf_counter() + 0.6
    i = 0
    while time.perf_counter() < t_end and len(sampler.samples) < 6:
        step(i)
        i += 1
        torch.cuda.synchronize()
    clocks = sampler.finish()
    ms_per_step = max_over_ranks(ms) / args.steps
    value = world * bytes_per_step / (ms_per_step * 1e-3) / 1e9
    achieved = bytes_per_step / (ms / args.steps * 1e-3) / 1e9          # this rank's kernel

    # ---------------- the other reading of "N GPUs" (more than one rank only)
    other = None
    if world > 1:
        other_name = "weak" if primary == "strong" else "strong"
        xo = shard(other_name)
        ms_o, _, _, sets_o = time_fq(xo, args.steps, args.warmup)
        ms_o = max_over_ranks(ms_o) / args.steps
        other = {"scaling": other_name, "per_gpu_shard": f"{xo.shape[0]}x{COLS}", "ms_per_step": ms_o,
                 "value": world * xo.numel() * 8 / (ms_o * 1e-3) / 1e9, "unit": UNIT, "rotating_buffer_sets": sets_o}
        del xo
        torch.cuda.empty_cache()

    # ---------------- end to end: host buffers through the Python operator
    e2e_steps = max(1, min(args.steps, 3))
    hx = torch.empty((rows, COLS), dtype=torch.float32, pin_memory=True)
    hy = torch.empty((rows, COLS), dtype=torch.float32, pin_memory=True)
    hx.copy_(x)

    def e2e_step():
        # host buffers in, host buffers out: chunks of rows pipelined over H2D copy, kernel and D2H copy
        qu.fused_fake_quantize_host(hx, hy, BLOCK)
    e2e_step()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record()
    for _ in range(e2e_steps):
        e2e_step()
    e1.record()
    barrier()
    e2e_ms = max_over_ranks(e0.elapsed_time(e1)) / e2e_steps
    e2e_val = world * bytes_per_step / (e2e_ms * 1e-3) / 1e9
    del hx, hy

    extra = {}
    cpu = None
    sections = {t for t in args.sections.split(",") if t}
    if rank == 0:
        if "codec" in sections:
            extra["codec"] = bench_codec(torch, lib, udist, dev, pk)
        if world == 1:
            cpu = cpu_baseline(x)
    del x
    torch.cuda.empty_cache()
    if rank == 0 and "fq_sweep" in sections:
        extra["fq_sweep"] = bench_sweep(torch, lib, dev, pk)
        try:
            extra["embedding_gather"] = bench_embedding(torch, dev)
        except Exception as e:
            extra["embedding_gather"] = {"error": repr(e)[:300]}
    torch.cuda.empty_cache()
    try:
        extra_linear = linear_section(args, rank, world, dev, pk) if "linear" in sections else None
        if extra_linear is not None and rank == 0:
            extra["linear"] = extra_linear
    except Exception as e:          # the linear metric is reported separately; never hide the headline
        if rank == 0:
            extra["linear"] = {"error": repr(e)}

    if world == 1 and rank == 0 and "gpu_reference" in sections:
        try:
            import bench_gpu_reference
            xr = make_input(ROWS, COLS, 1000, dev)
            lin_ms = extra.get("linear", {}).get("ms_per_step")
            extra["gpu_reference"] = bench_gpu_reference.run(dev, xr, ms_per_step, lin_ms)
            del xr
        except Exception as e:
            extra["gpu_reference"] = {"error": repr(e)[:300]}
        torch.cuda.empty_cache()

    if world > 1 and "grad_exchange" in sections:
        try:
            import bench_exchange
            ex = bench_exchange.run(rank, world, dev)
            if rank == 0:
                extra["grad_exchange"] = ex
        except Exception as e:
            if rank == 0:
                extra["grad_exchange"] = {"error": repr(e)}

    if "minigpt" in sections:
        try:
            import bench_minigpt
            mg = bench_minigpt.run(args, rank, world, dev)
            if rank == 0:
                extra["minigpt"] = mg
        except Exception as e:
            if rank == 0:
                extra["minigpt"] = {"error": repr(e)}

    if rank == 0:
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": True,
            "scaling": primary, "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": WORKLOAD, "per_gpu_shard": f"{rows}x{COLS}",
                       "parallelism": (f"the {ROWS}x{COLS} tensor split by rows over {world} GPU(s), no collective" if primary == "strong" or world == 1
                                       else f"one {ROWS}x{COLS} tensor per GPU ({world} GPU(s)), no collective"),
                       "l2": f"input {numel * 4 / 2**20:.0f} MiB + output {numel * 4 / 2**20:.0f} MiB per launch, "
                             f"{sets} rotating buffer set(s): every launch streams data larger than the 126 MB L2"},
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": pk["hbm_gbs"], "unit": "GB/s",
                         "frac": achieved / pk["hbm_gbs"], "traffic": TRAFFIC_BYTES_PER_LAUNCH.get(rows),
                         "traffic_captured": TRAFFIC_CAPTURED,
                         "peak_source": pk["source"], "kernel": "fq_vec_kernel<float,float,NF5,nearest>",
                         "algorithmic_bytes_per_launch": bytes_per_step},
            "e2e": {"value": e2e_val, "unit": UNIT, "h2d_bytes_per_step": numel * 4 * world,
                    "d2h_bytes_per_step": numel * 4 * world, "steps": e2e_steps},
            "gpu_launches": launches,
            "clocks": clocks,
        }
        if other is not None:
            line["other_scaling"] = other
        if cpu is not None:
            line["cpu_baseline"] = cpu
        line.update(extra)
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


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
    rt_bytes = 2 * (rows * cols * 2 + rec)
    rt_ms = res["pack"]["ms"] + res["unpack_bf16"]["ms"]
    res["roundtrip_bf16_GBps"] = rt_bytes / (rt_ms * 1e-3) / 1e9
    res["roofline"] = {"bound": "hbm", "achieved": res["roundtrip_bf16_GBps"], "peak": pk["hbm_gbs"], "unit": "GB/s",
                       "frac": res["roundtrip_bf16_GBps"] / pk["hbm_gbs"], "traffic": None, "peak_source": pk["source"],
                       "kernel": "pack_bf16_nf5_b32_bulk_kernel + unpack_nf5_b32_bulk_kernel<bf16>",
                       "algorithmic_bytes_per_roundtrip": rt_bytes,
                       "note": "encode + decode round trip of the bf16 8192x4096 tensor: (values + 25-byte records) read or written "
                               "by each of the two launches, over the sum of their CUDA-event times"}
    res["stream_status"] = int(lib.axs6_codec_status())
    res["workload"] = ("8192x4096, block 32, 25-byte wire records: pack = bf16 -> records, pack_f32 = fp32 -> records, unpack = records "
                       "-> fp32, unpack_bf16 = records -> bf16 (4 rotating buffer sets, 4 x 355 MiB > L2); pack_planes / unpack_planes = fp32 <-> "
                       "AXSTensor planes (exponent, sign and magnitude bytes: quantize_unified / dequantize_unified), 2 buffer sets")
    return res


def bench_embedding(torch, dev) -> dict:
    """The embedding lookup of the path: 8192 rows of a 32000 x 1024 fp32 table gathered and fake-quantised by ONE
    kernel (axs6_fq_gather) against the reference's two steps on the same GPU ops (F.embedding, then fake-quantise)."""
    import importlib
    from axs6_b200 import ops
    fu = importlib.import_module("axs6_b200.unified.functional_unified")
    g = torch.Generator(device=dev).manual_seed(31)
    table = torch.randn(32000, 1024, generator=g, device=dev)
    idx = torch.randint(0, 32000, (8, 1024), generator=g, device=dev)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)

    def t_of(fn, n=50):
        for _ in range(5):
            fn()
        torch.cuda.synchronize()
        e0.record()
        for _ in range(n):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / n * 1e3

    fused = t_of(lambda: ops.fake_quantize_gather(table, idx))
    two = t_of(lambda: fu.fake_quantize_unified(torch.nn.functional.embedding(idx, table), 32, "nearest"))
    a = ops.fake_quantize_gather(table, idx)
    b = fu.fake_quantize_unified(torch.nn.functional.embedding(idx, table), 32, "nearest")
    return {"fused_us": fused, "gather_then_fake_quantize_us": two, "bit_identical": bool(torch.equal(a, b)),
            "workload": "8192 looked-up rows of a 32000 x 1024 fp32 table, NF5, block 32 (64 MiB of rows in + out)"}


def bench_sweep(torch, lib, dev, pk) -> list:
    """Fake-quantise sweep: fp32 and bf16 at 1024^2 (the reference's CPU-runnable case), 256^2, 4096^2,
    8192x4096 and 32768x8192, per-row sigma log-uniform in [1e-4, 10] (N(0, 0.02) for 1024^2).  Shapes that
    fit L2 rotate through slots of a 512 Mi-value tensor so that every launch reads cold data."""
    stream = torch.cuda.current_stream().cuda_stream
    out = []
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    total = ROWS * COLS
    for dt_name, dt_code, esz, tdt in (("f32", 0, 4, torch.float32), ("bf16", 1, 2, torch.bfloat16)):
        src = torch.empty(total, dtype=tdt, device=dev)
        quarter = total // 4
        for q in range(4):                                   # filled in quarters: no 2 GiB fp32 temporary for bf16
            src[q * quarter:(q + 1) * quarter].copy_(make_input(ROWS // 4, COLS, 2000 + q, dev).view(-1))
        dst = torch.empty_like(src)
        for rows, cols in ((1024, 1024), (256, 256), (4096, 4096), (8192, 4096), (32768, 8192)):
            n = rows * cols
            slots = max(1, min(total // n, 64))
            iters = 30 if n >= (1 << 24) else 200
            if (rows, cols) == (1024, 1024):                 # values ~ N(0, 0.02) in every slot used
                g = torch.Generator(device=dev).manual_seed(0)
                src[:slots * n].copy_((torch.randn(slots * n, generator=g, device=dev) * 0.02).to(tdt))

            def run(i):
                off = (i % slots) * n * esz
                st = lib.axs6_fq(src.data_ptr() + off, dst.data_ptr() + off, dt_code, dt_code, rows, cols, cols, cols,
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
                        "frac_of_hbm_peak": gbs / pk["hbm_gbs"], "rotating_slots": slots,
                        "algorithmic_bytes": n * esz * 2})
            if (rows, cols) == (1024, 1024):                 # restore the sweep distribution in the slots just overwritten
                src[:quarter].copy_(make_input(ROWS // 4, COLS, 2000, dev).view(-1))
        del src, dst
        torch.cuda.empty_cache()
    return out


def linear_section(args, rank, world, dev, pk):
    """AXS-6 Linear forward + backward (M=16384, K=N=4096); see bench_linear.py."""
    import bench_linear
    return bench_linear.run(args, rank, world, dev, pk)


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--scaling", default="strong", choices=["weak", "strong"],
                    help="what N GPUs means for the headline: strong = the one 32768x8192 tensor split by rows (default), "
                         "weak = one such tensor per GPU; the other reading is reported under `other_scaling`")
    ap.add_argument("--sections", default="codec,fq_sweep,linear,gpu_reference,grad_exchange,minigpt",
                    help="extra sections of the JSON line to measure after the headline (comma list; empty = none)")
    ap.add_argument("--case", default=None,
                    help="run ONE kernel a few times on a small larger-than-L2 case and exit (for profilers); see bench_cases.py")
    ap.add_argument("--launches", type=int, default=3, help="launches of --case")
    args = ap.parse_args()
    if args.case:
        import bench_cases
        bench_cases.run_case(args.case, args.launches)
        return
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
               "--warmup", str(args.warmup), "--scaling", args.scaling, "--sections", args.sections]
        sys.exit(subprocess.call(cmd))
    run_ours(args, rank, local_rank, world)


if __name__ == "__main__":
    main()
