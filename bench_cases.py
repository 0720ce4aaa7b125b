"""Runs ONE kernel of the library a few times on a small, larger-than-L2 case, for profilers.

    python bench.py --case {fq_f32|fq_bf16|fq_bf16_stochastic|pack_wire|pack_wire_f32|unpack_wire|unpack_wire_bf16|
                            unpack_sum4|gemm_fwd|gemm_dx|gemm_dw|gemm_fwd_full|gemm_dw_full|gemm_packed_fwd|gemm_packed_fwd_w|gemm_packed_dx|
                            gemm_packed_dw|fq_f32_full|fq_gather|pack_ef} [--launches n]

Device footprint stays under 1 GB so that a multi-pass capture finishes quickly (fq_f32_full is the
benchmark's own 32768 x 8192 launch, 2 GiB, meant for single-pass metrics only).
"""
from __future__ import annotations

import sys

import torch

from axs6_b200 import _lib


def run_case(what: str = "fq_f32", n: int = 3) -> None:
    lib = _lib.load()
    dev = torch.device("cuda", 0)
    rows, cols = 8192, 8192                       # 256 MiB fp32 / 128 MiB bf16: larger than the 126 MB L2
    g = torch.Generator(device=dev).manual_seed(0)
    st = torch.cuda.current_stream().cuda_stream
    if what == "fq_f32_full":
        rows, cols = 32768, 8192
        x = torch.randn(rows, cols, generator=g, device=dev)
        y = torch.empty_like(x)
        run = lambda: lib.axs6_fq(x.data_ptr(), y.data_ptr(), 0, 0, rows, cols, cols, cols, 32, 1, 0, 0, 0, 0, st)
    elif what == "fq_f32":
        x = torch.randn(rows, cols, generator=g, device=dev)
        y = torch.empty_like(x)
        run = lambda: lib.axs6_fq(x.data_ptr(), y.data_ptr(), 0, 0, rows, cols, cols, cols, 32, 1, 0, 0, 0, 0, st)
    elif what == "fq_bf16":
        x = torch.randn(rows, cols, generator=g, device=dev).to(torch.bfloat16)
        y = torch.empty_like(x)
        run = lambda: lib.axs6_fq(x.data_ptr(), y.data_ptr(), 1, 1, rows, cols, cols, cols, 32, 1, 0, 0, 0, 0, st)
    elif what == "pack_wire":
        x = torch.randn(rows, cols, generator=g, device=dev).to(torch.bfloat16)
        w = torch.empty(rows * cols // 32 * 25, dtype=torch.uint8, device=dev)
        run = lambda: lib.axs6_pack(x.data_ptr(), 1, rows, cols, cols, 32, 1, 0, 0, 0, 0, None, 1, w.data_ptr(), None, None, st)
    elif what == "pack_wire_f32":
        x = torch.randn(rows, cols, generator=g, device=dev)
        w = torch.empty(rows * cols // 32 * 25, dtype=torch.uint8, device=dev)
        run = lambda: lib.axs6_pack(x.data_ptr(), 0, rows, cols, cols, 32, 1, 0, 0, 0, 0, None, 1, w.data_ptr(), None, None, st)
    elif what == "unpack_wire_bf16":
        x = torch.randn(rows, cols, generator=g, device=dev).to(torch.bfloat16)
        w = torch.empty(rows * cols // 32 * 25, dtype=torch.uint8, device=dev)
        assert lib.axs6_pack(x.data_ptr(), 1, rows, cols, cols, 32, 1, 0, 0, 0, 0, None, 1, w.data_ptr(), None, None, st) == 0
        y = torch.empty(rows, cols, dtype=torch.bfloat16, device=dev)
        run = lambda: lib.axs6_unpack(1, w.data_ptr(), None, None, y.data_ptr(), 1, rows, cols, cols, 32, 1, st)
    elif what == "unpack_sum4":
        from axs6_b200 import ops
        per = rows * cols // 32 * 25
        w = torch.empty(4 * per, dtype=torch.uint8, device=dev)
        for s_ in range(4):
            xs = torch.randn(rows, cols, generator=g, device=dev)
            w[s_ * per:(s_ + 1) * per] = ops.pack(xs, 32, 1, "nearest", 1)
            del xs
        y = torch.empty(rows, cols, device=dev)
        run = lambda: lib.axs6_unpack_sum(1, w.data_ptr(), 4, per, y.data_ptr(), 0, rows, cols, cols, 32, 1, 4.0, st)
    elif what == "unpack_wire":
        x = torch.randn(rows, cols, generator=g, device=dev).to(torch.bfloat16)
        w = torch.empty(rows * cols // 32 * 25, dtype=torch.uint8, device=dev)
        assert lib.axs6_pack(x.data_ptr(), 1, rows, cols, cols, 32, 1, 0, 0, 0, 0, None, 1, w.data_ptr(), None, None, st) == 0
        y = torch.empty(rows, cols, device=dev)
        run = lambda: lib.axs6_unpack(1, w.data_ptr(), None, None, y.data_ptr(), 0, rows, cols, cols, 32, 1, st)
    elif what == "fq_gather":                  # embedding lookup: 65536 rows of a 32000 x 1024 fp32 table (256 MiB in + out)
        table = torch.randn(32000, 1024, generator=g, device=dev)
        idx = torch.randint(0, 32000, (65536,), generator=g, device=dev)
        y = torch.empty(65536, 1024, device=dev)
        run = lambda: lib.axs6_fq_gather(table.data_ptr(), 32000, idx.data_ptr(), y.data_ptr(), 0, 0, 65536, 1024, 1024, 1024,
                                         32, 1, 0, 0, 0, st)
    elif what == "pack_ef":                    # error feedback in one pass, 8192 x 8192 fp32, uniform grid, planes out
        x = torch.randn(rows, cols, generator=g, device=dev)
        err = torch.zeros_like(x)
        se = torch.empty(rows * cols // 32, dtype=torch.uint8, device=dev)
        sg = torch.empty(rows * cols, dtype=torch.uint8, device=dev)
        mg = torch.empty(rows * cols, dtype=torch.uint8, device=dev)
        run = lambda: lib.axs6_pack_ef(x.data_ptr(), err.data_ptr(), rows, cols, cols, 32, 0, 0, 0, 0, se.data_ptr(), sg.data_ptr(),
                                       mg.data_ptr(), st)
    elif what == "fq_bf16_stochastic":
        x = torch.randn(rows, cols, generator=g, device=dev).to(torch.bfloat16)
        y = torch.empty_like(x)
        run = lambda: lib.axs6_fq(x.data_ptr(), y.data_ptr(), 1, 1, rows, cols, cols, cols, 32, 1, 1, 0, 99, 0, st)
    elif what in ("gemm_fwd", "gemm_dx", "gemm_dw", "gemm_fwd_full", "gemm_dw_full"):
        M, N, K = 8192, 4096, 4096                 # operands 64 + 32 MiB, output 64 MiB
        out_dt, out_code = torch.bfloat16, 1
        if what == "gemm_fwd_full":                # the Linear benchmark's forward product (bf16 out)
            M = 16384
        if what == "gemm_dw_full":                 # its weight gradient: 4096 x 4096 outputs over 16384 rows, fp32 out
            M, N, K, out_dt, out_code = 4096, 4096, 16384, torch.float32, 0
        a_mn, b_mn = {"gemm_fwd": (0, 0), "gemm_dx": (0, 1), "gemm_dw": (1, 1), "gemm_fwd_full": (0, 0), "gemm_dw_full": (1, 1)}[what]
        a = torch.randn((K, M) if a_mn else (M, K), generator=g, device=dev).to(torch.bfloat16)
        b = torch.randn((K, N) if b_mn else (N, K), generator=g, device=dev).to(torch.bfloat16)
        c = torch.empty(M, N, dtype=out_dt, device=dev)
        run = lambda: lib.axs6_gemm_bf16(a.data_ptr(), b.data_ptr(), c.data_ptr(), None, M, N, K, a.stride(0), b.stride(0),
                                         N, a_mn, b_mn, out_code, st)
    elif what in ("gemm_packed_fwd", "gemm_packed_dx", "gemm_packed_dw", "gemm_packed_fwd_w"):
        from axs6_b200 import ops
        M, N, K = 8192, 4096, 4096
        a_mn, b_mn = {"gemm_packed_fwd": (0, 0), "gemm_packed_fwd_w": (0, 0), "gemm_packed_dx": (0, 1), "gemm_packed_dw": (1, 1)}[what]
        a = torch.randn((K, M) if a_mn else (M, K), generator=g, device=dev).to(torch.bfloat16)
        b = torch.randn((K, N) if b_mn else (N, K), generator=g, device=dev).to(torch.bfloat16)
        pa, pb = ops.pack_split(a), ops.pack_split(b)
        c = torch.empty(M, N, dtype=torch.bfloat16, device=dev)
        if what == "gemm_packed_fwd_w":          # only the weight as codes
            run = lambda: lib.axs6_gemm_packed(a.data_ptr(), None, K, pb.codes.data_ptr(), pb.exps.data_ptr(), 0, c.data_ptr(), None,
                                               M, N, K, N, a_mn, b_mn, 1, st)
        else:
            run = lambda: lib.axs6_gemm_packed(pa.codes.data_ptr(), pa.exps.data_ptr(), 0, pb.codes.data_ptr(), pb.exps.data_ptr(), 0,
                                               c.data_ptr(), None, M, N, K, N, a_mn, b_mn, 1, st)
    else:
        raise SystemExit(f"unknown case {what}")
    for _ in range(n):
        assert run() == 0
    torch.cuda.synchronize()
    if what.startswith("gemm"):
        assert lib.axs6_gemm_status() == 0
    assert lib.axs6_codec_status() == 0
    print(f"{what}: {n} launches ok")


if __name__ == "__main__":
    run_case(sys.argv[1] if len(sys.argv) > 1 else "fq_f32", int(sys.argv[2]) if len(sys.argv) > 2 else 3)
