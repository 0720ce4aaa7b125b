"""Timing of the AXS-6 Linear forward + backward (bf16 activations (M, K), fp32 master weights
(N, K), block 32 along K) for ``bench.py``: K = N = 4096.

One step = ``axs6_linear_fwd`` + ``axs6_linear_bwd`` through the C ABI with caller-owned buffers:
fake-quantise passes for activations, weight and (stochastic) gradient, three tcgen05 GEMMs, the
bias-gradient column sums.  The backward reuses the forward's quantised weight.

More than one rank = data parallel over the batch: X, Y, dX sharded by rows, W replicated, the fp32
weight gradient summed with an NCCL all-reduce.  The backward is issued as two calls: the first
produces dW, whose all-reduce starts at once on NCCL's stream; the second produces dX and db under
it, with a few SMs left free for the collective's CTAs (``axs6_tune(8, n)``).  Both readings of
"N GPUs" are timed: ``weak`` = 16384 rows per GPU, ``strong`` = 16384 rows in total, and for the
strong case also the compute alone (all-reduce off).  The split over output columns (whole batch on
every rank, N/world rows of W each; all-gather of y, all-reduce of the partial dX) is timed beside the
strong case as ``column_split``.
"""
from __future__ import annotations

import torch

from axs6_b200 import _lib

M_ROWS, K, N, BLOCK = 16384, 4096, 4096, 32
FLAG_QGRAD, FLAG_REUSE_WQ, FLAG_REUSE_GQ, FLAG_PACKED = 2, 32, 64, 128


class _Case:
    """Buffers and launch closures of one Linear of M rows on this rank."""

    def __init__(self, lib, dev, M: int, seed: int, packed: bool = False):
        self.lib, self.M = lib, M
        self.pk = FLAG_PACKED if packed else 0
        g = torch.Generator(device=dev).manual_seed(seed)
        self.x = torch.randn(M, K, generator=g, device=dev).to(torch.bfloat16)
        self.w = torch.randn(N, K, generator=g, device=dev) * 0.02
        self.bias = torch.zeros(N, device=dev)
        self.go = torch.randn(M, N, generator=g, device=dev).to(torch.bfloat16)
        self.y = torch.empty(M, N, dtype=torch.bfloat16, device=dev)
        self.dx = torch.empty(M, K, dtype=torch.bfloat16, device=dev)
        self.dws = [torch.empty(N, K, dtype=torch.float32, device=dev) for _ in range(2)]
        self.db = torch.empty(N, dtype=torch.float32, device=dev)
        codes = (8, 9, 10, 3) if packed else (0, 1, 2, 3)
        ws = [torch.empty(int(lib.axs6_linear_workspace_bytes(i, M, N, K)), dtype=torch.uint8, device=dev) for i in codes]
        self.xq, self.wq, self.gq, self.part = ws
        self.stream = torch.cuda.current_stream().cuda_stream

    def fwd(self):
        st = self.lib.axs6_linear_fwd(self.x.data_ptr(), 1, K, self.w.data_ptr(), 0, K, self.bias.data_ptr(), self.y.data_ptr(),
                                      1, N, self.M, N, K, BLOCK, 1, 1 | self.pk, self.xq.data_ptr(), self.wq.data_ptr(), self.stream)
        assert st == 0, st

    def _bwd(self, i, dx, dw, db, flags):
        M = self.M
        st = self.lib.axs6_linear_bwd(self.go.data_ptr(), 1, N, self.xq.data_ptr(), self.w.data_ptr(), 0, K, dx, 1, K, dw, K, db,
                                      M, N, K, BLOCK, 1, flags | self.pk, 1234, i * (M * N // 8), None, self.gq.data_ptr(),
                                      self.wq.data_ptr(), self.part.data_ptr(), None, self.stream)
        assert st == 0, st

    def bwd_dw(self, i):
        self._bwd(i, None, self.dws[i % 2].data_ptr(), None, FLAG_QGRAD)

    def bwd_dx(self, i):
        self._bwd(i, self.dx.data_ptr(), None, self.db.data_ptr(), FLAG_QGRAD | FLAG_REUSE_WQ | FLAG_REUSE_GQ)

    def bwd_all(self, i):
        self._bwd(i, self.dx.data_ptr(), self.dws[i % 2].data_ptr(), self.db.data_ptr(), FLAG_QGRAD | FLAG_REUSE_WQ)


class _ColumnCase:
    """The other way the Linear splits: output columns.  Every rank holds the whole batch (x and the incoming
    gradient are replicated) and N/world rows of W.  Forward: y[:, mine] = FQ(x) FQ(W_mine)^T, then an all-gather of the
    column blocks.  Backward: dW_mine and db_mine are local; dX is a sum over the ranks' column blocks, so the bf16
    partial dX is all-reduced -- started right after the dX product so that it runs under the dW product."""

    def __init__(self, lib, dev, rank: int, world: int, seed: int):
        self.lib, self.world, self.rank = lib, world, rank
        M, Nl = M_ROWS, N // world
        self.M, self.Nl = M, Nl
        g = torch.Generator(device=dev).manual_seed(seed)        # the same seed on every rank: replicated operands
        self.x = torch.randn(M, K, generator=g, device=dev).to(torch.bfloat16)
        self.w_full = torch.randn(N, K, generator=g, device=dev) * 0.02
        self.go_full = torch.randn(M, N, generator=g, device=dev).to(torch.bfloat16)
        self.w = self.w_full[rank * Nl:(rank + 1) * Nl]
        self.go = self.go_full[:, rank * Nl:(rank + 1) * Nl]     # a column block: row pitch N
        self.bias = torch.zeros(Nl, device=dev)
        self.y_mine = torch.empty(M, Nl, dtype=torch.bfloat16, device=dev)
        self.y_blocks = torch.empty(world, M, Nl, dtype=torch.bfloat16, device=dev)
        self.y = torch.empty(M, N, dtype=torch.bfloat16, device=dev)
        self.dx = torch.empty(M, K, dtype=torch.bfloat16, device=dev)
        self.dw = torch.empty(Nl, K, dtype=torch.float32, device=dev)
        self.db = torch.empty(Nl, dtype=torch.float32, device=dev)
        ws = [torch.empty(int(lib.axs6_linear_workspace_bytes(i, M, Nl, K)), dtype=torch.uint8, device=dev) for i in (0, 1, 2, 3)]
        self.xq, self.wq, self.gq, self.part = ws
        self.stream = torch.cuda.current_stream().cuda_stream

    def fwd_mine(self):
        st = self.lib.axs6_linear_fwd(self.x.data_ptr(), 1, K, self.w.data_ptr(), 0, K, self.bias.data_ptr(),
                                      self.y_mine.data_ptr(), 1, self.Nl, self.M, self.Nl, K, BLOCK, 1, 1,
                                      self.xq.data_ptr(), self.wq.data_ptr(), self.stream)
        assert st == 0, st

    def gather(self, dist, group):
        dist.all_gather_into_tensor(self.y_blocks, self.y_mine)       # nothing runs beside it: the default group, all CTAs
        self.lay_side_by_side()

    def lay_side_by_side(self):
        torch.cat(list(self.y_blocks.unbind(0)), dim=1, out=self.y)                        # (world, M, N/world) -> (M, N)

    def _bwd(self, i, dx, dw, db, flags):
        M, Nl = self.M, self.Nl
        st = self.lib.axs6_linear_bwd(self.go.data_ptr(), 1, N, self.xq.data_ptr(), self.w.data_ptr(), 0, K, dx, 1, K, dw, K, db,
                                      M, Nl, K, BLOCK, 1, flags, 1234, i * (M * N // 8), None, self.gq.data_ptr(),
                                      self.wq.data_ptr(), self.part.data_ptr(), None, self.stream)
        assert st == 0, st

    def step(self, i, dist, group, collectives: bool, reserve: int):
        self.fwd_mine()
        if collectives:
            self.gather(dist, group)
        self._bwd(i, self.dx.data_ptr(), None, None, FLAG_QGRAD | FLAG_REUSE_WQ)
        pending = dist.all_reduce(self.dx, group=group, async_op=True) if collectives else None
        if reserve and collectives:
            self.lib.axs6_tune(8, reserve)
        self._bwd(i, None, self.dw.data_ptr(), self.db.data_ptr(), FLAG_QGRAD | FLAG_REUSE_GQ)
        if reserve and collectives:
            self.lib.axs6_tune(8, 0)
        if pending is not None:
            pending.wait()


def _column_split(lib, dev, rank: int, world: int, dist, group, steps: int, reserve: int) -> dict:
    """Times the column-split step (with and without its two collectives, max over ranks) and checks that the gathered
    forward output equals, bit for bit, the forward of the whole weight matrix on one GPU."""
    case = _ColumnCase(lib, dev, rank, world, 4200)
    case.fwd_mine()
    case.gather(dist, group)
    whole = torch.empty(M_ROWS, N, dtype=torch.bfloat16, device=dev)
    ws = [torch.empty(int(lib.axs6_linear_workspace_bytes(i, M_ROWS, N, K)), dtype=torch.uint8, device=dev) for i in (0, 1)]
    st = lib.axs6_linear_fwd(case.x.data_ptr(), 1, K, case.w_full.data_ptr(), 0, K, torch.zeros(N, device=dev).data_ptr(),
                             whole.data_ptr(), 1, N, M_ROWS, N, K, BLOCK, 1, 1, ws[0].data_ptr(), ws[1].data_ptr(), case.stream)
    assert st == 0, st
    torch.cuda.synchronize()
    same = torch.tensor([1.0 if torch.equal(case.y, whole) else 0.0], dtype=torch.float64, device=dev)
    dist.all_reduce(same, op=dist.ReduceOp.MIN)
    del whole, ws

    def timed(collectives: bool, res: int) -> float:
        for i in range(3):
            case.step(i, dist, group, collectives, res)
        dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(steps):
            case.step(i, dist, group, collectives, res)
        e1.record()
        dist.barrier()
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1)], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item()) / steps

    def alone(fn) -> float:
        """One collective (or copy) by itself, max over ranks."""
        for _ in range(2):
            fn()
        dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1)], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item()) / steps

    flops = 6.0 * M_ROWS * N * K                                  # whole job: every rank does 1/world of it
    m_all, m_none = timed(True, reserve), timed(False, 0)
    phases = {"all_gather_y_ms": alone(lambda: dist.all_gather_into_tensor(case.y_blocks, case.y_mine)),
              "lay_blocks_side_by_side_ms": alone(case.lay_side_by_side),
              "all_reduce_dx_alone_ms": alone(lambda: dist.all_reduce(case.dx, group=group))}
    return {"columns_per_gpu": case.Nl, "rows": M_ROWS, "ms_per_step": m_all, "TFLOPs": flops / (m_all * 1e-3) / 1e12,
            "compute_only": {"ms_per_step": m_none, "TFLOPs": flops / (m_none * 1e-3) / 1e12},
            "gathered_forward_equals_one_gpu_forward": bool(same.item() == 1.0), "collectives_alone": phases,
            "collectives": f"all-gather of the (M, N/{world}) bf16 column blocks of y + one copy that lays them side by side; "
                           f"all-reduce of the bf16 partial dX ({M_ROWS}x{K}) under the dW product",
            "wire_bytes_per_rank": {"all_gather_y": M_ROWS * case.Nl * 2, "all_reduce_dx": M_ROWS * K * 2}}


def _rel(a, b) -> float:
    a, b = a.double(), b.double()
    return float((a - b).norm() / b.norm())


def _parity(case: _Case) -> dict:
    """One forward + backward, then 64 sampled rows of y, dX and dW against fp32 products (cuBLAS, TF32 off) of the
    quantised operands the step itself produced.  Tolerances: bf16 outputs 4e-3, fp32 dW 1e-3 (relative Frobenius)."""
    M = case.M
    case.fwd()
    case.bwd_all(0)
    torch.cuda.synchronize()
    prev = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    try:
        xq = case.xq.view(torch.bfloat16).view(M, K)
        wq = case.wq.view(torch.bfloat16).view(N, K)
        gq = case.gq.view(torch.bfloat16).view(M, N)
        g = torch.Generator(device="cpu").manual_seed(5)
        ri = torch.randperm(M, generator=g)[:64].to(xq.device)
        ni = torch.randperm(N, generator=g)[:64].to(xq.device)
        ey = _rel(case.y[ri].float(), xq[ri].float() @ wq.float().t() + case.bias.to(torch.bfloat16).float())
        edx = _rel(case.dx[ri].float(), gq[ri].float() @ wq.float())
        edw = _rel(case.dws[0][ni], gq[:, ni].float().t() @ xq.float())
        edb = _rel(case.db, case.go.float().sum(0))
    finally:
        torch.backends.cuda.matmul.allow_tf32 = prev
    ok = ey < 4e-3 and edx < 4e-3 and edw < 1e-3 and edb < 1e-4
    return {"parity_checked": bool(ok), "rel_err": {"y": ey, "dx": edx, "dw": edw, "db": edb},
            "against": "fp32 matmul (TF32 off) of the step's own quantised operands, 64 sampled rows per product"}


def _time_steps(case: _Case, steps: int, world: int, dist, group, allreduce: bool, reserve: int, lib, dev, warm: int = 3):
    """CUDA-event time per step, max over ranks; kernel launches of this library per step.  `warm` untimed steps come
    first (the variants compared with each other all take the same, longer warm-up, so that none is measured on a
    cooler GPU than the others)."""
    pending = [None, None]

    def step(i):
        case.fwd()
        if pending[i % 2] is not None:
            pending[i % 2].wait()
            pending[i % 2] = None
        if allreduce and world > 1:
            case.bwd_dw(i)
            pending[i % 2] = dist.all_reduce(case.dws[i % 2], group=group, async_op=True)
            if reserve:
                lib.axs6_tune(8, reserve)
            case.bwd_dx(i)
            if reserve:
                lib.axs6_tune(8, 0)
        else:
            case.bwd_all(i)

    def drain():
        for j in range(2):
            if pending[j] is not None:
                pending[j].wait()
                pending[j] = None

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for i in range(warm):
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
    t = torch.tensor([e0.elapsed_time(e1)], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item()) / steps, (_lib.launches() - l0) / steps


def _packed_variant(lib, dev, steps: int, t_of) -> dict:
    """The same step with AXS6_LINEAR_OPERANDS_PACKED, and its kernels alone (M = 16384, one GPU)."""
    M = M_ROWS
    c = _Case(lib, dev, M, 4000, packed=True)
    st = c.stream

    def step(i=[0]):
        c.fwd()
        c.bwd_all(i[0])
        i[0] += 1
    step()
    torch.cuda.synchronize()
    ms = t_of(step, max(5, steps // 2))
    off = lambda rows, cols: (rows * (cols // 32) * 24 + 255) // 256 * 256
    xq, wq, gq = c.xq.data_ptr(), c.wq.data_ptr(), c.gq.data_ptr()
    xe, we, ge = xq + off(M, K), wq + off(N, K), gq + off(M, N)
    fl = 2.0 * M * N * K
    out = {"ms_per_step": ms, "TFLOPs": 3 * fl / (ms * 1e-3) / 1e12, "parts": {}}
    gf = lambda: lib.axs6_gemm_packed(xq, xe, 0, wq, we, 0, c.y.data_ptr(), None, M, N, K, N, 0, 0, 1, st)
    gdx = lambda: lib.axs6_gemm_packed(gq, ge, 0, wq, we, 0, c.dx.data_ptr(), None, M, K, N, K, 0, 1, 1, st)
    gdw = lambda: lib.axs6_gemm_packed(gq, ge, 0, xq, xe, 0, c.dws[0].data_ptr(), None, N, K, M, K, 1, 1, 0, st)
    for name, fn in (("gemm_fwd", gf), ("gemm_dx", gdx), ("gemm_dw", gdw)):
        assert fn() == 0
        m = t_of(fn)
        out["parts"][name] = {"ms": m, "TFLOPs": fl / (m * 1e-3) / 1e12}
    px = lambda: lib.axs6_pack(c.x.data_ptr(), 1, M, K, K, 32, 1, 0, 1, 0, 0, None, 3, xq, xe, None, st)
    pw = lambda: lib.axs6_pack(c.w.data_ptr(), 0, N, K, K, 32, 1, 0, 1, 0, 0, None, 3, wq, we, None, st)
    pg = lambda: lib.axs6_pack(c.go.data_ptr(), 1, M, N, N, 32, 1, 1, 1, 7, 0, None, 3, gq, ge, None, st)
    for name, fn, nb in (("pack_x", px, M * K * 2.78125), ("pack_w", pw, N * K * 4.78125), ("pack_g_stochastic", pg, M * N * 2.78125)):
        assert fn() == 0
        m = t_of(fn)
        out["parts"][name] = {"ms": m, "GBps": nb / (m * 1e-3) / 1e9}
    # only W as codes (activations and gradient stay bf16 tiles fed by TMA)
    bx = torch.empty(M, K, dtype=torch.bfloat16, device=dev)
    gw = lambda: lib.axs6_gemm_packed(bx.data_ptr(), None, K, wq, we, 0, c.y.data_ptr(), None, M, N, K, N, 0, 0, 1, st)
    assert gw() == 0
    m = t_of(gw)
    out["parts"]["gemm_fwd_only_w_packed"] = {"ms": m, "TFLOPs": fl / (m * 1e-3) / 1e12}
    # the cheap way to the same saved-activation size: records written beside the bf16 path, unpacked in backward
    rec = torch.empty(M * (K // 32) * 25, dtype=torch.uint8, device=dev)
    pr = lambda: lib.axs6_pack(c.x.data_ptr(), 1, M, K, K, 32, 1, 0, 0, 0, 0, None, 1, rec.data_ptr(), None, None, st)
    ur = lambda: lib.axs6_unpack(1, rec.data_ptr(), None, None, bx.data_ptr(), 1, M, K, K, 32, 1, st)
    assert pr() == 0 and ur() == 0
    m_p, m_u = t_of(pr), t_of(ur)
    out["saved_activation_as_records"] = {
        "pack_ms": m_p, "unpack_ms": m_u, "bytes_saved_for_backward": int(rec.numel()), "bf16_bytes": M * K * 2,
        "note": "mixed_precision.SAVE_PACKED_INPUT: the default step plus one pack (forward) and one unpack (backward) of the "
                "activation; the saved tensor shrinks 2.56x without the decode-on-load GEMM"}
    out["gemm_status"] = int(lib.axs6_gemm_status())
    out["note"] = ("activations, weight and gradient written to HBM as 6-bit codes (0.78 bytes per value) by axs6_pack and decoded "
                   "to bf16 by the decode warps of axs6_gemm_packed; compare with `parts` (bf16 workspaces + plain GEMM)")
    return out


def _fp32_graph(dev, t_of) -> dict:
    """axs_linear_unified forward + backward at the same size with fp32 tensors (one GPU)."""
    import importlib
    fu = importlib.import_module("axs6_b200.unified.functional_unified")
    g = torch.Generator(device=dev).manual_seed(4200)
    x = torch.randn(M_ROWS, K, generator=g, device=dev).requires_grad_(True)
    w = (torch.randn(N, K, generator=g, device=dev) * 0.02).requires_grad_(True)
    b = torch.zeros(N, device=dev, requires_grad=True)
    go = torch.randn(M_ROWS, N, generator=g, device=dev)

    def step():
        x.grad = w.grad = b.grad = None
        fu.axs_linear_unified(x, w, b).backward(go)

    ms = t_of(step, 5)
    return {"ms_per_step": ms, "TFLOPs": 6.0 * M_ROWS * N * K / (ms * 1e-3) / 1e12,
            "workload": f"axs_linear_unified forward + backward, M={M_ROWS}, K={K}, N={N}, fp32 tensors: fake-quantise in fp32, "
                        "forward as three TF32 products (fp32 accuracy), backward products in TF32"}


def run(args, rank: int, world: int, dev, pk: dict, steps: int | None = None) -> dict:
    import torch.distributed as dist
    lib = _lib.load()
    steps = steps or max(5, min(args.steps, 20))
    weak = _Case(lib, dev, M_ROWS, 4000 + rank)
    parity = _parity(weak) if rank == 0 else {}
    flops_weak = 6.0 * M_ROWS * N * K

    # a process group of its own whose collective kernels use few CTAs, so that they fit beside the GEMM
    group, nccl_ctas = None, None
    if world > 1:
        try:
            opts = dist.ProcessGroupNCCL.Options()
            opts.config.max_ctas = 16
            opts.config.min_ctas = 1
            group = dist.new_group(ranks=list(range(world)), pg_options=opts)
            nccl_ctas = 16
        except Exception:
            group = None

    res = {}
    # SMs the dX product leaves to the all-reduce that runs beside it.  32 was the best value in every interleaved sweep
    # on 4 GPUs (see `reserved_sm_sweep` below): with fewer, the collective's CTAs do not all fit beside the persistent
    # GEMM grid, finish after it and hold SMs that the next GEMM's statically assigned clusters then wait for.
    reserve, sweep = (32 if world > 1 else 0), None
    ms, launches = _time_steps(weak, steps, world, dist, group, True, reserve, lib, dev)
    res_weak = {"ms_per_step": ms, "TFLOPs": world * flops_weak / (ms * 1e-3) / 1e12, "rows_per_gpu": M_ROWS}
    if world > 1:
        # Evidence for that choice, measured AFTER the headline so that the headline runs on a GPU in the same state as
        # the one-GPU run: the candidates (and the step with the all-reduce off) timed in turn, three rounds of 10
        # steps each, so that clock and temperature drift hits them all alike.
        import statistics
        cands = [0, 16, 24, 32, 40, 48]
        times = {str(n): [] for n in cands}
        times["allreduce_off"] = []
        for _ in range(3):
            for n in cands:
                times[str(n)].append(_time_steps(weak, 10, world, dist, group, True, n, lib, dev, warm=2)[0])
            times["allreduce_off"].append(_time_steps(weak, 10, world, dist, group, False, 0, lib, dev, warm=2)[0])
        med = {k: statistics.median(v) for k, v in times.items()}
        sweep = {"median_ms_per_step": med, "all_ms_per_step": times,
                 "note": "interleaved: 3 rounds x (reserved SMs 0, 16, 24, 32, 40, 48, all-reduce off) x 10 steps, after the headline"}
        res_weak["reserved_sms"] = reserve
        res_weak["reserved_sm_sweep"] = sweep
    status = int(lib.axs6_gemm_status())

    # the three GEMMs and the fake-quantise passes alone, and the library GEMM (cuBLAS through torch.matmul) on the
    # same quantised bf16 operands in the same process
    parts = {}
    if rank == 0:
        c, M = weak, M_ROWS
        stream = c.stream
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)

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
        xq, wq, gq = c.xq, c.wq, c.gq
        gf = lambda: lib.axs6_gemm_bf16(xq.data_ptr(), wq.data_ptr(), c.y.data_ptr(), None, M, N, K, K, K, N, 0, 0, 1, stream)
        gdx = lambda: lib.axs6_gemm_bf16(gq.data_ptr(), wq.data_ptr(), c.dx.data_ptr(), None, M, K, N, N, K, K, 0, 1, 1, stream)
        gdw = lambda: lib.axs6_gemm_bf16(gq.data_ptr(), xq.data_ptr(), c.dws[0].data_ptr(), None, N, K, M, N, K, K, 1, 1, 0, stream)
        fqx = lambda: lib.axs6_fq(c.x.data_ptr(), xq.data_ptr(), 1, 1, M, K, K, K, BLOCK, 1, 0, 1, 0, 0, stream)
        fqw = lambda: lib.axs6_fq(c.w.data_ptr(), wq.data_ptr(), 0, 1, N, K, K, K, BLOCK, 1, 0, 1, 0, 0, stream)
        fqg = lambda: lib.axs6_fq(c.go.data_ptr(), gq.data_ptr(), 1, 1, M, N, N, N, BLOCK, 1, 1, 1, 7, 0, stream)
        dbs = lambda: lib.axs6_bias_grad(c.go.data_ptr(), 1, N, M, N, c.db.data_ptr(), c.part.data_ptr(), stream)
        txq, twq, tgq = (t.view(torch.bfloat16) for t in (xq, wq, gq))
        txq, twq, tgq = txq.view(M, K), twq.view(N, K), tgq.view(M, N)
        ty, tdx, tdw = torch.empty_like(c.y), torch.empty_like(c.dx), torch.empty(N, K, dtype=torch.bfloat16, device=dev)
        lib_f = lambda: torch.matmul(txq, twq.t(), out=ty)
        lib_dx = lambda: torch.matmul(tgq, twq, out=tdx)
        lib_dw = lambda: torch.matmul(tgq.t(), txq, out=tdw)
        fl = 2.0 * M * N * K
        for name, fn, lfn in (("gemm_fwd", gf, lib_f), ("gemm_dx", gdx, lib_dx), ("gemm_dw", gdw, lib_dw)):
            m = t_of(fn)
            ml = t_of(lfn)
            parts[name] = {"ms": m, "TFLOPs": fl / (m * 1e-3) / 1e12,
                           "library_ms": ml, "library_TFLOPs": fl / (ml * 1e-3) / 1e12, "vs_library": ml / m}
        for name, fn, nb in (("fq_x", fqx, M * K * 4), ("fq_w", fqw, N * K * 6), ("fq_g_stochastic", fqg, M * N * 4),
                             ("bias_grad", dbs, M * N * 2)):
            m = t_of(fn)
            parts[name] = {"ms": m, "GBps": nb / (m * 1e-3) / 1e9}
        parts["library"] = "torch.matmul (cuBLAS) on the same quantised bf16 operands, bf16 output, same process"
        del ty, tdx, tdw
    best = max((v["TFLOPs"] for k, v in parts.items() if k.startswith("gemm")), default=0.0)
    del weak
    torch.cuda.empty_cache()

    # the quantise-on-load variant: operands in HBM as 6-bit codes, decoded to bf16 inside the GEMMs
    packed = None
    if rank == 0:
        try:
            packed = _packed_variant(lib, dev, steps, t_of)
        except Exception as e:
            packed = {"error": repr(e)}
        torch.cuda.empty_cache()

    # the fp32 graph of the same layer (the unified Linear: fp32 in / out, fp32-accurate forward through three TF32
    # products, TF32 backward products), through the Python operator
    fp32_graph = None
    if rank == 0:
        try:
            fp32_graph = _fp32_graph(dev, t_of)
        except Exception as e:
            fp32_graph = {"error": repr(e)[:300]}
        torch.cuda.empty_cache()

    strong = None
    if world > 1:
        Ms = M_ROWS // world
        sc = _Case(lib, dev, Ms, 4100 + rank)
        flops_strong = 6.0 * M_ROWS * N * K                 # whole job
        m_s, _ = _time_steps(sc, steps, world, dist, group, True, reserve, lib, dev)
        m_c, _ = _time_steps(sc, steps, world, dist, group, False, 0, lib, dev)
        strong = {"rows_per_gpu": Ms, "ms_per_step": m_s, "TFLOPs": flops_strong / (m_s * 1e-3) / 1e12,
                  "compute_only": {"ms_per_step": m_c, "TFLOPs": flops_strong / (m_c * 1e-3) / 1e12,
                                   "note": "the same sharded step with the dW all-reduce switched off"}}
        del sc
        torch.cuda.empty_cache()
        try:
            strong["column_split"] = _column_split(lib, dev, rank, world, dist, group, steps, reserve)
        except Exception as e:
            strong["column_split"] = {"error": repr(e)[:300]}
        torch.cuda.empty_cache()

    tflops = res_weak["TFLOPs"]
    out = {
        "metric": "axs6_linear_fwd_bwd_TFLOPs", "value": tflops, "unit": "TFLOP/s", "ms_per_step": res_weak["ms_per_step"],
        "steps": steps, "n_gpus": world, "scaling": "weak", "gpu_launches": launches * steps, "gemm_status": status,
        "workload": (f"AXS-6 Linear fwd+bwd, M={M_ROWS} rows per GPU, K={K}, N={N}, bf16 activations, fp32 master weights, "
                     f"block {BLOCK} along K, stochastic gradient rounding" +
                     (", dW all-reduced over NCCL under the dX product" if world > 1 else "")),
        "algorithmic_flops_per_step": flops_weak,
        "roofline": {"bound": "tensor", "achieved": tflops / world, "peak": pk["bf16_tflops_sustained"], "unit": "TFLOP/s",
                     "frac": tflops / world / pk["bf16_tflops_sustained"], "peak_burst": pk["bf16_tflops"],
                     "frac_of_burst": tflops / world / pk["bf16_tflops"], "peak_source": pk["source"],
                     "note": "whole step (fake-quantise passes + 3 GEMMs + column sums) over 6*M*N*K flops, against the "
                             "sustained cuBLAS bf16 figure; per-kernel figures in `parts`"},
        "best_gemm_TFLOPs": best,
        "parts": parts,
        "weak": res_weak,
    }
    out.update(parity)
    if packed is not None:
        out["operands_packed"] = packed
    if fp32_graph is not None:
        out["fp32_graph"] = fp32_graph
    if strong is not None:
        out["strong"] = strong
        out["nccl_max_ctas"] = nccl_ctas
    return out
