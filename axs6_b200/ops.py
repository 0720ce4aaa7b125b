"""Tensor-level wrappers over the C ABI: argument checking, views, output allocation.

Everything here is host plumbing; all arithmetic happens in the CUDA library.  Inputs must be
CUDA tensors (fp32 or bf16); a CPU tensor raises ``RuntimeError`` -- there is no CPU path.
"""
from __future__ import annotations

import torch

from . import _lib
from ._lib import (BF16, F32, FLAG_INPUT_VIA_BF16, GRID_NF5, GRID_UNIFORM, LAYOUT_PLANES, LAYOUT_SPEC,
                   LAYOUT_WIRE, ROUND_NEAREST, ROUND_STOCHASTIC)

VALID_BLOCK_SIZES = (8, 16, 32)
_DT = {torch.float32: F32, torch.bfloat16: BF16}

# Stochastic rounding: Philox stream keyed by torch's seed; the counter advances by the
# number of draws of every call, so no two calls of a process reuse a draw and no device
# sync is needed (the reference draws a seed with .item(), which synchronises).
_philox_offset = 0


def next_philox(n_draws: int) -> tuple[int, int]:
    global _philox_offset
    off = _philox_offset
    _philox_offset += (n_draws + 7) // 8
    return torch.initial_seed() & 0xFFFFFFFFFFFFFFFF, off


def philox_offset() -> int:
    """The host-side Philox counter (what the next stochastic call starts from)."""
    return _philox_offset


def reset_philox(offset: int = 0) -> None:
    global _philox_offset
    _philox_offset = offset


def philox_advance(delta: int = 1 << 40, reset: bool = False, device=None) -> None:
    """Enqueue ``epoch += delta`` for the device-resident addend of every stochastic kernel's counter
    (see ``axs6_philox_advance``): call it at the start of a step that is captured in a CUDA graph."""
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    with _on(dev):
        st = _lib.load().axs6_philox_advance(delta, int(reset), _stream(dev))
    _lib.check("axs6_philox_advance", st)


def philox_epoch(device=None) -> int:
    """The device-resident epoch that ``philox_advance`` maintains (one 8-byte read; synchronises the device)."""
    import ctypes
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    out = ctypes.c_uint64(0)
    with _on(dev):
        st = _lib.load().axs6_philox_epoch(ctypes.byref(out))
    _lib.check("axs6_philox_epoch", st)
    return int(out.value)


def set_philox_epoch(value: int, device=None) -> None:
    """Restore a saved epoch: reset, then advance by ``value``."""
    philox_advance(0, reset=True, device=device)
    if value:
        philox_advance(int(value), device=device)


def _rounding(rounding: str) -> int:
    if rounding == "nearest":
        return ROUND_NEAREST
    if rounding == "stochastic":
        return ROUND_STOCHASTIC
    raise ValueError(f"Unknown rounding mode: {rounding}")


def _check_input(t: torch.Tensor, who: str) -> None:
    if not isinstance(t, torch.Tensor):
        raise TypeError(f"{who} expects a torch.Tensor")
    if not t.is_cuda:
        raise RuntimeError(f"{who} requires a CUDA tensor")
    if t.dim() == 0:
        raise ValueError(f"{who} needs at least one dimension")


def _as_rows(t: torch.Tensor) -> tuple[torch.Tensor, int, int, int]:
    """-> (2-D view or copy with unit inner stride, rows, cols, leading dimension)."""
    if t.dtype not in _DT:
        t = t.float()
    cols = t.shape[-1]
    if t.numel() == 0:
        rows = 1
        for d in t.shape[:-1]:
            rows *= d
        return t.new_empty((rows, cols)), rows, cols, cols
    t2 = t.reshape(-1, cols)
    rows, cols = t2.shape
    if cols > 0 and rows > 0 and (t2.stride(1) != 1 or (rows > 1 and t2.stride(0) < cols)):
        t2 = t2.contiguous()
    ld = t2.stride(0) if rows > 1 else cols
    return t2, rows, cols, max(ld, cols)


def _stream(dev: torch.device) -> int:
    return torch.cuda.current_stream(dev).cuda_stream


class _on:
    """Make `dev` current for the duration of a call (the library works on the current device)."""

    def __init__(self, dev: torch.device):
        self.dev = dev
        self.prev = None

    def __enter__(self):
        if self.dev.index is not None:
            cur = torch.cuda.current_device()
            if self.dev.index != cur:
                self.prev = cur
                torch.cuda.set_device(self.dev)

    def __exit__(self, *exc):
        if self.prev is not None:
            torch.cuda.set_device(self.prev)


def fake_quantize(x: torch.Tensor, block_size: int = 32, grid: int = GRID_NF5, rounding: str = "nearest",
                  out_dtype: torch.dtype | None = None, via_bf16: bool = False,
                  noise: torch.Tensor | None = None, who: str = "fake_quantize") -> torch.Tensor:
    """One-pass fake-quantise of the last dimension in blocks; returns a new tensor."""
    _check_input(x, who)
    assert block_size in VALID_BLOCK_SIZES, f"block_size must be one of {VALID_BLOCK_SIZES}"
    if x.dtype not in _DT and x.is_floating_point():       # fp16, fp64: the kernels read fp32 / bf16 only
        y = fake_quantize(x.float(), block_size, grid, rounding, out_dtype, via_bf16, noise, who)
        return y if out_dtype is not None else y.to(x.dtype)
    rnd = _rounding(rounding)
    x2, rows, cols, ldx = _as_rows(x)
    odt = out_dtype if out_dtype is not None else (x.dtype if x.dtype in _DT else torch.float32)
    y = torch.empty((rows, cols), dtype=odt, device=x.device)
    lib = _lib.load()
    flags = FLAG_INPUT_VIA_BF16 if (via_bf16 and x2.dtype == torch.float32) else 0
    with _on(x.device):
        if noise is not None:
            nz = noise.to(device=x.device, dtype=torch.float32).contiguous()
            st = lib.axs6_fq_with_noise(x2.data_ptr(), y.data_ptr(), _DT[x2.dtype], _DT[odt], rows, cols, ldx, cols,
                                        block_size, grid, flags, nz.data_ptr(), _stream(x.device))
            _lib.check("axs6_fq_with_noise", st)
        else:
            seed, off = (0, 0)
            if rnd == ROUND_STOCHASTIC:
                seed, off = next_philox(rows * (-(-cols // block_size)) * block_size)
            st = lib.axs6_fq(x2.data_ptr(), y.data_ptr(), _DT[x2.dtype], _DT[odt], rows, cols, ldx, cols,
                             block_size, grid, rnd, flags, seed, off, _stream(x.device))
            _lib.check("axs6_fq", st)
    return y.reshape(x.shape)


def fake_quantize_gather(table: torch.Tensor, index: torch.Tensor, block_size: int = 32, grid: int = GRID_NF5,
                         rounding: str = "nearest", out_dtype: torch.dtype | None = None,
                         who: str = "fake_quantize_gather") -> torch.Tensor:
    """``fake_quantize(table[index])`` in one pass: the looked-up rows are never written to HBM unquantised.
    ``table`` (rows, cols) fp32 / bf16 with unit inner stride, ``index`` any shape of integers; returns
    ``index.shape + (cols,)``.  An index outside the table raises (after the launch, like torch's device assert)."""
    _check_input(table, who)
    _check_input(index, who)
    assert block_size in VALID_BLOCK_SIZES, f"block_size must be one of {VALID_BLOCK_SIZES}"
    assert table.dim() == 2 and table.dtype in _DT
    t2 = table if table.stride(1) == 1 else table.contiguous()
    idx = index.reshape(-1).to(torch.int64).contiguous()
    rows, cols = idx.numel(), t2.shape[1]
    odt = out_dtype if out_dtype is not None else t2.dtype
    y = torch.empty((rows, cols), dtype=odt, device=table.device)
    rnd = _rounding(rounding)
    seed, off = (0, 0)
    if rnd == ROUND_STOCHASTIC:
        seed, off = next_philox(rows * (-(-cols // block_size)) * block_size)
    lib = _lib.load()
    with _on(table.device):
        st = lib.axs6_fq_gather(t2.data_ptr(), t2.shape[0], idx.data_ptr(), y.data_ptr(), _DT[t2.dtype], _DT[odt], rows, cols,
                                t2.stride(0) if t2.shape[0] > 1 else cols, cols, block_size, grid, rnd, seed, off,
                                _stream(table.device))
    _lib.check("axs6_fq_gather", st)
    return y.reshape(*index.shape, cols)


def gather_index_error() -> bool:
    """True once after a ``fake_quantize_gather`` launch met an index outside its table (synchronises)."""
    return bool(_lib.load().axs6_fq_gather_status())


def unpack_sum(layout: int, buf: torch.Tensor, nsrc: int, src_stride: int, rows: int, cols: int, block_size: int = 32,
               grid: int = GRID_NF5, out_dtype: torch.dtype = torch.float32, divisor: float = 1.0,
               out: torch.Tensor | None = None) -> torch.Tensor:
    """(sum of the ``nsrc`` record buffers' reconstructions) / divisor in one pass; source ``s`` starts at byte
    ``s * src_stride`` of ``buf``.  Summed in fp32 in source order, like unpacking one by one and adding.
    ``out``: a contiguous fp32 / bf16 tensor of rows * cols values to write into instead of a new one."""
    assert block_size in VALID_BLOCK_SIZES, f"block_size must be one of {VALID_BLOCK_SIZES}"
    _check_input(buf, "unpack_sum")
    buf = buf.contiguous()
    nblk = -(-cols // block_size)
    need = rows * nblk * record_bytes(layout, block_size)
    if nsrc < 1 or (nsrc > 1 and src_stride < need) or buf.numel() * buf.element_size() < (nsrc - 1) * src_stride + need:
        raise ValueError(f"buffer of {buf.numel() * buf.element_size()} bytes does not hold {nsrc} sources of {need} bytes "
                         f"at stride {src_stride}")
    if out is not None:
        if out.dtype not in _DT or out.device != buf.device or not out.is_contiguous() or out.numel() != rows * cols:
            raise ValueError("out must be a contiguous fp32 or bf16 tensor of rows * cols values on the records' device")
        y, out_dtype = out.view(rows, cols), out.dtype
    else:
        y = torch.empty((rows, cols), dtype=out_dtype, device=buf.device)
    with _on(buf.device):
        st = _lib.load().axs6_unpack_sum(layout, buf.data_ptr(), nsrc, src_stride, y.data_ptr(), _DT[out_dtype], rows, cols,
                                         cols, block_size, grid, float(divisor), _stream(buf.device))
    _lib.check("axs6_unpack_sum", st)
    return y


# ---------------------------------------------------------------------------------- host buffers
# Fake-quantise of a tensor that lives in pinned HOST memory: rows are cut into chunks (blocks never cross a
# row) that flow through a ring of device buffers on three streams -- host->device copy, kernel, device->host
# copy -- so that the two PCIe directions run at the same time and the kernel hides under the copies.
_HOST_RING: dict = {}


def _host_ring(dev: torch.device, in_dtype: torch.dtype, out_dtype: torch.dtype, chunk_elems: int, depth: int):
    key = (dev.index, in_dtype, out_dtype, depth)
    ring = _HOST_RING.get(key)
    if ring is None or ring["elems"] < chunk_elems:
        ring = {"elems": chunk_elems,
                "x": [torch.empty(chunk_elems, dtype=in_dtype, device=dev) for _ in range(depth)],
                "y": [torch.empty(chunk_elems, dtype=out_dtype, device=dev) for _ in range(depth)],
                "s_in": torch.cuda.Stream(dev), "s_k": torch.cuda.Stream(dev), "s_out": torch.cuda.Stream(dev)}
        _HOST_RING[key] = ring
    return ring


def fake_quantize_host(src: torch.Tensor, dst: torch.Tensor | None = None, block_size: int = 32, grid: int = GRID_NF5,
                       rounding: str = "nearest", device=None, chunk_bytes: int = 32 << 20, depth: int = 3) -> torch.Tensor:
    """``dst = fake_quantize(src)`` for PINNED host tensors (fp32 or bf16, same shape; ``dst`` is allocated pinned
    when omitted), computed on the GPU in chunks of about ``chunk_bytes`` with the copies in both directions and
    the kernel overlapped.  Returns ``dst`` after the last copy has been enqueued; the current stream of
    ``device`` waits for it, so ``torch.cuda.current_stream().synchronize()`` (or any later work on that
    stream) sees the finished result."""
    if not isinstance(src, torch.Tensor) or src.is_cuda:
        raise TypeError("fake_quantize_host expects a host tensor; use fake_quantize for device tensors")
    if src.dtype not in _DT:
        raise TypeError("fake_quantize_host takes fp32 or bf16 tensors")
    if dst is None:
        dst = torch.empty(src.shape, dtype=src.dtype, pin_memory=True)
    if dst.is_cuda or dst.shape != src.shape or dst.dtype not in _DT:
        raise ValueError("dst must be a host tensor of the same shape, fp32 or bf16")
    if not (src.is_pinned() and dst.is_pinned() and src.is_contiguous() and dst.is_contiguous()):
        raise ValueError("fake_quantize_host needs contiguous pinned host tensors (tensor.pin_memory())")
    assert block_size in VALID_BLOCK_SIZES, f"block_size must be one of {VALID_BLOCK_SIZES}"
    rnd = _rounding(rounding)
    if src.dim() == 0:
        raise ValueError("fake_quantize_host needs at least one dimension")
    if src.numel() == 0:
        return dst
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    cols = src.shape[-1]
    rows = src.numel() // cols
    s2, d2 = src.view(rows, cols), dst.view(rows, cols)
    rows_per_chunk = max(1, min(rows, chunk_bytes // max(1, cols * src.element_size())))
    ring = _host_ring(dev, src.dtype, dst.dtype, rows_per_chunk * cols, depth)
    lib = _lib.load()
    main = torch.cuda.current_stream(dev)
    s_in, s_k, s_out = ring["s_in"], ring["s_k"], ring["s_out"]
    start = torch.cuda.Event()
    start.record(main)
    for st in (s_in, s_k, s_out):
        st.wait_event(start)                              # whatever produced src on the caller's stream is done
    s_in.wait_stream(s_k)                                 # and so is an earlier call that used the ring from
    s_in.wait_stream(s_out)                               # another stream of the caller
    s_k.wait_stream(s_out)
    x_free = [None] * depth                               # kernel that last read x[b]
    y_free = [None] * depth                               # copy that last read y[b]
    nblk = -(-cols // block_size)
    with _on(dev):
        for i, r0 in enumerate(range(0, rows, rows_per_chunk)):
            b = i % depth
            r1 = min(rows, r0 + rows_per_chunk)
            n = (r1 - r0) * cols
            xb, yb = ring["x"][b][:n], ring["y"][b][:n]
            if x_free[b] is not None:
                s_in.wait_event(x_free[b])
            with torch.cuda.stream(s_in):
                xb.copy_(s2[r0:r1].reshape(-1), non_blocking=True)
                ev_in = torch.cuda.Event()
                ev_in.record(s_in)
            s_k.wait_event(ev_in)
            if y_free[b] is not None:
                s_k.wait_event(y_free[b])
            seed, off = (0, 0)
            if rnd == ROUND_STOCHASTIC:
                seed, off = next_philox((r1 - r0) * nblk * block_size)
            st_code = lib.axs6_fq(xb.data_ptr(), yb.data_ptr(), _DT[src.dtype], _DT[dst.dtype], r1 - r0, cols, cols, cols,
                                  block_size, grid, rnd, 0, seed, off, s_k.cuda_stream)
            _lib.check("axs6_fq", st_code)
            ev_k = torch.cuda.Event()
            ev_k.record(s_k)
            x_free[b] = ev_k
            s_out.wait_event(ev_k)
            with torch.cuda.stream(s_out):
                d2[r0:r1].reshape(-1).copy_(yb, non_blocking=True)
                ev_out = torch.cuda.Event()
                ev_out.record(s_out)
            y_free[b] = ev_out
    main.wait_stream(s_out)
    return dst


def pack_error_feedback(x: torch.Tensor, err: torch.Tensor, block_size: int = 32, grid: int = GRID_UNIFORM,
                        rounding: str = "nearest"):
    """Planes of ``x + err`` and ``err <- (x + err) - reconstruction`` in ONE kernel, or None when the tensors do not
    qualify (fp32, contiguous, same shape, last dimension a multiple of 8): the caller then composes the steps."""
    if not (x.is_cuda and err.is_cuda and x.dtype == torch.float32 and err.dtype == torch.float32 and x.shape == err.shape
            and x.dim() >= 1 and x.is_contiguous() and err.is_contiguous() and x.shape[-1] % 8 == 0 and x.numel() > 0):
        return None
    assert block_size in VALID_BLOCK_SIZES, f"block_size must be one of {VALID_BLOCK_SIZES}"
    cols = x.shape[-1]
    rows = x.numel() // cols
    nblk = -(-cols // block_size)
    se = torch.empty((rows, nblk), dtype=torch.uint8, device=x.device)
    sg = torch.empty((rows, nblk, block_size), dtype=torch.bool, device=x.device)
    mg = torch.empty((rows, nblk, block_size), dtype=torch.uint8, device=x.device)
    rnd = _rounding(rounding)
    seed, off = (0, 0)
    if rnd == ROUND_STOCHASTIC:
        seed, off = next_philox(rows * nblk * block_size)
    with _on(x.device):
        st = _lib.load().axs6_pack_ef(x.data_ptr(), err.data_ptr(), rows, cols, cols, block_size, grid, rnd, seed, off,
                                      se.data_ptr(), sg.data_ptr(), mg.data_ptr(), _stream(x.device))
    if st == -6:          # AXS6_ERR_UNSUPPORTED: misaligned pointers
        return None
    _lib.check("axs6_pack_ef", st)
    return se, sg, mg


def record_bytes(layout: int, block_size: int) -> int:
    return int(_lib.load().axs6_record_bytes(layout, block_size))


def pack(x: torch.Tensor, block_size: int = 32, grid: int = GRID_NF5, rounding: str = "nearest",
         layout: int = LAYOUT_PLANES, via_bf16: bool = False, noise: torch.Tensor | None = None,
         who: str = "pack", out: torch.Tensor | None = None):
    """Quantise to codes.  PLANES -> (exponents u8 (rows, nblk), signs bool (rows, nblk, B),
    magnitudes u8 (rows, nblk, B)); WIRE / SPEC -> flat uint8 tensor of block records (written into
    ``out`` when given: a contiguous uint8 tensor on the same device with room for the records)."""
    _check_input(x, who)
    assert block_size in VALID_BLOCK_SIZES, f"block_size must be one of {VALID_BLOCK_SIZES}"
    rnd = _rounding(rounding)
    x2, rows, cols, ldx = _as_rows(x)
    nblk = -(-cols // block_size)
    dev = x.device
    flags = FLAG_INPUT_VIA_BF16 if (via_bf16 and x2.dtype == torch.float32) else 0
    if layout == LAYOUT_PLANES:
        se = torch.empty((rows, nblk), dtype=torch.uint8, device=dev)
        sg = torch.empty((rows, nblk, block_size), dtype=torch.bool, device=dev)
        mg = torch.empty((rows, nblk, block_size), dtype=torch.uint8, device=dev)
        outs = (se, sg, mg)
        ptrs = (se.data_ptr(), sg.data_ptr(), mg.data_ptr())
    else:
        need = rows * nblk * record_bytes(layout, block_size)
        if out is not None:
            if out.dtype != torch.uint8 or out.device != dev or not out.is_contiguous() or out.numel() < need:
                raise ValueError(f"out must be a contiguous uint8 tensor on {dev} with at least {need} bytes")
            buf = out
        else:
            buf = torch.empty(need, dtype=torch.uint8, device=dev)
        outs = buf
        ptrs = (buf.data_ptr(), None, None)
    nz = None
    seed, off = 0, 0
    if rnd == ROUND_STOCHASTIC:
        if noise is not None:
            nz = noise.to(device=dev, dtype=torch.float32).contiguous()
        else:
            seed, off = next_philox(rows * nblk * block_size)
    with _on(dev):
        st = _lib.load().axs6_pack(x2.data_ptr(), _DT[x2.dtype], rows, cols, ldx, block_size, grid, rnd, flags,
                                   seed, off, nz.data_ptr() if nz is not None else None, layout,
                                   ptrs[0], ptrs[1], ptrs[2], _stream(dev))
    _lib.check("axs6_pack", st)
    return outs


def unpack(layout: int, parts, rows: int, cols: int, block_size: int = 32, grid: int = GRID_NF5,
           out_dtype: torch.dtype = torch.float32) -> torch.Tensor:
    """Codes back to values, (rows, cols)."""
    assert block_size in VALID_BLOCK_SIZES, f"block_size must be one of {VALID_BLOCK_SIZES}"
    if layout == LAYOUT_PLANES:
        se, sg, mg = parts
        for t in (se, sg, mg):
            _check_input(t, "unpack")
        se, sg, mg = se.contiguous(), sg.contiguous(), mg.contiguous()
        dev = mg.device
        ptrs = (se.data_ptr(), sg.data_ptr(), mg.data_ptr())
        keep = (se, sg, mg)
    else:
        buf = parts
        _check_input(buf, "unpack")
        buf = buf.contiguous()
        nblk = -(-cols // block_size)
        need = rows * nblk * record_bytes(layout, block_size)
        if buf.numel() * buf.element_size() < need:
            raise ValueError(f"buffer holds {buf.numel() * buf.element_size()} bytes, {need} needed")
        dev = buf.device
        ptrs = (buf.data_ptr(), None, None)
        keep = (buf,)
    y = torch.empty((rows, cols), dtype=out_dtype, device=dev)
    with _on(dev):
        st = _lib.load().axs6_unpack(layout, ptrs[0], ptrs[1], ptrs[2], y.data_ptr(), _DT[out_dtype], rows, cols,
                                     cols, block_size, grid, _stream(dev))
    _lib.check("axs6_unpack", st)
    del keep
    return y


# ------------------------------------------------------------------------------------------ linear
def gemm_bf16(a: torch.Tensor, b: torch.Tensor, bias: torch.Tensor | None = None, a_mn: bool = False,
              b_mn: bool = False, out_dtype: torch.dtype = torch.float32) -> torch.Tensor:
    """C = op(A) op(B) on the tensor cores.  ``a`` is (M, K) (or (K, M) with ``a_mn``), ``b`` is
    (N, K) (or (K, N) with ``b_mn``); 2-D, unit inner stride; both bf16 (bf16 tensor cores) or both
    fp32 (consumed as TF32)."""
    _check_input(a, "gemm_bf16")
    _check_input(b, "gemm_bf16")
    assert a.dtype == b.dtype and a.dtype in (torch.bfloat16, torch.float32) and a.dim() == 2 and b.dim() == 2
    if a.dtype == torch.float32:          # the TF32 instruction takes K-major operands only
        if a_mn:
            a, a_mn = transpose_f32(a), False
        if b_mn:
            b, b_mn = transpose_f32(b), False
    per16 = 16 // a.element_size()
    if a.stride(1) != 1 or a.stride(0) % per16 or a.data_ptr() % 16:
        a = _padded_copy(a)
    if b.stride(1) != 1 or b.stride(0) % per16 or b.data_ptr() % 16:
        b = _padded_copy(b)
    M, K = (a.shape[1], a.shape[0]) if a_mn else a.shape
    N, K2 = (b.shape[1], b.shape[0]) if b_mn else b.shape
    assert K == K2, "contraction lengths differ"
    c = torch.empty((M, N), dtype=out_dtype, device=a.device)
    bias_f = None
    if bias is not None:
        bias_f = bias.to(device=a.device, dtype=torch.float32).contiguous()
    lib = _lib.load()
    with _on(a.device):
        # fp32 results of bf16 products with few output tiles: a workspace lets the library split the contraction
        # more than two ways and still add the partials in a fixed order
        ws_bytes = _splitk_bytes(M, N, K) if (a.dtype == torch.bfloat16 and out_dtype == torch.float32) else 0
        if ws_bytes:
            ws = torch.empty(ws_bytes, dtype=torch.uint8, device=a.device)
            st = lib.axs6_gemm_bf16_ws(a.data_ptr(), b.data_ptr(), c.data_ptr(), bias_f.data_ptr() if bias_f is not None else None,
                                       M, N, K, _row_pitch(a), _row_pitch(b), N, int(a_mn), int(b_mn), _DT[out_dtype],
                                       ws.data_ptr(), ws_bytes, _stream(a.device))
        else:
            fn = lib.axs6_gemm_bf16 if a.dtype == torch.bfloat16 else lib.axs6_gemm_tf32
            st = fn(a.data_ptr(), b.data_ptr(), c.data_ptr(),
                    bias_f.data_ptr() if bias_f is not None else None, M, N, K,
                    _row_pitch(a), _row_pitch(b), N,
                    int(a_mn), int(b_mn), _DT[out_dtype], _stream(a.device))
    _lib.check("axs6_gemm", st)
    return c


class PackedOperand:
    """A matrix held as AXS-6 codes in the split layout: ``codes`` uint8 (rows, cols // 32, 24), ``exps`` uint8
    (cols // 64, rows, 2) -- the exponent of block b of row r is ``exps[b // 2, r, b % 2]``; NF5 grid, blocks of 32
    along the columns."""

    def __init__(self, codes: torch.Tensor, exps: torch.Tensor, rows: int, cols: int):
        self.codes, self.exps, self.rows, self.cols = codes, exps, rows, cols

    @property
    def shape(self):
        return (self.rows, self.cols)


def pack_split(x: torch.Tensor, rounding: str = "nearest", via_bf16: bool = False, noise: torch.Tensor | None = None) -> PackedOperand:
    """Quantise a 2-D tensor (NF5, block 32 along the last dimension) into the split layout that
    ``gemm_packed`` reads; the last dimension must be a multiple of 64."""
    _check_input(x, "pack_split")
    assert x.dim() == 2 and x.shape[1] % 64 == 0, "pack_split takes a 2-D tensor whose last dimension is a multiple of 64"
    rows, cols = x.shape
    codes = torch.empty((rows, cols // 32, 24), dtype=torch.uint8, device=x.device)
    exps = torch.empty((cols // 64, rows, 2), dtype=torch.uint8, device=x.device)
    x2, _, _, ldx = _as_rows(x)
    rnd = _rounding(rounding)
    seed, off, nz = 0, 0, None
    if rnd == ROUND_STOCHASTIC:
        if noise is not None:
            nz = noise.to(device=x.device, dtype=torch.float32).contiguous()
        else:
            seed, off = next_philox(rows * cols)
    flags = FLAG_INPUT_VIA_BF16 if (via_bf16 and x2.dtype == torch.float32) else 0
    with _on(x.device):
        st = _lib.load().axs6_pack(x2.data_ptr(), _DT[x2.dtype], rows, cols, ldx, 32, GRID_NF5, rnd, flags, seed, off,
                                   nz.data_ptr() if nz is not None else None, _lib.LAYOUT_SPLIT, codes.data_ptr(),
                                   exps.data_ptr(), None, _stream(x.device))
    _lib.check("axs6_pack", st)
    return PackedOperand(codes, exps, rows, cols)


def unpack_split(pk: PackedOperand, out_dtype: torch.dtype = torch.float32) -> torch.Tensor:
    """Values of a :class:`PackedOperand`, (rows, cols)."""
    y = torch.empty((pk.rows, pk.cols), dtype=out_dtype, device=pk.codes.device)
    with _on(y.device):
        st = _lib.load().axs6_unpack(_lib.LAYOUT_SPLIT, pk.codes.data_ptr(), pk.exps.data_ptr(), None, y.data_ptr(), _DT[out_dtype],
                                     pk.rows, pk.cols, pk.cols, 32, GRID_NF5, _stream(y.device))
    _lib.check("axs6_unpack", st)
    return y


def gemm_packed(a, b, bias: torch.Tensor | None = None, a_mn: bool = False, b_mn: bool = False,
                out_dtype: torch.dtype = torch.float32) -> torch.Tensor:
    """C = op(A) op(B) with one or both operands given as :class:`PackedOperand` (decoded to bf16 inside the
    kernel); the other, if any, a 2-D bf16 tensor with 16-byte aligned rows.  Shapes as in ``gemm_bf16``."""
    pa, pb = isinstance(a, PackedOperand), isinstance(b, PackedOperand)
    assert pa or pb, "gemm_packed needs at least one PackedOperand"
    M, K = (a.shape[1], a.shape[0]) if a_mn else a.shape
    N, K2 = (b.shape[1], b.shape[0]) if b_mn else b.shape
    assert K == K2, "contraction lengths differ"
    dev = (a.codes if pa else a).device
    c = torch.empty((M, N), dtype=out_dtype, device=dev)
    bias_f = bias.to(device=dev, dtype=torch.float32).contiguous() if bias is not None else None

    def args(t, packed):
        if packed:
            return t.codes.data_ptr(), t.exps.data_ptr(), 0
        assert t.dtype == torch.bfloat16 and t.dim() == 2 and t.stride(1) == 1
        return t.data_ptr(), None, _row_pitch(t)
    ap, ae, lda = args(a, pa)
    bp, be, ldb = args(b, pb)
    with _on(dev):
        st = _lib.load().axs6_gemm_packed(ap, ae, lda, bp, be, ldb, c.data_ptr(), bias_f.data_ptr() if bias_f is not None else None,
                                          M, N, K, N, int(a_mn), int(b_mn), _DT[out_dtype], _stream(dev))
    _lib.check("axs6_gemm_packed", st)
    return c


def _row_pitch(t: torch.Tensor) -> int:
    """Leading dimension handed to the library: the row stride, or for a one-row operand (whose stride means
    nothing) the row length rounded up to a 16-byte multiple."""
    if t.shape[0] > 1:
        return t.stride(0)
    per16 = 16 // t.element_size()
    return max((t.shape[1] + per16 - 1) // per16 * per16, per16)


def _padded_copy(t: torch.Tensor) -> torch.Tensor:
    """Copy into a buffer whose rows start 16-byte aligned (row length rounded up to 8 elements)."""
    rows, cols = t.shape
    per16 = 16 // t.element_size()
    ld = (cols + per16 - 1) // per16 * per16
    buf = torch.zeros((rows, ld), dtype=t.dtype, device=t.device)
    buf[:, :cols].copy_(t)
    return buf[:, :cols]


def _r8(v: int) -> int:
    return (v + 7) // 8 * 8


def _r4(v: int) -> int:
    return (v + 3) // 4 * 4


def _ws_bytes(what: int, M: int, N: int, K: int) -> int:
    """Python twin of axs6_linear_workspace_bytes (saves a library call per buffer)."""
    if what == 0: return M * _r8(K) * 2
    if what == 1: return N * _r8(K) * 2
    if what == 2: return M * _r8(N) * 2
    if what == 3: return 32 * N * 4
    if what == 4: return M * _r4(K) * 4
    if what == 5: return N * _r4(K) * 4
    if what == 6: return M * _r4(N) * 4
    if what == 7: return (K * _r4(N) + N * _r4(M) + K * _r4(M)) * 4
    if what == 12: return M * _r4(K) * 16
    if what == 13: return N * _r4(K) * 16
    if what in (8, 9, 10):
        rows, cols = {8: (M, K), 9: (N, K), 10: (M, N)}[what]
        nblk = (cols + 31) // 32
        return (rows * nblk * 24 + 255) // 256 * 256 + (nblk + 1) // 2 * rows * 2
    raise ValueError(what)


def _ws(what: int, M: int, N: int, K: int, dev, dtype=torch.uint8) -> torch.Tensor:
    return torch.empty(max(_ws_bytes(what, M, N, K), 16), dtype=torch.uint8, device=dev)


def _carve(dev, sizes: list[int]) -> list[int]:
    """One allocation for several 256-byte aligned scratch regions; returns (keep-alive tensor, pointers)."""
    offs, total = [], 0
    for n in sizes:
        offs.append(total)
        total += (max(n, 16) + 255) // 256 * 256
    buf = torch.empty(total, dtype=torch.uint8, device=dev)
    base = buf.data_ptr()
    return buf, [base + o for o in offs]


def linear_fwd(x2: torch.Tensor, w: torch.Tensor, bias_f32: torch.Tensor | None, block_size: int, grid: int,
               quantize_input: bool, out_dtype: torch.dtype, tf32: bool = False, bias_via_bf16: bool = False,
               return_wq: bool = False, packed: bool = False, fp32_accuracy: bool = False):
    """-> (y (M, N), xq workspace holding the quantised activations that backward needs); with
    ``return_wq`` also the workspace that holds the quantised weight (backward can reuse it while the
    weight is unchanged).  ``tf32``: the fp32 graph (operands fake-quantised in fp32, TF32 tensor cores)
    instead of bf16.  ``packed``: the workspaces hold 6-bit codes and the GEMM decodes them on load
    (``linear_packed_ok`` says whether the shapes allow it).  ``fp32_accuracy`` (with ``tf32``): three TF32
    products per output instead of one, for fp32 accuracy (what the reference's forward has)."""
    M, K = x2.shape
    N = w.shape[0]
    dev = x2.device
    x3 = bool(fp32_accuracy and tf32)
    xq = torch.empty(max(_ws_bytes(8 if packed else (12 if x3 else (4 if tf32 else 0)), M, N, K), 16), dtype=torch.uint8, device=dev)
    wq = torch.empty(max(_ws_bytes(9 if packed else (13 if x3 else (5 if tf32 else 1)), M, N, K), 16), dtype=torch.uint8, device=dev)
    y = torch.empty((M, N), dtype=out_dtype, device=dev)
    flags = (_lib.LINEAR_QUANTIZE_INPUT if quantize_input else 0) | (_lib.LINEAR_COMPUTE_TF32 if tf32 else 0) | \
            (_lib.LINEAR_BIAS_VIA_BF16 if bias_via_bf16 else 0) | (_lib.LINEAR_OPERANDS_PACKED if packed else 0) | \
            (_lib.LINEAR_FP32_ACCURACY if x3 else 0)
    with _on(dev):
        st = _lib.load().axs6_linear_fwd(x2.data_ptr(), _DT[x2.dtype], x2.stride(0) if M > 1 else K,
                                         w.data_ptr(), _DT[w.dtype], w.stride(0) if N > 1 else K,
                                         bias_f32.data_ptr() if bias_f32 is not None else None,
                                         y.data_ptr(), _DT[out_dtype], N, M, N, K, block_size, grid, flags,
                                         xq.data_ptr(), wq.data_ptr(), _stream(dev))
    _lib.check("axs6_linear_fwd", st)
    if x3:
        # backward needs the fp32 quantised activations only (the head of the buffer): keep a copy of that part
        # and let the three-part split go
        xq = xq[: M * _r4(K) * 4].clone()
    if return_wq:
        return y, xq, wq
    return y, xq


def linear_bwd(g2: torch.Tensor, xq: torch.Tensor, w: torch.Tensor, M: int, N: int, K: int, block_size: int,
               grid: int, quantize_grad: bool, need_dx: bool, need_dw: bool, need_db: bool,
               dx_dtype: torch.dtype = torch.bfloat16, noise: torch.Tensor | None = None, tf32: bool = False,
               bias_from_quantized: bool = False, wq: torch.Tensor | None = None, packed: bool = False):
    """-> (dx (M, K) or None, dw fp32 (N, K) or None, db fp32 (N,) or None).  ``wq``: the quantised-weight
    workspace of the forward call, valid only while the weight has not changed (bf16 graph); without it the
    quantised weight is recomputed."""
    dev = g2.device
    reuse_wq = wq is not None and need_dx and not tf32
    splitk = 0
    if need_dw and not tf32 and not packed:
        splitk = _splitk_bytes(N, K, M)
    dx = torch.empty((M, K), dtype=dx_dtype, device=dev) if need_dx else None
    dw = torch.empty((N, K), dtype=torch.float32, device=dev) if need_dw else None
    db = torch.empty((N,), dtype=torch.float32, device=dev) if need_db else None
    keep, (p_gq, p_wq, p_part, p_tscr) = _carve(dev, [
        _ws_bytes(10 if packed else (6 if tf32 else 2), M, N, K),
        _ws_bytes(9 if packed else (5 if tf32 else 1), M, N, K) if (need_dx and not reuse_wq) else 0,
        _ws_bytes(3, M, N, K) if need_db else 0,
        _ws_bytes(7, M, N, K) if (tf32 and (need_dx or need_dw)) else splitk])
    seed, off = (0, 0)
    nz = None
    if quantize_grad:
        if noise is not None:
            nz = noise.to(device=dev, dtype=torch.float32).contiguous()
        else:
            seed, off = next_philox(M * (-(-N // block_size)) * block_size)
    flags = (_lib.LINEAR_QUANTIZE_GRAD if quantize_grad else 0) | (_lib.LINEAR_COMPUTE_TF32 if tf32 else 0) | \
            (_lib.LINEAR_BIAS_FROM_QUANTIZED if bias_from_quantized else 0) | (_lib.LINEAR_REUSE_WQ if reuse_wq else 0) | \
            (_lib.LINEAR_OPERANDS_PACKED if packed else 0) | (_lib.LINEAR_SPLITK_WORKSPACE if splitk else 0)
    if reuse_wq:
        p_wq = wq.data_ptr()
    with _on(dev):
        st = _lib.load().axs6_linear_bwd(
            g2.data_ptr(), _DT[g2.dtype], g2.stride(0) if M > 1 else N, xq.data_ptr() if need_dw else None,
            w.data_ptr(), _DT[w.dtype], w.stride(0) if N > 1 else K,
            dx.data_ptr() if need_dx else None, _DT[dx_dtype], K, dw.data_ptr() if need_dw else None, K,
            db.data_ptr() if need_db else None, M, N, K, block_size, grid, flags, seed, off,
            nz.data_ptr() if nz is not None else None, p_gq, p_wq if need_dx else None,
            p_part if need_db else None, p_tscr if ((tf32 and (need_dx or need_dw)) or splitk) else None, _stream(dev))
    _lib.check("axs6_linear_bwd", st)
    del keep
    return dx, dw, db


_SPLITK_CACHE: dict = {}


def _splitk_bytes(M: int, N: int, K: int) -> int:
    """Workspace from which the (M, N) = (., K) fp32 product profits (see axs6_gemm_workspace_bytes); cached per shape."""
    key = (M, N, K, torch.cuda.current_device())
    v = _SPLITK_CACHE.get(key)
    if v is None:
        v = int(_lib.load().axs6_gemm_workspace_bytes(M, N, K, F32))
        _SPLITK_CACHE[key] = v
    return v


def linear_packed_ok(N: int, K: int, block_size: int, quantize_input: bool, quantize_grad: bool) -> bool:
    """Whether the quantise-on-load Linear (operands as codes) can serve this layer."""
    return block_size == 32 and quantize_input and quantize_grad and K % 64 == 0 and N % 64 == 0


def bias_grad(g: torch.Tensor) -> torch.Tensor:
    """fp32 column sums of a 2-D fp32 / bf16 gradient (deterministic order)."""
    _check_input(g, "bias_grad")
    g2, rows, cols, ld = _as_rows(g)
    out = torch.empty((cols,), dtype=torch.float32, device=g.device)
    part = _ws(3, 0, cols, 0, g.device)
    with _on(g.device):
        st = _lib.load().axs6_bias_grad(g2.data_ptr(), _DT[g2.dtype], ld, rows, cols, out.data_ptr(), part.data_ptr(),
                                        _stream(g.device))
    _lib.check("axs6_bias_grad", st)
    return out


def transpose_f32(t: torch.Tensor) -> torch.Tensor:
    """(rows, cols) fp32 -> contiguous-row (cols, rows) copy whose rows start 16-byte aligned."""
    _check_input(t, "transpose_f32")
    assert t.dtype == torch.float32 and t.dim() == 2
    if t.stride(1) != 1:
        t = t.contiguous()
    rows, cols = t.shape
    ld = (rows + 3) // 4 * 4
    out = torch.empty((cols, ld), dtype=torch.float32, device=t.device)
    with _on(t.device):
        st = _lib.load().axs6_transpose_f32(t.data_ptr(), out.data_ptr(), rows, cols, t.stride(0) if rows > 1 else cols,
                                            ld, _stream(t.device))
    _lib.check("axs6_transpose_f32", st)
    return out[:, :rows]
