"""Gradient packing in the 25-byte wire layout (mirror of the codec half of
``axs/unified/distributed.py``: ``_pack_gradient`` :70-120, ``_unpack_gradient`` :123-144,
``_pack_to_flat_buffer`` :147-198, ``_unpack_from_flat_buffer`` :201-232).

``pack_wire`` / ``unpack_wire`` do value -> bytes and bytes -> value in ONE kernel each; the
four reference-named helpers are kept for call-site compatibility and go through the planes.
"""
from __future__ import annotations

import torch

from .. import ops
from ..core import DEFAULT_BLOCK_SIZE


def pack_wire(tensor: torch.Tensor, block_size: int = DEFAULT_BLOCK_SIZE, rounding: str = "nearest") -> torch.Tensor:
    """tensor -> flat int8 buffer: per block 1 exponent byte + 6-bit codes (25 B per 32 values)."""
    return ops.pack(tensor, block_size, ops.GRID_NF5, rounding, ops.LAYOUT_WIRE, who="pack_wire").view(torch.int8)


def unpack_wire(buffer: torch.Tensor, shape, block_size: int = DEFAULT_BLOCK_SIZE,
                dtype: torch.dtype = torch.float32) -> torch.Tensor:
    """Inverse of :func:`pack_wire`; returns a tensor of ``shape``."""
    shape = torch.Size(shape)
    rows = 1
    for s in shape[:-1]:
        rows *= s
    y = ops.unpack(ops.LAYOUT_WIRE, buffer.view(torch.uint8), rows, shape[-1], block_size, ops.GRID_NF5, dtype)
    return y.reshape(shape)


def _pack_gradient(tensor: torch.Tensor, block_size: int = DEFAULT_BLOCK_SIZE):
    se, sg, mg = ops.pack(tensor, block_size, ops.GRID_NF5, "nearest", ops.LAYOUT_PLANES, who="_pack_gradient")
    return se, sg, mg, tensor.shape


def _unpack_gradient(shared_exponents, signs, magnitudes, original_shape, block_size: int = DEFAULT_BLOCK_SIZE):
    rows = magnitudes.shape[0]
    y = ops.unpack(ops.LAYOUT_PLANES, (shared_exponents, signs, magnitudes), rows, original_shape[-1], block_size,
                   ops.GRID_NF5, torch.float32)
    return y.reshape(original_shape)


def _pack_to_flat_buffer(shared_exponents: torch.Tensor, signs: torch.Tensor, magnitudes: torch.Tensor) -> torch.Tensor:
    """Planes -> flat int8 buffer of wire records (reference: distributed.py:147-198)."""
    rows, num_blocks, block_size = magnitudes.shape
    se = shared_exponents.contiguous()
    sg = signs.contiguous()
    mg = magnitudes.contiguous()
    rec = 1 + block_size * 3 // 4
    out = torch.empty(rows * num_blocks * rec, dtype=torch.uint8, device=mg.device)
    st = ops._lib.load().axs6_repack(1, ops.LAYOUT_WIRE, block_size, rows * num_blocks, se.data_ptr(), sg.data_ptr(),
                                     mg.data_ptr(), out.data_ptr(), torch.cuda.current_stream(mg.device).cuda_stream)
    ops._lib.check("axs6_repack", st)
    return out.view(torch.int8)


def _unpack_from_flat_buffer(buffer: torch.Tensor, rows: int, num_blocks: int, block_size: int):
    """Flat wire records -> (exponents u8, signs bool, magnitudes u8) (reference: distributed.py:201-232)."""
    buf = buffer.contiguous()
    dev = buf.device
    se = torch.empty((rows, num_blocks), dtype=torch.uint8, device=dev)
    sg = torch.empty((rows, num_blocks, block_size), dtype=torch.bool, device=dev)
    mg = torch.empty((rows, num_blocks, block_size), dtype=torch.uint8, device=dev)
    st = ops._lib.load().axs6_repack(0, ops.LAYOUT_WIRE, block_size, rows * num_blocks, se.data_ptr(), sg.data_ptr(),
                                     mg.data_ptr(), buf.data_ptr(), torch.cuda.current_stream(dev).cuda_stream)
    ops._lib.check("axs6_repack", st)
    return se, sg, mg


# ---------------------------------------------------------------------------------------------
# Row sharding and gradient exchange (host logic over torch.distributed)
# ---------------------------------------------------------------------------------------------
import math
from dataclasses import dataclass
from typing import Any, Callable

import torch.distributed as dist


def shard_rows(rows: int, rank: int, world: int) -> tuple[int, int]:
    """Contiguous row range [start, stop) of `rank`: blocks never cross a row, so fake-quantise,
    pack and unpack shard by rows with no exchange of data.  The first ``rows % world`` ranks
    take one extra row."""
    base, extra = divmod(rows, world)
    start = rank * base + min(rank, extra)
    return start, start + base + (1 if rank < extra else 0)


class CudaCodec:
    """The three codec operations the gradient hooks need, on the CUDA kernels."""

    def __init__(self, block_size: int = DEFAULT_BLOCK_SIZE):
        self.block_size = block_size

    def pack(self, flat: torch.Tensor) -> torch.Tensor:
        """1-D tensor -> uint8 wire records of its zero-padded blocks."""
        return ops.pack(flat.reshape(1, -1), self.block_size, ops.GRID_NF5, "nearest", ops.LAYOUT_WIRE, who="pack")

    def pack_padded16(self, flat: torch.Tensor) -> torch.Tensor:
        """The same records at the front of a buffer whose size is rounded up to a multiple of 16 bytes."""
        nblk = -(-flat.numel() // self.block_size)
        n = nblk * ops.record_bytes(ops.LAYOUT_WIRE, self.block_size)
        buf = torch.empty((n + 15) // 16 * 16, dtype=torch.uint8, device=flat.device)
        ops.pack(flat.reshape(1, -1), self.block_size, ops.GRID_NF5, "nearest", ops.LAYOUT_WIRE, who="pack", out=buf)
        return buf

    def unpack(self, buf: torch.Tensor, numel: int, dtype: torch.dtype) -> torch.Tensor:
        out_dt = dtype if dtype in (torch.float32, torch.bfloat16) else torch.float32
        y = ops.unpack(ops.LAYOUT_WIRE, buf, 1, numel, self.block_size, ops.GRID_NF5, out_dt)
        return y.reshape(-1).to(dtype)

    def unpack_mean(self, gathered: torch.Tensor, world: int, stride: int, numel: int, dtype: torch.dtype,
                    out: torch.Tensor | None = None) -> torch.Tensor:
        """Mean of the ``world`` record buffers' reconstructions (buffer r at byte ``r * stride``), one fused pass;
        written into ``out`` (fp32 or bf16, contiguous, ``numel`` values) when given."""
        if out is not None and out.dtype in (torch.float32, torch.bfloat16) and out.is_contiguous():
            ops.unpack_sum(ops.LAYOUT_WIRE, gathered, world, stride, 1, numel, self.block_size, ops.GRID_NF5,
                           divisor=float(world), out=out)
            return out
        out_dt = dtype if dtype in (torch.float32, torch.bfloat16) else torch.float32
        y = ops.unpack_sum(ops.LAYOUT_WIRE, gathered, world, stride, 1, numel, self.block_size, ops.GRID_NF5, out_dt, float(world))
        return y.reshape(-1).to(dtype)

    def roundtrip(self, flat: torch.Tensor) -> torch.Tensor:
        """unpack(pack(flat)): what a peer would reconstruct from this rank's records."""
        return self.unpack(self.pack(flat), flat.numel(), flat.dtype)


@dataclass
class HookState:
    """State object for the communication hooks: the process group and the codec."""
    group: Any = None
    codec: Any = None

    def resolve(self):
        group = self.group if self.group is not None else dist.group.WORLD
        return group, (self.codec if self.codec is not None else CudaCodec())


def _state(state) -> tuple[Any, Any]:
    if isinstance(state, HookState):
        return state.resolve()
    group = state if (state is not None and isinstance(state, dist.ProcessGroup)) else dist.group.WORLD
    return group, CudaCodec()


def _allreduce_mean(flat: torch.Tensor, group, world: int) -> "torch.futures.Future[torch.Tensor]":
    fut = dist.all_reduce(flat, op=dist.ReduceOp.SUM, group=group, async_op=True).get_future()

    def done(f):
        v = f.value()
        v = v[0] if isinstance(v, list) else v
        return v.div_(world)

    return fut.then(done)


def axs6_gradient_hook(state: Any, bucket) -> "torch.futures.Future[torch.Tensor]":
    """DDP communication hook with the semantics of the reference's ``axs6_gradient_hook``
    (distributed.py:239-305): every rank replaces its flat gradient bucket by its AXS-6 NF5
    reconstruction (pack -> unpack, block 32 over the zero-padded flat buffer), the reconstructions
    are all-reduced in the gradient's own dtype and divided by the world size."""
    group, codec = _state(state)
    world = dist.get_world_size(group)
    grad = bucket.buffer()
    recon = codec.roundtrip(grad.reshape(-1)).to(grad.dtype)
    return _allreduce_mean(recon, group, world)


def _packed16(codec, flat: torch.Tensor) -> torch.Tensor:
    return codec.pack_padded16(flat) if hasattr(codec, "pack_padded16") else _padded16(codec.pack(flat))


def _padded16(records: torch.Tensor) -> torch.Tensor:
    """The records in a buffer whose size is a multiple of 16 bytes, so that every rank's slice of the
    gathered buffer starts 16-byte aligned (the fused unpack-and-average kernel moves them with bulk copies)."""
    n = records.numel()
    n16 = (n + 15) // 16 * 16
    if n16 == n:
        return records
    out = torch.zeros(n16, dtype=records.dtype, device=records.device)
    out[:n] = records
    return out


def _mean_of_gathered(codec, gathered: torch.Tensor, world: int, stride: int, numel: int, dtype: torch.dtype,
                      out: torch.Tensor | None = None) -> torch.Tensor:
    """Mean of the ranks' reconstructions, summed in fp32 in rank order: fused when the codec can, and then
    written straight into ``out`` (the gradient bucket itself) so that nothing is allocated after the gather."""
    if hasattr(codec, "unpack_mean"):
        return codec.unpack_mean(gathered, world, stride, numel, dtype, out)
    acc = None
    for r in range(world):
        part = codec.unpack(gathered[r * stride:(r + 1) * stride], numel, torch.float32)
        acc = part if acc is None else acc.add_(part)
    return acc.div_(world).to(dtype)


def axs6_gradient_hook_packed(state: Any, bucket) -> "torch.futures.Future[torch.Tensor]":
    """Compressed exchange: each rank packs its bucket to 25-byte records (6.25 bits per value on
    the wire), the records are all-gathered, and every rank decodes all of them and averages in ONE fused pass
    (``axs6_unpack_sum``: every record read once, the mean written once).

    Same name and registration as the reference's packed hook (distributed.py:308-367) but not
    its arithmetic: the reference all-reduces the bit-packed bytes as integers and averages
    them, which mixes unrelated bit fields; here the result is exactly the mean of the ranks'
    reconstructions, i.e. identical to :func:`axs6_gradient_hook` up to summation order."""
    group, codec = _state(state)
    world = dist.get_world_size(group)
    grad = bucket.buffer()
    numel, dtype = grad.numel(), grad.dtype
    mine = _packed16(codec, grad.reshape(-1))
    gathered = torch.empty(world * mine.numel(), dtype=mine.dtype, device=mine.device)
    fut = dist.all_gather_into_tensor(gathered, mine, group=group, async_op=True).get_future()

    flat = grad.reshape(-1)

    def done(f):
        # the records were read before the gather; the bucket can take the result
        return _mean_of_gathered(codec, gathered, world, mine.numel(), numel, dtype, out=flat).reshape(grad.shape)

    return fut.then(done)


class AXS6GradCompressor:
    """Manual-loop counterpart of the hooks (reference: distributed.py:374-440).
    ``packed=False``: all-reduce of the local reconstructions; ``packed=True``: all-gather of the
    packed records (see :func:`axs6_gradient_hook_packed` for how this differs from the reference)."""

    def __init__(self, process_group=None, block_size: int = DEFAULT_BLOCK_SIZE, packed: bool = False,
                 codec=None) -> None:
        self.group = process_group
        self.block_size = block_size
        self.packed = packed
        self.codec = codec

    def compress_and_allreduce(self, grad: torch.Tensor) -> torch.Tensor:
        group = self.group if self.group is not None else dist.group.WORLD
        codec = self.codec if self.codec is not None else CudaCodec(self.block_size)
        world = dist.get_world_size(group)
        flat = grad.reshape(-1)
        if not self.packed:
            recon = codec.roundtrip(flat).to(grad.dtype)
            dist.all_reduce(recon, op=dist.ReduceOp.SUM, group=group)
            return recon.div_(world).reshape(grad.shape)
        mine = _packed16(codec, flat)
        gathered = torch.empty(world * mine.numel(), dtype=mine.dtype, device=mine.device)
        dist.all_gather_into_tensor(gathered, mine, group=group)
        return _mean_of_gathered(codec, gathered, world, mine.numel(), flat.numel(), grad.dtype).reshape(grad.shape)
