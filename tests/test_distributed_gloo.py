"""Host-side logic of the multi-rank paths on CPU: two gloo ranks (spawned processes).  The codec
used inside the hooks is the CPU oracle, injected through HookState -- the CUDA kernels are
checked against that same oracle in the GPU tests, so what is tested here is the sharding,
gathering, averaging and the hook plumbing."""
import importlib
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


class OracleCodec:
    """pack / unpack / roundtrip on the CPU oracle (block 32, NF5, wire layout)."""

    def __init__(self):
        import oracle
        self.o = oracle

    def pack(self, flat):
        x = flat.detach().float().numpy().reshape(1, -1)
        se, sg, mg = self.o.quantize(x, 32, self.o.GRID_NF5)
        return torch.from_numpy(self.o.pack_bytes(se, sg, mg, self.o.LAYOUT_WIRE))

    def unpack(self, buf, numel, dtype):
        nblk = -(-numel // 32)
        se, sg, mg = self.o.unpack_bytes(buf.numpy(), 1, nblk, 32, self.o.LAYOUT_WIRE)
        return torch.from_numpy(self.o.dequantize(se, sg, mg, numel, self.o.GRID_NF5)).reshape(-1).to(dtype)

    def roundtrip(self, flat):
        return self.unpack(self.pack(flat), flat.numel(), flat.dtype)


class FakeBucket:
    def __init__(self, t):
        self.t = t

    def buffer(self):
        return self.t


def _worker(rank, world, port, results):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import oracle
        ud = importlib.import_module("axs6_b200.unified.distributed")
        codec = OracleCodec()
        state = ud.HookState(group=None, codec=codec)
        out = {}

        # 1. row-sharded fake-quantise == fake-quantise of the whole tensor
        rng = np.random.default_rng(0)
        full = rng.standard_normal((38, 96), dtype=np.float32)
        lo, hi = ud.shard_rows(38, rank, world)
        mine = torch.from_numpy(oracle.fused_fake_quantize(full[lo:hi]))
        sizes = [ud.shard_rows(38, r, world) for r in range(world)]
        parts = [torch.empty((b - a, 96)) for a, b in sizes]
        dist.all_gather(parts, mine)
        out["shard_equal"] = bool(np.array_equal(torch.cat(parts).numpy().view(np.uint32),
                                                 oracle.fused_fake_quantize(full).view(np.uint32)))

        # 2. the two hooks: mean of the ranks' reconstructions
        g = torch.from_numpy(np.random.default_rng(10 + rank).standard_normal(1000, dtype=np.float32))
        recon_all = [OracleCodec().roundtrip(torch.from_numpy(
            np.random.default_rng(10 + r).standard_normal(1000, dtype=np.float32))) for r in range(world)]
        want = sum(recon_all) / world
        a = ud.axs6_gradient_hook(state, FakeBucket(g.clone())).wait()
        b = ud.axs6_gradient_hook_packed(state, FakeBucket(g.clone())).wait()
        out["hook_close"] = bool(torch.allclose(a, want, rtol=0, atol=1e-7))
        out["packed_close"] = bool(torch.allclose(b, want, rtol=0, atol=1e-7))
        out["shape_dtype"] = (tuple(a.shape), str(a.dtype), tuple(b.shape), str(b.dtype))

        # 3. manual compressor, both modes, 2-D gradient
        g2 = torch.from_numpy(np.random.default_rng(20 + rank).standard_normal((10, 50), dtype=np.float32))
        want2 = sum(OracleCodec().roundtrip(torch.from_numpy(
            np.random.default_rng(20 + r).standard_normal((10, 50), dtype=np.float32)).reshape(-1)) for r in range(world)) / world
        for packed in (False, True):
            c = ud.AXS6GradCompressor(packed=packed, codec=codec)
            r = c.compress_and_allreduce(g2.clone())
            out[f"compressor_{packed}"] = bool(torch.allclose(r.reshape(-1), want2, rtol=0, atol=1e-7)) and r.shape == g2.shape
        results[rank] = out
    finally:
        dist.destroy_process_group()


def test_shard_rows_partition():
    ud = importlib.import_module("axs6_b200.unified.distributed")
    for rows in (0, 1, 7, 8, 37, 32768):
        for world in (1, 2, 3, 8):
            spans = [ud.shard_rows(rows, r, world) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == rows
            assert all(spans[i][1] == spans[i + 1][0] for i in range(world - 1))
            assert max(b - a for a, b in spans) - min(b - a for a, b in spans) <= 1


def test_two_gloo_ranks():
    world = 2
    port = 29500 + (os.getpid() % 2000)
    with mp.Manager() as m:
        results = m.dict()
        mp.spawn(_worker, args=(world, port, results), nprocs=world, join=True)
        assert len(results) == world
        for rank in range(world):
            out = results[rank]
            assert out["shard_equal"], rank
            assert out["hook_close"] and out["packed_close"], (rank, out)
            assert out["shape_dtype"] == ((1000,), "torch.float32", (1000,), "torch.float32")
            assert out["compressor_False"] and out["compressor_True"], (rank, out)
