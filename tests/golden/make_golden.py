"""Generate the golden fixtures in this folder by running the reference implementation.

Usage:  python tests/golden/make_golden.py --reference <path to a checkout of bwiemz/axs-6>

The reference (pure Python + torch, CPU eager) is imported from the given path; nothing of
it is copied.  Inputs are stored as raw bit patterns next to the outputs the reference
produced for them, so the fixtures can be replayed on a machine without the reference.
Stochastic rounding is made reproducible by substituting ``torch.rand_like`` with a
recorded noise tensor while the reference runs.

Files written:
  tables.npz         NF5 codebook, 1024-entry LUT, reverse LUT (+ sha256 in manifest.json)
  log2_bump_set.npy  every positive fp32 whose ``log2().floor()`` exceeds its true exponent
  fq_cases.npz       fake-quantise / quantise / byte-layout cases (nearest and stochastic)
  linear_cases.npz   small Linear forward/backward cases of the three autograd Functions
  manifest.json      case list, torch version, sha256 of the large-config outputs
  block_cases.npz    per-block host utilities of axs/core.py (axs_encode_block / axs_decode_block /
                     AXSBlock.to_bytes) and quantization_error; written alone with --only blocks
"""
from __future__ import annotations

import argparse
import hashlib
import json
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def sha(a) -> str:
    if isinstance(a, torch.Tensor):
        a = a.contiguous().view(torch.uint8).numpy() if a.dtype != torch.bool else a.to(torch.uint8).numpy()
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def bits(t: torch.Tensor) -> np.ndarray:
    t = t.contiguous()
    if t.dtype == torch.float32:
        return t.view(torch.int32).numpy().view(np.uint32).copy()
    if t.dtype == torch.bfloat16:
        return t.view(torch.int16).numpy().view(np.uint16).copy()
    raise TypeError(t.dtype)


class fixed_noise:
    """Context manager: torch.rand_like returns the recorded noise (reshaped)."""

    def __init__(self, noise: torch.Tensor):
        self.noise = noise

    def __enter__(self):
        self._orig = torch.rand_like
        noise = self.noise

        def fake(t, *a, **k):
            assert t.numel() == noise.numel(), (t.shape, noise.shape)
            return noise.reshape(t.shape).to(t.dtype)

        torch.rand_like = fake
        return self

    def __exit__(self, *exc):
        torch.rand_like = self._orig


def rand24(gen: np.random.Generator, n: int) -> torch.Tensor:
    """U[0,1) on the 24-bit grid torch.rand uses for fp32."""
    return torch.from_numpy((gen.integers(0, 1 << 24, size=n).astype(np.float32) * np.float32(2.0 ** -24)))


def bump_boundary_blocks(gen: np.random.Generator) -> torch.Tensor:
    """Blocks of 32 whose amax sits at / next to the top-of-binade inputs where the fp32 log2
    rounds up to the next integer; exponent fields 1..252 and the denormal sub-binades."""
    rows = []
    for ef in range(1, 253):
        for d in (0, 1, 2, 4, 5, 10, 11, 21, 22, 43, 44, 45, 90):
            amax = np.array([(ef << 23) | (0x7FFFFF - d)], dtype=np.uint32).view(np.float32)[0]
            blk = (gen.random(32).astype(np.float32) * 2 - 1) * amax
            blk[gen.integers(0, 32)] = amax * (1 if gen.random() < 0.5 else -1)
            rows.append(blk)
    for top in range(1, 24):  # denormal amax with top bit at position top-1
        for d in (1, 2, 3, 5, 6, 11, 12, 22, 23):
            m = (1 << top) - d
            if m <= 0:
                continue
            amax = np.array([m], dtype=np.uint32).view(np.float32)[0]
            blk = np.zeros(32, dtype=np.float32)
            blk[gen.integers(0, 32)] = -amax
            blk[gen.integers(0, 32)] = amax
            rows.append(blk)
    a = np.stack(rows)
    return torch.from_numpy(a.reshape(-1, 32 * 8).copy()) if a.shape[0] % 8 == 0 else torch.from_numpy(a)


def special_blocks() -> torch.Tensor:
    rows = []
    z = np.zeros(32, dtype=np.float32)
    rows.append(z.copy())
    nz = z.copy(); nz[::2] = -0.0
    rows.append(nz)
    for k in list(range(-126, 127, 7)) + [-126, -1, 0, 1, 126]:
        b = np.linspace(-1, 1, 32, dtype=np.float32) * np.float32(2.0 ** k)
        b[5] = np.float32(2.0 ** k)          # amax exactly a power of two
        b[9] = 0.0
        b[11] = -0.0
        rows.append(b)
        b2 = b.copy(); b2[5] = -np.float32(2.0 ** k)
        rows.append(b2)
    den = np.array([1, 2, 3, 7, 100, 0x7FFFFF, 0x400000, 0x3FFFFF], dtype=np.uint32).view(np.float32)
    b = z.copy(); b[:8] = den; b[8:16] = -den
    rows.append(b)
    b = z.copy(); b[3] = den[0]
    rows.append(b)
    b = z.copy(); b[0] = np.float32(2.0 ** -126); b[1] = den[5]; b[2] = -den[4]
    rows.append(b)
    # one large value among tiny ones (tiny ones underflow in the normalisation)
    b = np.full(32, np.float32(1e-40), dtype=np.float32); b[17] = np.float32(3.0e38 / 4)
    rows.append(b)
    b = np.full(32, np.float32(-1e-30), dtype=np.float32); b[0] = np.float32(1.5)
    rows.append(b)
    return torch.from_numpy(np.stack(rows))


def grid_boundary_blocks() -> torch.Tensor:
    """Values next to every decision threshold of both grids, in blocks with amax = 0.75
    (scale 1): LUT-index steps (k/1023) and uniform-grid ties ((j+0.5)/31)."""
    vals = []
    for k in range(0, 1024):
        c = np.float32(k) / np.float32(1023)
        for s in (-2, -1, 0, 1, 2):
            v = c
            for _ in range(abs(s)):
                v = np.nextafter(v, np.float32(2 if s > 0 else -2), dtype=np.float32)
            vals.append(v)
    for j in range(0, 31):
        c = np.float32((j + 0.5) / 31.0)
        for s in range(-3, 4):
            v = c
            for _ in range(abs(s)):
                v = np.nextafter(v, np.float32(2 if s > 0 else -2), dtype=np.float32)
            vals.append(v)
    v = np.array(vals, dtype=np.float32)
    v = v[(v >= 0) & (v < 1.0)]
    pad = (-len(v)) % 31
    v = np.concatenate([v, np.zeros(pad, dtype=np.float32)])
    blocks = v.reshape(-1, 31)
    sign = np.where(np.arange(blocks.size).reshape(blocks.shape) % 3 == 0, -1, 1).astype(np.float32)
    blocks = blocks * sign
    blocks = np.concatenate([np.full((blocks.shape[0], 1), 0.75, dtype=np.float32), blocks], axis=1)
    # second copy at another scale (amax 0.75 * 2^-9)
    return torch.from_numpy(np.concatenate([blocks, blocks * np.float32(2.0 ** -9)], axis=0))


def block_cases(ref_core) -> None:
    """Inputs and the reference's outputs for the per-block encoder / decoder (numpy, double precision) and for
    quantization_error (torch, CPU)."""
    gen = np.random.default_rng(77)
    store = {}
    n = 0
    for B in (8, 16, 32):
        blocks = [gen.standard_normal(B) * s for s in (1.0, 1e-3, 37.5, 2.0 ** -130, 1e30)]
        blocks.append(np.zeros(B))
        blocks.append(np.full(B, 0.5))                                   # maximum exactly a power of two
        tie = (np.arange(B) % 32 + 0.5) / 31.0 * 0.999                   # values near half-way points of the grid
        blocks.append(tie)
        blocks.append(np.float64(np.float32(gen.standard_normal(B))))    # fp32-representable values
        neg = gen.standard_normal(B)
        neg[::3] = -0.0
        blocks.append(neg)
        for v in blocks:
            for rounding in ("nearest", "stochastic"):
                name = f"blk{n}"
                np.random.seed(1000 + n)
                draws = np.random.uniform(0, 1, size=B)
                np.random.seed(1000 + n)
                blk = ref_core.axs_encode_block(v, rounding)
                store[f"{name}.values"] = np.asarray(v, dtype=np.float64)
                store[f"{name}.rounding"] = np.array([rounding == "stochastic"])
                store[f"{name}.seed"] = np.array([1000 + n])
                store[f"{name}.draws"] = draws
                store[f"{name}.exponent"] = np.array([blk.shared_exponent])
                store[f"{name}.signs"] = np.asarray(blk.signs, dtype=bool)
                store[f"{name}.magnitudes"] = np.asarray(blk.magnitudes, dtype=np.uint8)
                store[f"{name}.bytes"] = np.frombuffer(blk.to_bytes(), dtype=np.uint8)
                store[f"{name}.decoded"] = ref_core.axs_decode_block(blk)
                store[f"{name}.props"] = np.array([blk.scale, blk.total_bits, blk.bits_per_value])
                n += 1
    store["count"] = np.array([n])
    tg = torch.Generator().manual_seed(5)
    x = torch.randn(64, 256, generator=tg)
    for B in (8, 16, 32):
        e = ref_core.quantization_error(x, B, "nearest")
        store[f"qerr.b{B}"] = np.array([e["mse"], e["rmse"], e["max_abs_error"], e["mean_abs_error"], e["signal_to_noise_db"]])
    store["qerr.x"] = bits(x)
    # gradient-aware stochastic rounding (axs/quantize.py:203-307) with recorded draws
    ref_q = __import__("importlib").import_module("axs.quantize")
    for B, shape in ((32, (48, 96)), (16, (20, 50)), (8, (7, 24))):
        xg = torch.randn(*shape, generator=tg) * 0.3
        gg = torch.randn(*shape, generator=tg) * torch.rand(shape[0], 1, generator=tg) * 4
        nblk = -(-shape[1] // B)
        noise = rand24(gen, shape[0] * nblk * B).reshape(shape[0], nblk, B)
        for temp in (1.0, 3.0):
            with fixed_noise(noise):
                q = ref_q.quantize_gasr(xg, gg, B, temp)
            key = f"gasr.b{B}.t{int(temp)}"
            store[f"{key}.x"] = bits(xg); store[f"{key}.g"] = bits(gg); store[f"{key}.noise"] = noise.numpy()
            store[f"{key}.se"] = q.shared_exponents.numpy(); store[f"{key}.sign"] = q.signs.numpy(); store[f"{key}.mag"] = q.magnitudes.numpy()
    np.savez_compressed(os.path.join(HERE, "block_cases.npz"), **store)
    print(f"wrote {n} block cases")


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True)
    ap.add_argument("--only", default="", help="'blocks' = write block_cases.npz only")
    args = ap.parse_args()
    sys.path.insert(0, args.reference)
    torch.set_num_threads(max(1, os.cpu_count() or 1))

    import importlib
    import warnings
    warnings.simplefilter("ignore", DeprecationWarning)
    # import_module, not "from axs.unified import x": the package re-exports functions
    # under the same names as some of its sub-modules.
    ref_core = importlib.import_module("axs.core")
    ref_nnf = importlib.import_module("axs.nn.functional")
    ref_dist = importlib.import_module("axs.unified.distributed")
    ref_fu = importlib.import_module("axs.unified.functional_unified")
    ref_mp = importlib.import_module("axs.unified.mixed_precision")
    ref_qu = importlib.import_module("axs.unified.quantize_unified")

    block_cases(ref_core)
    if args.only == "blocks":
        return

    manifest: dict = {"torch": torch.__version__, "cases": {}, "hashes": {}}

    # ------------------------------------------------------------------ tables
    cb = ref_qu.NF5_CODEBOOK.numpy()
    lut = ref_qu.FUSED_NF5_LUT.numpy()
    rev = ref_qu.REVERSE_NF5_LUT.numpy()
    np.savez_compressed(os.path.join(HERE, "tables.npz"), codebook=cb, lut=lut, reverse=rev)
    manifest["hashes"]["NF5_CODEBOOK"] = sha(cb)
    manifest["hashes"]["FUSED_NF5_LUT"] = sha(lut)
    manifest["hashes"]["REVERSE_NF5_LUT"] = sha(rev)

    # ------------------------------------------------------------------ log2 bump set
    out = []
    CH = 1 << 23
    for e in range(0, 255):
        b = torch.arange(CH, dtype=torch.int32) | (e << 23)
        x = b.view(torch.float32)
        if e == 0:
            m = b.double(); m[0] = 1
            true = torch.floor(torch.log2(m)) - 149
        else:
            true = torch.full((CH,), float(e - 127), dtype=torch.float64)
        bad = x.log2().floor().double() != true
        if e == 0:
            bad[0] = False
        out.append(b[bad].numpy().astype(np.uint32))
    bump = np.sort(np.concatenate(out))
    np.save(os.path.join(HERE, "log2_bump_set.npy"), bump)
    manifest["hashes"]["log2_bump_set"] = sha(bump)

    # ------------------------------------------------------------------ fq / codec cases
    gen = np.random.default_rng(20240611)
    tg = torch.Generator().manual_seed(1234)
    store: dict[str, np.ndarray] = {}

    def add_case(name: str, x: torch.Tensor, block: int, stochastic: bool = False, bytes_too: bool = True):
        info = {"shape": list(x.shape), "dtype": str(x.dtype).replace("torch.", ""), "block": block,
                "stochastic": stochastic}
        store[f"{name}.x"] = bits(x)
        x2 = x.reshape(-1, x.shape[-1])
        nblk = -(-x2.shape[1] // block)
        npad = x2.shape[0] * nblk * block
        if stochastic:
            noise = rand24(gen, npad)
            store[f"{name}.noise"] = noise.numpy()
            with fixed_noise(noise):
                y = ref_qu.fused_fake_quantize(x, block, "stochastic")
            with fixed_noise(noise):
                qn = ref_qu.quantize_unified(x, block, "stochastic")
            with fixed_noise(noise):
                qu = ref_core.quantize(x, block, "stochastic")
        else:
            y = ref_qu.fused_fake_quantize(x, block, "nearest")
            qn = ref_qu.quantize_unified(x, block, "nearest")
            qu = ref_core.quantize(x, block, "nearest")
            # the wire packer's own quantiser must agree with quantize_unified
            se2, sg2, mg2, _ = ref_dist._pack_gradient(x, block)
            assert torch.equal(se2, qn.shared_exponents) and torch.equal(mg2, qn.magnitudes) and torch.equal(sg2, qn.signs)
        store[f"{name}.fq_nf5"] = bits(y)
        store[f"{name}.nf5.se"] = qn.shared_exponents.numpy()
        store[f"{name}.nf5.sign"] = qn.signs.to(torch.uint8).numpy()
        store[f"{name}.nf5.mag"] = qn.magnitudes.numpy()
        store[f"{name}.uni.se"] = qu.shared_exponents.numpy()
        store[f"{name}.uni.sign"] = qu.signs.to(torch.uint8).numpy()
        store[f"{name}.uni.mag"] = qu.magnitudes.numpy()
        store[f"{name}.deq_nf5"] = bits(ref_qu.dequantize_unified(qn))
        store[f"{name}.deq_uni"] = bits(ref_core.dequantize(qu))
        if not stochastic:
            v1 = ref_nnf.fake_quantize(x, block, "nearest")
            assert v1.dtype == torch.float32
            assert torch.equal(v1, ref_core.dequantize(qu))
        if bytes_too and not stochastic:
            wire = ref_dist._pack_to_flat_buffer(qn.shared_exponents, qn.signs, qn.magnitudes)
            store[f"{name}.nf5.wire"] = wire.view(torch.uint8).numpy()
            se3, sg3, mg3 = ref_dist._unpack_from_flat_buffer(wire, x2.shape[0], nblk, block)
            assert torch.equal(se3, qn.shared_exponents) and torch.equal(sg3, qn.signs) and torch.equal(mg3, qn.magnitudes)
            # spec layout, block by block through AXSBlock.to_bytes (python loop: small cases only)
            if x2.shape[0] * nblk <= 4096:
                recs = []
                se_n = qn.shared_exponents.numpy(); sg_n = qn.signs.numpy(); mg_n = qn.magnitudes.numpy()
                for r in range(x2.shape[0]):
                    for b in range(nblk):
                        blk = ref_core.AXSBlock(int(se_n[r, b]), ref_core.BlockConfig.DENSE,
                                                sg_n[r, b], mg_n[r, b], block)
                        by = blk.to_bytes()
                        back = ref_core.AXSBlock.from_bytes(by, block)
                        assert back.shared_exponent == int(se_n[r, b]) and (back.magnitudes == mg_n[r, b]).all()
                        recs.append(np.frombuffer(by, dtype=np.uint8))
                store[f"{name}.nf5.spec"] = np.concatenate(recs)
        manifest["cases"][name] = info

    for B in (32, 16, 8):
        add_case(f"randn_f32_b{B}", torch.randn(64, 96, generator=tg) * 0.02, B)
        xb = torch.randn(48, 128, generator=tg)
        xb[torch.rand(48, 128, generator=tg) < 0.01] *= 10
        xb[torch.rand(48, 128, generator=tg) < 0.02] = 0
        add_case(f"randn_bf16_b{B}", xb.to(torch.bfloat16), B)
        for shp in ((5, 33), (3, 50), (7, 100), (2, 127), (4, 255), (1, 1), (3, 7), (2, 3, 40), (6,)):
            nm = "x".join(map(str, shp))
            add_case(f"ragged_{nm}_f32_b{B}", torch.randn(*shp, generator=tg), B)
            add_case(f"ragged_{nm}_bf16_b{B}", torch.randn(*shp, generator=tg).to(torch.bfloat16), B)
        add_case(f"stoch_f32_b{B}", torch.randn(32, 96, generator=tg), B, stochastic=True)
        add_case(f"stoch_bf16_b{B}", (torch.randn(16, 104, generator=tg) * 3).to(torch.bfloat16), B, stochastic=True)
    # row scales spread log-uniform over [1e-4, 10] as in the large sweep
    sig = 10 ** (torch.rand(128, 1, generator=tg) * 5 - 4)
    add_case("rowscale_f32_b32", torch.randn(128, 256, generator=tg) * sig, 32)
    add_case("rowscale_bf16_b32", (torch.randn(128, 256, generator=tg) * sig).to(torch.bfloat16), 32)
    add_case("bump_f32_b32", bump_boundary_blocks(gen), 32, bytes_too=False)
    sp = special_blocks()
    add_case("special_f32_b32", sp, 32)
    add_case("special_f32_b16", sp, 16)
    add_case("special_f32_b8", sp, 8)
    add_case("gridedge_f32_b32", grid_boundary_blocks(), 32, bytes_too=False)
    add_case("gridedge_stoch_f32_b32", grid_boundary_blocks(), 32, stochastic=True)
    np.savez_compressed(os.path.join(HERE, "fq_cases.npz"), **store)

    # ------------------------------------------------------------------ linear cases
    lstore: dict[str, np.ndarray] = {}

    def add_linear(name: str, fn, M: tuple[int, ...], K: int, N: int, dtype, bias: bool, qin: bool, qgrad: bool):
        x = (torch.randn(*M, K, generator=tg)).to(dtype).requires_grad_(True)
        w = (torch.randn(N, K, generator=tg) * 0.05).requires_grad_(True)
        b = (torch.randn(N, generator=tg) * 0.1).requires_grad_(True) if bias else None
        g = torch.randn(*M, N, generator=tg)
        rows = int(np.prod(M))
        noise = rand24(gen, rows * (-(-N // 32)) * 32)
        with fixed_noise(noise):
            y = fn(x, w, b, 32, qin, qgrad)
            y.backward(g.to(y.dtype))
        lstore[f"{name}.x"] = bits(x.detach()); lstore[f"{name}.w"] = bits(w.detach())
        if bias:
            lstore[f"{name}.b"] = bits(b.detach()); lstore[f"{name}.db"] = bits(b.grad.float())
        lstore[f"{name}.g"] = bits(g); lstore[f"{name}.noise"] = noise.numpy()
        lstore[f"{name}.y"] = bits(y.detach().float()); lstore[f"{name}.dx"] = bits(x.grad.float())
        lstore[f"{name}.dw"] = bits(w.grad.float())
        manifest["cases"][name] = {"M": list(M), "K": K, "N": N, "x_dtype": str(dtype).replace("torch.", ""),
                                   "y_dtype": str(y.dtype).replace("torch.", ""),
                                   "dx_dtype": str(x.grad.dtype).replace("torch.", ""),
                                   "dw_dtype": str(w.grad.dtype).replace("torch.", ""),
                                   "bias": bias, "quantize_input": qin, "quantize_grad": qgrad}

    for tag, fn in (("mixed", ref_mp.axs_linear_mixed_precision), ("unified", ref_fu.axs_linear_unified),
                    ("v1", ref_nnf.axs_linear)):
        add_linear(f"lin_{tag}_a", fn, (40,), 96, 64, torch.float32, True, True, True)
        add_linear(f"lin_{tag}_b", fn, (3, 16), 128, 32, torch.bfloat16 if tag == "mixed" else torch.float32,
                   False, True, False)
        add_linear(f"lin_{tag}_c", fn, (24,), 50, 24, torch.float32, True, False, True)
    np.savez_compressed(os.path.join(HERE, "linear_cases.npz"), **lstore)

    # ------------------------------------------------------------------ large-config hashes
    torch.manual_seed(0)
    x1 = torch.randn(1024, 1024) * 0.02
    manifest["hashes"]["config1.input"] = sha(x1)
    manifest["hashes"]["config1.fq_nf5"] = sha(ref_qu.fused_fake_quantize(x1))
    manifest["hashes"]["config1.fq_uniform"] = sha(ref_core.dequantize(ref_core.quantize(x1)))
    g2 = np.random.default_rng(2)
    x2 = g2.standard_normal((2048, 4096), dtype=np.float32)
    x2[g2.random((2048, 4096)) < 1e-3] *= 10
    x2[g2.random((2048, 4096)) < 1e-2] = 0
    x2 = torch.from_numpy(x2).to(torch.bfloat16)
    manifest["hashes"]["config2_quarter.input"] = sha(x2)
    q2 = ref_qu.quantize_unified(x2)
    wire2 = ref_dist._pack_to_flat_buffer(q2.shared_exponents, q2.signs, q2.magnitudes)
    manifest["hashes"]["config2_quarter.wire"] = sha(wire2.view(torch.uint8))
    manifest["hashes"]["config2_quarter.roundtrip"] = sha(ref_qu.dequantize_unified(q2))
    manifest["hashes"]["config2_quarter.fq_nf5"] = sha(ref_qu.fused_fake_quantize(x2))
    g3 = np.random.default_rng(3)
    sig = (10.0 ** (g3.random((4096, 1)) * 5 - 4)).astype(np.float32)
    x3 = torch.from_numpy(g3.standard_normal((4096, 4096), dtype=np.float32) * sig)
    manifest["hashes"]["config3_4096.input"] = sha(x3)
    manifest["hashes"]["config3_4096.fq_nf5_f32"] = sha(ref_qu.fused_fake_quantize(x3))
    manifest["hashes"]["config3_4096.fq_nf5_bf16"] = sha(ref_qu.fused_fake_quantize(x3.to(torch.bfloat16)))

    with open(os.path.join(HERE, "manifest.json"), "w") as f:
        json.dump(manifest, f, indent=1, sort_keys=True)
    print("cases:", len(manifest["cases"]))


if __name__ == "__main__":
    main()
