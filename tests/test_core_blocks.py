"""Per-block host utilities of axs6_b200.core against outputs recorded from the reference
(tests/golden/block_cases.npz, written by tests/golden/make_golden.py --only blocks from
axs/core.py:59-152, :214-286) and against the byte fixtures of AXSBlock.to_bytes.  CPU only."""
import os

import numpy as np
import pytest

from axs6_b200 import core

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


@pytest.fixture(scope="module")
def blocks():
    return np.load(os.path.join(GOLDEN, "block_cases.npz"))


def test_encode_decode_block_match_the_reference(blocks):
    n = int(blocks["count"][0])
    assert n >= 60, n
    for i in range(n):
        name = f"blk{i}"
        v = blocks[f"{name}.values"]
        stochastic = bool(blocks[f"{name}.rounding"][0])
        np.random.seed(int(blocks[f"{name}.seed"][0]))
        blk = core.axs_encode_block(v, "stochastic" if stochastic else "nearest")
        assert blk.shared_exponent == int(blocks[f"{name}.exponent"][0]), name
        assert blk.config == core.BlockConfig.DENSE and blk.block_size == len(v)
        assert np.array_equal(blk.signs, blocks[f"{name}.signs"]), name
        assert np.array_equal(blk.magnitudes, blocks[f"{name}.magnitudes"]), name
        assert blk.magnitudes.dtype == np.uint8 and blk.signs.dtype == bool
        by = blk.to_bytes()
        assert np.array_equal(np.frombuffer(by, dtype=np.uint8), blocks[f"{name}.bytes"]), name
        dec = core.axs_decode_block(blk)
        assert dec.dtype == np.float64
        assert np.array_equal(dec.view(np.uint64), blocks[f"{name}.decoded"].view(np.uint64)), name   # bit for bit, -0.0 included
        scale, bits_total, bpv = blocks[f"{name}.props"]
        assert blk.scale == scale and blk.total_bits == bits_total and blk.bits_per_value == bpv
        back = core.AXSBlock.from_bytes(by, len(v))
        assert back.shared_exponent == blk.shared_exponent and back.config == blk.config
        assert np.array_equal(back.signs, blk.signs) and np.array_equal(back.magnitudes, blk.magnitudes)


def test_block_bytes_match_the_spec_layout_fixtures(fq_cases, manifest):
    """AXSBlock.to_bytes on the reference's NF5 planes gives the recorded 26-byte records (and 8 / 14-byte ones for
    blocks of 8 / 16), and from_bytes inverts them."""
    seen = 0
    for name, info in manifest["cases"].items():
        key = f"{name}.nf5.spec"
        if key not in fq_cases.files:
            continue
        B = info["block"]
        se, sg, mg = fq_cases[f"{name}.nf5.se"], fq_cases[f"{name}.nf5.sign"], fq_cases[f"{name}.nf5.mag"]
        rec = 2 + (6 * B + 7) // 8
        want = fq_cases[key].reshape(-1, rec)
        se, sg, mg = se.reshape(-1), sg.reshape(-1, B), mg.reshape(-1, B)
        assert want.shape[0] == se.shape[0]
        for b in range(0, se.shape[0], max(1, se.shape[0] // 16)):          # a sample of blocks per case
            blk = core.AXSBlock(int(se[b]), core.BlockConfig.DENSE, sg[b].astype(bool), mg[b], B)
            by = blk.to_bytes()
            assert np.array_equal(np.frombuffer(by, dtype=np.uint8), want[b]), (name, b)
            back = core.AXSBlock.from_bytes(by, B)
            assert back.shared_exponent == int(se[b]) and np.array_equal(back.magnitudes, mg[b])
            assert np.array_equal(back.signs, sg[b].astype(bool))
            seen += 1
    assert seen > 100


def test_block_config_and_validation():
    assert [int(c) for c in core.BlockConfig] == [0, 1, 2, 3]
    assert core.BlockConfig(2) is core.BlockConfig.HIGH_PREC
    with pytest.raises(AssertionError):
        core.axs_encode_block(np.zeros(7))
    z = core.axs_encode_block(np.zeros(16))
    assert z.shared_exponent == 0 and not z.signs.any() and not z.magnitudes.any()
    import axs6_b200
    for name in ("AXSBlock", "BlockConfig", "axs_encode_block", "axs_decode_block", "quantization_error", "RoundingMode",
                 "quantize_nearest", "quantize_stochastic", "quantize_with_error_feedback"):
        assert hasattr(axs6_b200, name)
