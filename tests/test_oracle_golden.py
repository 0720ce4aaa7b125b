"""Pins the CPU oracle (oracle/) to the reference: every fixture under tests/golden/ was
produced by running the reference itself (tests/golden/make_golden.py)."""
import numpy as np
import pytest

import oracle
from helpers import (bits_equal, case_input, config1_input, config2_input, config3_input,
                     expect_bits, fq_case_names, sha)


def test_tables_match_reference(tables, manifest):
    assert bits_equal(oracle.NF5_CODEBOOK, tables["codebook"])
    assert bits_equal(oracle.FUSED_NF5_LUT, tables["lut"])
    assert np.array_equal(oracle.REVERSE_NF5_LUT, tables["reverse"])
    assert sha(oracle.NF5_CODEBOOK) == manifest["hashes"]["NF5_CODEBOOK"]
    assert sha(oracle.FUSED_NF5_LUT) == manifest["hashes"]["FUSED_NF5_LUT"]
    assert sha(oracle.REVERSE_NF5_LUT) == manifest["hashes"]["REVERSE_NF5_LUT"]
    # the LUT is the codebook gathered through the reverse table
    assert bits_equal(oracle.FUSED_NF5_LUT, oracle.NF5_CODEBOOK[oracle.REVERSE_NF5_LUT])


def test_log2_bump_set_exhaustive(manifest):
    """Scan all 2^31 positive floats: the inputs whose block exponent is one above the true
    exponent must be exactly the set recorded from torch's fp32 log2."""
    import os
    golden = np.load(os.path.join(os.path.dirname(__file__), "golden", "log2_bump_set.npy"))
    assert sha(golden) == manifest["hashes"]["log2_bump_set"]
    got = oracle.log2_bump_scan()
    assert np.array_equal(got, golden)


def _all_cases(manifest):
    return fq_case_names(manifest)


def pytest_generate_tests(metafunc):
    if "case" in metafunc.fixturenames:
        import json, os
        with open(os.path.join(os.path.dirname(__file__), "golden", "manifest.json")) as f:
            m = json.load(f)
        metafunc.parametrize("case", fq_case_names(m))


def test_fake_quantize_nf5(case, fq_cases, manifest):
    x, noise, info = case_input(fq_cases, manifest, case)
    y = oracle.fused_fake_quantize(x, info["block"], noise)
    assert bits_equal(y, expect_bits(fq_cases, case, "fq_nf5", y))


@pytest.mark.parametrize("grid,tag", [(oracle.GRID_NF5, "nf5"), (oracle.GRID_UNIFORM, "uni")])
def test_quantize_planes_and_dequantize(case, grid, tag, fq_cases, manifest):
    x, noise, info = case_input(fq_cases, manifest, case)
    se, sg, mg = oracle.quantize(x, info["block"], grid, noise)
    assert np.array_equal(se, fq_cases[f"{case}.{tag}.se"].reshape(se.shape))
    assert np.array_equal(mg, fq_cases[f"{case}.{tag}.mag"].reshape(mg.shape))
    assert np.array_equal(sg, fq_cases[f"{case}.{tag}.sign"].reshape(sg.shape))
    x2 = x.reshape(-1, x.shape[-1])
    y = oracle.dequantize(se, sg, mg, x2.shape[1], grid).reshape(x.shape)
    assert bits_equal(y, expect_bits(fq_cases, case, f"deq_{tag}", y))


def test_byte_layouts(case, fq_cases, manifest):
    if f"{case}.nf5.wire" not in fq_cases.files:
        pytest.skip("no byte-layout fixture for this case")
    x, noise, info = case_input(fq_cases, manifest, case)
    B = info["block"]
    se, sg, mg = oracle.quantize(x, B, oracle.GRID_NF5)
    wire = oracle.pack_bytes(se, sg, mg, oracle.LAYOUT_WIRE)
    assert np.array_equal(wire, fq_cases[f"{case}.nf5.wire"])
    se2, sg2, mg2 = oracle.unpack_bytes(wire, se.shape[0], se.shape[1], B, oracle.LAYOUT_WIRE)
    assert np.array_equal(se, se2) and np.array_equal(sg, sg2) and np.array_equal(mg, mg2)
    if f"{case}.nf5.spec" in fq_cases.files:
        spec = oracle.pack_bytes(se, sg, mg, oracle.LAYOUT_SPEC)
        assert np.array_equal(spec, fq_cases[f"{case}.nf5.spec"])
        se3, sg3, mg3 = oracle.unpack_bytes(spec, se.shape[0], se.shape[1], B, oracle.LAYOUT_SPEC)
        assert np.array_equal(se, se3) and np.array_equal(sg, sg3) and np.array_equal(mg, mg3)


def test_config1_hashes(manifest):
    x = config1_input()
    if sha(x) != manifest["hashes"]["config1.input"]:
        pytest.skip("torch RNG stream differs from the one the fixture was made with")
    assert sha(oracle.fused_fake_quantize(x)) == manifest["hashes"]["config1.fq_nf5"]
    assert sha(oracle.fake_quantize_uniform(x)) == manifest["hashes"]["config1.fq_uniform"]


def test_config2_quarter_hashes(manifest):
    xb = oracle.f32_to_bf16(config2_input(2048, 4096))
    assert sha(xb) == manifest["hashes"]["config2_quarter.input"]
    se, sg, mg = oracle.quantize(xb, 32, oracle.GRID_NF5)
    wire = oracle.pack_bytes(se, sg, mg, oracle.LAYOUT_WIRE)
    assert sha(wire) == manifest["hashes"]["config2_quarter.wire"]
    se2, sg2, mg2 = oracle.unpack_bytes(wire, 2048, 128, 32, oracle.LAYOUT_WIRE)
    assert sha(oracle.dequantize(se2, sg2, mg2, 4096, oracle.GRID_NF5)) == manifest["hashes"]["config2_quarter.roundtrip"]
    assert sha(oracle.fused_fake_quantize(xb)) == manifest["hashes"]["config2_quarter.fq_nf5"]


def test_config3_hashes(manifest):
    x = config3_input(4096, 4096)
    assert sha(x) == manifest["hashes"]["config3_4096.input"]
    assert sha(oracle.fused_fake_quantize(x)) == manifest["hashes"]["config3_4096.fq_nf5_f32"]
    assert sha(oracle.fused_fake_quantize(oracle.f32_to_bf16(x))) == manifest["hashes"]["config3_4096.fq_nf5_bf16"]
