"""The C-ABI library loads and exports every symbol the public header declares, and the ctypes
binding covers the same set (no compute calls: runs without a GPU)."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    names = set()
    inc = os.path.join(ROOT, "include")
    for f in os.listdir(inc):
        if f.endswith(".h"):
            text = open(os.path.join(inc, f)).read()
            text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
            names |= set(re.findall(r"\b(axs6_[a-z0-9_]+)\s*\(", text))
    return sorted(names)


def test_header_declares_the_hot_path():
    names = declared_symbols()
    for must in ("axs6_fq", "axs6_fq_with_noise", "axs6_pack", "axs6_unpack", "axs6_strerror", "axs6_query"):
        assert must in names


def test_library_exports_every_declared_symbol():
    from axs6_b200 import _lib, build
    path = build.build()
    lib = ctypes.CDLL(path)
    for name in declared_symbols():
        assert hasattr(lib, name), f"{name} declared in include/ but not exported"
    assert set(_lib.SIGNATURES) == set(declared_symbols())


def test_host_only_entry_points():
    from axs6_b200 import _lib
    lib = _lib.load()
    assert lib.axs6_strerror(0) == b"ok"
    assert lib.axs6_strerror(-3).decode().startswith("current CUDA device")
    assert lib.axs6_record_bytes(1, 32) == 25 and lib.axs6_record_bytes(2, 32) == 26
    assert lib.axs6_record_bytes(1, 16) == 13 and lib.axs6_record_bytes(2, 8) == 8
    assert lib.axs6_record_bytes(1, 12) == 0
    assert lib.axs6_query(2) >= 1


def test_ops_reject_cpu_tensors():
    import torch
    import importlib
    qu = importlib.import_module("axs6_b200.unified.quantize_unified")
    from axs6_b200 import core
    with pytest.raises(RuntimeError, match="requires a CUDA tensor"):
        qu.fused_fake_quantize(torch.randn(4, 32))
    with pytest.raises(RuntimeError, match="requires a CUDA tensor"):
        core.quantize(torch.randn(4, 32))


def test_product_never_imports_the_oracle():
    """The oracle is test infrastructure: nothing under the package may reference it."""
    pkg = os.path.join(ROOT, "axs6_b200")
    for root, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h")):
                text = open(os.path.join(root, f)).read()
                assert not re.search(r"^\s*(import|from)\s+oracle\b", text, flags=re.M), f
                assert "liboracle" not in text, f


def test_unified_package_exports_the_reference_names():
    """Every public name of the reference's ``axs.unified`` (its ``__all__``, axs/unified/__init__.py:80-127)
    exists in ``axs6_b200.unified``, so `import axs6_b200.unified as unified` needs no further edits."""
    import axs6_b200.unified as u
    names = ["fused_fake_quantize", "quantize_unified", "dequantize_unified", "quantization_error_unified",
             "FUSED_NF5_LUT", "NF5_CODEBOOK", "REVERSE_NF5_LUT", "fake_quantize_unified", "axs_linear_unified",
             "axs_matmul_unified", "AXSLinearUnified", "AXSLayerNormUnified", "AXSEmbeddingUnified",
             "AXSMultiheadAttentionUnified", "convert_to_axs_unified", "AXSTrainingPipelineUnified", "AmaxEMA",
             "BackendType", "accelerated_fake_quantize", "accelerated_linear", "accelerated_matmul", "backend_info",
             "clear_int8_weight_cache", "detect_best_backend", "get_backend", "set_backend", "has_triton",
             "triton_fused_fake_quantize", "triton_fused_linear", "AXSLinearMixedPrecision",
             "axs_linear_mixed_precision", "convert_to_axs_mixed_precision", "estimate_memory_savings",
             "AXS6GradCompressor", "axs6_gradient_hook", "axs6_gradient_hook_packed"]
    missing = [n for n in names if not hasattr(u, n)]
    assert not missing, missing
    assert set(names) <= set(u.__all__)
    u.clear_int8_weight_cache()
    assert u.detect_best_backend() == u.get_backend()


def test_environment_knobs_are_applied_and_checked():
    """AXS6_TUNE="key=value,..." is handed to axs6_tune when the library is loaded; a key outside the table is an error."""
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    code = "from axs6_b200 import _lib; _lib.load(); print('loaded')"
    ok = subprocess.run([sys.executable, "-c", code], cwd=root, env=dict(os.environ, AXS6_TUNE="8=32,15=1"),
                        capture_output=True, text=True, timeout=300)
    assert ok.returncode == 0 and "loaded" in ok.stdout, ok.stderr[-1000:]
    bad = subprocess.run([sys.executable, "-c", code], cwd=root, env=dict(os.environ, AXS6_TUNE="99=1"),
                         capture_output=True, text=True, timeout=300)
    assert bad.returncode != 0 and "AXS6_TUNE" in bad.stderr
