"""CPU checks of the benchmark's host logic: the reference arm's JSON line and the same-GPU comparator's
behaviour when no copy of the reference is present."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_reference_arm_prints_the_contract_line():
    env = dict(os.environ)
    env.pop("RANK", None)
    env.pop("WORLD_SIZE", None)
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--steps", "1", "--warmup", "1"],
                         cwd=ROOT, env=env, capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stderr[-2000:]
    line = json.loads(out.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference"
    for key in ("metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "config",
                "cpu_baseline", "e2e"):
        assert key in line, key
    assert line["metric"] == "axs6_fake_quant_GBps" and line["unit"] == "GB/s"
    assert line["value"] > 0 and line["e2e"]["value"] == line["value"]
    assert line["e2e"]["h2d_bytes_per_step"] == 0 and line["e2e"]["d2h_bytes_per_step"] == 0
    cpu = line["cpu_baseline"]
    assert cpu["kind"] in ("reference", "port") and cpu["cores"] >= 1 and "sample" in cpu


def test_same_gpu_comparator_reports_a_missing_reference(monkeypatch, tmp_path):
    sys.path.insert(0, ROOT)
    try:
        import bench_gpu_reference
    finally:
        sys.path.pop(0)
    monkeypatch.setattr(bench_gpu_reference, "REF_DIR", str(tmp_path / "nothing_here"))
    res = bench_gpu_reference.run(None, None, 1.0)
    assert "unavailable" in res and "baseline/_ref" in res["unavailable"]
