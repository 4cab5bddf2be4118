"""bench.py on a machine without a GPU: the reference (CPU) arm prints one well-formed JSON
line, ranks other than 0 stay silent, and the timing helpers that need no GPU behave."""
import json
import os
import subprocess
import sys

from tests.conftest import ROOT


def _run(extra_env=None, *args):
    env = dict(os.environ)
    env.update(extra_env or {})
    return subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), *args], capture_output=True, text=True,
                          env=env, timeout=600)


def test_reference_arm_prints_one_json_line():
    r = _run(None, "--impl", "reference", "--steps", "1", "--warmup", "0")
    assert r.returncode == 0, r.stderr[-500:]
    lines = [l for l in r.stdout.strip().splitlines() if l.startswith("{")]
    assert len(lines) == 1
    d = json.loads(lines[0])
    assert d["impl"] == "reference" and d["unit"] == "TFLOP/s" and d["higher_is_better"] is True
    assert d["metric"] == "bf16 GEMM TFLOPS @8192^3" and d["value"] > 0
    assert d["config"]["workload"].startswith("gemm_bf16_8192x8192x8192")
    assert d["cpu_baseline"]["kind"] == "port" and d["cpu_baseline"]["cores"] >= 1
    assert d["cpu_baseline"]["value"] == d["value"]
    assert d["e2e"] == {"value": d["value"], "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}


def test_reference_arm_is_silent_on_other_ranks():
    r = _run({"RANK": "1", "WORLD_SIZE": "2"}, "--impl", "reference", "--steps", "1", "--warmup", "0")
    assert r.returncode == 0 and r.stdout.strip() == ""


def test_reference_arm_uses_all_cores_under_torchrun_env():
    r = _run({"OMP_NUM_THREADS": "1"}, "--impl", "reference", "--steps", "1", "--warmup", "0")
    d = json.loads(r.stdout.strip().splitlines()[-1])
    import bench
    assert d["cpu_baseline"]["cores"] == bench.host_cores()


def test_own_arm_fails_loudly_without_a_gpu():
    import torch
    if torch.cuda.is_available():
        return
    r = _run(None, "--steps", "1", "--warmup", "1")
    assert r.returncode != 0 and "no CUDA device" in (r.stderr + r.stdout)


def test_peaks_loader_has_a_stated_fallback(tmp_path, monkeypatch):
    import bench
    peaks, kind = bench.load_peaks()
    assert set(peaks) == {"hbm_gbs", "bf16_tflops", "bf16_tflops_sustained"} and kind in ("measured", "fallback")
    monkeypatch.setattr(bench, "ROOT", str(tmp_path))
    peaks, kind = bench.load_peaks()
    assert kind == "fallback" and peaks == bench.FALLBACK_PEAKS
