"""The reference arm of ``bench.py`` (the CPU restatement timed on the host cores) runs without a
GPU; its JSON line carries the keys the measurement contract names."""

import json
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent


def test_reference_arm_prints_one_contract_line():
    p = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--impl", "reference", "--steps", "1", "--warmup", "0"],
                       capture_output=True, text=True, timeout=600, cwd=str(ROOT))
    assert p.returncode == 0, p.stderr[-2000:]
    lines = [l for l in p.stdout.splitlines() if l.startswith("{")]
    assert len(lines) == 1
    r = json.loads(lines[0])
    assert r["impl"] == "reference" and r["n_gpus"] == 1 and r["steps"] == 1 and r["warmup"] == 0
    assert r["unit"] == "GB/s" and r["higher_is_better"] is True and r["vs_baseline"] is None
    assert r["value"] > 0 and r["ms_per_step"] > 0 and r["gpu_launches"] == 0
    assert r["data"] == "synthetic" and "workload" in r["config"] and "model" not in r["config"]
    cb = r["cpu_baseline"]
    assert cb["kind"] == "port" and cb["cores"] >= 1 and cb["value"] == r["value"] and cb["sample"]
    e = r["e2e"]
    assert e["value"] == r["value"] and e["unit"] == r["unit"]
    assert e["h2d_bytes_per_step"] == 0 and e["d2h_bytes_per_step"] == 0


def _bench(extra_args, env_extra=None):
    import os
    env = dict(os.environ)
    env.update(env_extra or {})
    return subprocess.run([sys.executable, str(ROOT / "bench.py"), *extra_args], capture_output=True, text=True,
                          timeout=600, cwd=str(ROOT), env=env)


def test_reference_arm_runs_on_rank_zero_only():
    p = _bench(["--impl", "reference", "--gpus", "2", "--steps", "1", "--warmup", "0"],
               {"RANK": "1", "LOCAL_RANK": "1", "WORLD_SIZE": "2"})
    assert p.returncode == 0, p.stderr[-2000:]
    assert not [l for l in p.stdout.splitlines() if l.startswith("{")]


def test_product_arm_refuses_to_run_without_a_gpu():
    import torch
    if torch.cuda.is_available():
        import pytest
        pytest.skip("a GPU is present")
    p = _bench(["--steps", "1", "--warmup", "3"])
    assert p.returncode != 0 and "no CPU fallback" in (p.stderr + p.stdout)
