"""The reference arm of bench.py, run for real on the host cores: one JSON line with the keys the benchmark contract
names, for exactly the steps asked for.  (The GPU arm needs a B200; its line has the same keys plus `roofline`,
`clocks`, `latency_us` and `stages`.)"""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_reference_arm_prints_the_contract_line():
    res = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--steps", "1", "--warmup", "0"],
                         cwd=ROOT, capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stderr[-2000:]
    lines = [ln for ln in res.stdout.splitlines() if ln.strip()]
    assert len(lines) == 1
    out = json.loads(lines[0])
    assert out["impl"] == "reference" and out["steps"] == 1 and out["warmup"] == 0 and out["n_gpus"] == 1
    assert out["metric"] == "bert_base_12layer_seq128_batch64_sequences_per_second" and out["unit"] == "sequences/s"
    assert out["higher_is_better"] is True and out["vs_baseline"] is None and out["gpu_launches"] == 0
    assert 0 < out["value"] < 1e4 and abs(out["value"] - 64 / (out["ms_per_step"] * 1e-3)) < 1e-6 * out["value"]
    assert out["cpu_baseline"]["kind"] == "port" and out["cpu_baseline"]["cores"] >= 1 and out["cpu_baseline"]["value"] == out["value"]
    assert out["e2e"] == {"value": out["value"], "unit": "sequences/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
    assert "workload" in out["config"] and "model" not in out["config"]


def test_reference_arm_is_silent_on_other_ranks():
    env = dict(os.environ, RANK="1", LOCAL_RANK="1", WORLD_SIZE="2", MASTER_ADDR="127.0.0.1", MASTER_PORT="29599")
    res = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--gpus", "2", "--steps", "1",
                          "--warmup", "0"], cwd=ROOT, env=env, capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stderr[-2000:]
    assert res.stdout.strip() == ""
