"""The bench's reference arm runs without a GPU: check that it prints exactly one JSON line with the
keys the measurement contract asks for (the GPU arm prints the same keys plus the device-side ones)."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def run_reference_arm(extra_env=None):
    env = dict(os.environ)
    env.update(extra_env or {})
    done = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--steps", "1", "--warmup",
                           "0", "--cpu-sample-tokens", "64"], capture_output=True, text=True, timeout=600, env=env,
                          cwd=ROOT)
    assert done.returncode == 0, done.stderr[-2000:]
    return [l for l in done.stdout.splitlines() if l.strip()]


def test_reference_arm_prints_one_json_line_with_the_contract_keys():
    lines = run_reference_arm()
    assert len(lines) == 1
    d = json.loads(lines[0])
    assert d["impl"] == "reference" and d["unit"] == "tokens/s" and d["higher_is_better"] is True
    assert d["value"] > 0 and d["ms_per_step"] > 0 and d["scaling"] == "strong" and d["vs_baseline"] is None
    assert d["config"]["workload"] and "model" not in d["config"]
    cpu = d["cpu_baseline"]
    assert cpu["kind"] in ("reference", "port") and cpu["cores"] >= 1 and "64-token sample" in cpu["sample"]
    assert cpu["extrapolated"] is False and cpu["sample_tokens"] == 64
    assert cpu["value"] == d["value"]
    assert d["e2e"] == {"value": d["value"], "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
    assert d["gpu_launches"] == 0


def test_reference_arm_runs_on_rank_zero_only():
    assert run_reference_arm({"RANK": "1", "WORLD_SIZE": "2", "LOCAL_RANK": "1"}) == []
