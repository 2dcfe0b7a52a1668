"""bench.py's reference arm runs without a GPU: one JSON line with the contract's keys, the whole configuration-2
workload per step on the host cores; under a multi-rank launch only rank 0 prints."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(extra_env=None, *args):
    env = dict(os.environ)
    env.pop("RANK", None)
    env.pop("WORLD_SIZE", None)
    env.update(extra_env or {})
    return subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", *args],
                          capture_output=True, text=True, env=env, timeout=600, cwd=ROOT)


def test_reference_arm_prints_one_contract_line():
    done = _run(None, "--steps", "1", "--warmup", "0")
    assert done.returncode == 0, done.stderr[-2000:]
    lines = [ln for ln in done.stdout.splitlines() if ln.startswith("{")]
    assert len(lines) == 1
    d = json.loads(lines[0])
    assert d["impl"] == "reference" and d["higher_is_better"] is True and d["n_gpus"] == 1
    assert d["steps"] == 1 and d["unit"] == "TFLOP/s" and d["value"] > 0 and d["ms_per_step"] > 0
    assert d["config"]["workload"] == "mxfp8_glu_mlp_fwd_m8192_k4096_i14336"
    assert d["vs_baseline"] is None and d["data"] == "synthetic"
    base = d["cpu_baseline"]
    assert base["kind"] in ("port", "reference") and base["cores"] >= 1 and base["sample"] and base["value"] == d["value"]
    e2e = d["e2e"]
    assert e2e["value"] == d["value"] and e2e["unit"] == d["unit"]
    assert e2e["h2d_bytes_per_step"] == 0 and e2e["d2h_bytes_per_step"] == 0
    # whole workload per step: 2.886e12 flop in ms_per_step
    assert abs(d["value"] - 2.886e12 / (d["ms_per_step"] * 1e-3) / 1e12) / d["value"] < 0.01


def test_reference_arm_is_silent_on_other_ranks():
    done = _run({"RANK": "1", "WORLD_SIZE": "2", "LOCAL_RANK": "1"}, "--gpus", "2", "--steps", "1", "--warmup", "0")
    assert done.returncode == 0, done.stderr[-2000:]
    assert not [ln for ln in done.stdout.splitlines() if ln.startswith("{")]
