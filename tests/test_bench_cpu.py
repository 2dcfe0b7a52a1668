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


def test_clock_sampler_assigns_samples_to_marked_regions(tmp_path):
    """bench.py's sampler: nvidia-smi lines whose timestamp falls inside a marked region count for that label;
    median clock, power and the active throttle reasons come out per label."""
    import datetime
    import importlib.util

    spec = importlib.util.spec_from_file_location("bench_under_test", os.path.join(ROOT, "bench.py"))
    bench = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(bench)

    class _Done:
        def terminate(self): pass
        def wait(self, timeout=None): return 0
        def kill(self): pass

    t0 = datetime.datetime(2026, 1, 2, 3, 4, 5).timestamp()
    stamp = lambda dt: datetime.datetime.fromtimestamp(t0 + dt).strftime("%Y/%m/%d %H:%M:%S.%f")[:-3]
    rows = [(0.00, 1965, 300, "Not Active"), (0.01, 1950, 310, "Not Active"), (0.02, 1900, 320, "Active"),
            (1.00, 1300, 990, "Active"), (1.01, 1290, 995, "Active"), (5.00, 210, 90, "Not Active")]
    path = tmp_path / "smi.csv"
    path.write_text("".join(f"{stamp(dt)}, {mhz}, 1965, {w}, Not Active, Not Active, Not Active, {cap}\n"
                            for dt, mhz, w, cap in rows) + "garbage line\n")
    s = bench.ClockSampler(0)
    s.proc, s.path = _Done(), str(path)
    s.mark("burst", t0 - 0.001, t0 + 0.025)
    s.mark("sustained", t0 + 0.99, t0 + 1.02)
    out = s.stop()
    assert out["burst"]["samples"] == 3 and out["burst"]["sm_mhz"] == 1950 and out["burst"]["sm_max_mhz"] == 1965
    assert out["burst"]["reasons"] == ["sw_power_cap"] and out["burst"]["power_w"] == 310
    assert out["sustained"]["samples"] == 2 and out["sustained"]["sm_mhz"] == 1295 and out["sustained"]["samples_total"] == 6
    assert not os.path.exists(path)          # the sampler removes its file
