"""Autotune campaigns (rtx_b200/campaign.py) without a GPU: manifest parsing in the reference's format
(rtx/autotune/dataset.py:224-440), the search / confirm / gate / install sequence with a scripted clock, and
that an installed winner is what a module with autotune="cache" resolves."""

import json

import pytest

from rtx_b200 import autotune, campaign
from rtx_b200.configs import MXFP8GemmConfig, MXFP8PrequantConfig

MANIFEST = {
    "schema_version": 2, "name": "unit_campaign", "seed": 11,
    "jobs": [
        {"family": "mxfp8_prequant_fwd",
         "shapes": [{"m": 512, "n": 1024, "k": 1024, "name": "proj"}, {"m": 64, "n": 1024, "k": 1024}],
         "regimes": ["hot"], "promote": 2,
         "tuning": {"max_trials": 192, "cost_model_trials": 72},
         "protocol": {"warmup_calls": 3, "samples": 5, "confirm_samples": 9, "telemetry": True}},
        {"family": "mxfp8_bwd", "shapes": [{"m": 512, "n": 1024, "k": 1024}], "regimes": ["hot"], "promote": 1},
    ],
}


def test_manifest_parsing_and_validation():
    m = campaign.Manifest.from_dict(MANIFEST)
    assert m.name == "unit_campaign" and m.seed == 11 and len(m.jobs) == 2
    job = m.jobs[0]
    assert job.family == "mxfp8_prequant_fwd" and job.promote == 2
    assert job.shapes[0] == campaign.ShapeSpec(512, 1024, 1024, "proj") and job.shapes[1].label == "m64_n1024_k1024"
    assert job.protocol == campaign.Protocol(3, 5, 9)
    assert job.tuning["max_trials"] == 192          # recorded, not used
    for bad in ({**MANIFEST, "schema_version": 9}, {**MANIFEST, "name": "../x"},
                {**MANIFEST, "jobs": [{"family": "nope", "shapes": []}]},
                {**MANIFEST, "jobs": [{"family": "mxfp8_bwd", "shapes": [{"m": 0, "n": 1, "k": 1}]}]},
                {**MANIFEST, "jobs": [{"family": "mxfp8_bwd", "shapes": [], "regimes": ["cold"]}]},
                {**MANIFEST, "jobs": [{"family": "mxfp8_bwd", "shapes": [], "promote": 0}]}):
        with pytest.raises(ValueError):
            campaign.Manifest.from_dict(bad)


class _Clock:
    """Scripted timings per schedule; counts the calls of each phase."""

    def __init__(self, ms_by_schedule):
        self.ms, self.calls = ms_by_schedule, []

    def measure(self, run, warmup, samples):
        schedule = run()
        self.calls.append((schedule, warmup, samples))
        ms = self.ms.get(schedule)
        if ms is None:
            return autotune.TrialOutcome("failed", detail="scripted failure")
        return autotune.TrialOutcome("ok", median_ms=ms)


def _fake_build(outputs):
    def build(family, shape, regime, seed, device="cpu"):
        adapter = autotune.ADAPTERS["mxfp8_prequant_fwd"]()
        ctx = autotune.KernelContext("mxfp8_prequant_fwd", shape.m, shape.n, shape.k, regime=regime)
        return campaign.Target(ctx, adapter, MXFP8PrequantConfig(), lambda cfg: (lambda: cfg.gemm.schedule),
                               output=lambda cfg: outputs.get(cfg.gemm.schedule, "same"))
    return build


def test_campaign_search_confirm_gate_install(tmp_path):
    clock = _Clock({"auto": 1.0, "single": 1.2, "pair": 0.8, "stream": 0.5, "fused_x": 3.0})
    # "stream" is fastest but produces different bits -> the gate rejects it and the next finalist wins
    summary = campaign.run_campaign(campaign.Manifest.from_dict(MANIFEST), tmp_path / "out", cache_dir=tmp_path / "cache",
                                    build=_fake_build({"stream": "different"}), measure=clock.measure,
                                    same=lambda a, b: a == b)
    assert summary["skipped"] == [{"family": "mxfp8_bwd", "shapes": 1, "why": "one schedule per launch: nothing to choose"}]
    big, small = summary["targets"]
    assert big["shape"] == "proj" and json.loads(big["winner"])["gemm"]["schedule"] == "pair"
    assert big["gain"] == pytest.approx(1.0 / 0.8) and "installed" in big
    # M = 64 admits the streaming schedule; M = 512 does not (rejected before any timing)
    searched_big = clock.calls[:4]
    assert {c[0] for c in searched_big} == {"auto", "single", "pair", "fused_x"}
    assert all(c[1:] == (3, 5) for c in searched_big)
    # confirmation: the two fastest plus the configured schedule, with the confirmation sample count
    assert clock.calls[4:6] == [("pair", 3, 9), ("auto", 3, 9)]
    assert json.loads(small["winner"])["gemm"]["schedule"] == "pair"   # stream failed the gate
    trials = [json.loads(l) for l in open(tmp_path / "out" / "unit_campaign" / "trials.jsonl")]
    assert {t["phase"] for t in trials} == {"search", "confirm", "gate"}
    gate = [t for t in trials if t["phase"] == "gate"]
    assert len(gate) == 1 and json.loads(gate[0]["config_key"])["gemm"]["schedule"] == "stream"
    assert json.load(open(tmp_path / "out" / "unit_campaign" / "summary.json"))["targets"][0]["winner"] == big["winner"]

    # the installed winner is what a frontend resolves with autotune="cache"
    res = autotune.ScheduleResolver("mxfp8_prequant_fwd", 1024, 1024, "cache", tmp_path / "cache")
    assert res.resolve(512, MXFP8PrequantConfig()).gemm == MXFP8GemmConfig.for_schedule("pair")
    assert res.sources[512] == "stored winner"
    assert res.resolve(256, MXFP8PrequantConfig()).gemm.schedule == "auto"   # no campaign covered this M


def test_campaign_min_gain_failed_trials_and_dry_run(tmp_path):
    clock = _Clock({"auto": 1.0, "single": 0.99, "pair": None, "fused_x": None, "stream": None})
    summary = campaign.run_campaign(campaign.Manifest.from_dict(MANIFEST), tmp_path / "o", cache_dir=tmp_path / "c",
                                    build=_fake_build({}), measure=clock.measure, same=lambda a, b: a == b, min_gain=1.05)
    t = summary["targets"][0]
    assert json.loads(t["winner"])["gemm"]["schedule"] == "single" and "installed" not in t   # 1 % is below the bar
    trials = [json.loads(l) for l in open(tmp_path / "o" / "unit_campaign" / "trials.jsonl")]
    assert any(x["status"] == "failed" and x["detail"] == "scripted failure" for x in trials)

    nothing = _Clock({})
    summary = campaign.run_campaign(campaign.Manifest.from_dict(MANIFEST), tmp_path / "o2", build=_fake_build({}),
                                    measure=nothing.measure)
    assert summary["targets"][0]["decision"] == "no candidate ran"

    dry = campaign.run_campaign(campaign.Manifest.from_dict(MANIFEST), tmp_path / "o3", dry_run=True,
                                families=["mxfp8_prequant_fwd"])
    assert len(dry["targets"]) == 2 and dry["skipped"] == []
    assert len(dry["targets"][1]["candidates"]) == len(dry["targets"][0]["candidates"]) + 1   # + stream at M = 64
    assert not (tmp_path / "o3" / "unit_campaign" / "trials.jsonl").exists()


def test_campaign_cli_dry_run(tmp_path, capsys):
    path = tmp_path / "m.json"
    path.write_text(json.dumps(MANIFEST))
    assert campaign.main([str(path), "--out", str(tmp_path / "out"), "--dry-run"]) == 0
    line = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert line == {"manifest": "unit_campaign", "targets": 2, "installed": 0,
                    "skipped": [{"family": "mxfp8_bwd", "shapes": 1, "why": "one schedule per launch: nothing to choose"}]}
