"""Autotune campaigns over the reference's shape manifests.

A manifest is the reference's campaign file (autotune_manifests/*.json, parsed by
rtx/autotune/dataset.py:224-440): `{"schema_version": 2, "name", "seed", "jobs": [{"family", "shapes":
[{"m", "n", "k", "name"}], "regimes": ["hot" | "rotate"], "promote", "tuning", "protocol"}]}`.  A campaign
times every legal schedule of a family on every shape, confirms the best few with more samples, checks that
the winner's output equals the configured schedule's output bit for bit, and installs it in the runtime
winner store that `autotune="cache"` on the modules reads (rtx/autotune/promotion.py:111-…,
rtx/autotune/winners.py:117-170).  Every trial is appended to `<out>/<manifest name>/trials.jsonl`.

The candidate space here is the handful of built kernels, so the search is exhaustive: the manifest's
`tuning` block (trial limits, cost-model and bandit settings of the reference's search engine) is read and
recorded but drives nothing.  `protocol.warmup_calls`, `protocol.samples`, `protocol.confirm_samples` and
`promote` (how many candidates go to confirmation) are honoured.

    python -m rtx_b200.campaign MANIFEST.json --out DIR [--cache-dir DIR] [--family F ...] [--dry-run]
"""

from __future__ import annotations

import argparse
import json
import sys
import time
from dataclasses import dataclass, field
from pathlib import Path
from typing import Any, Callable, Iterable, Mapping, Optional, Sequence

from .autotune import ADAPTERS, KernelContext, save_runtime_winner, time_call

SUPPORTED_SCHEMA_VERSIONS = (1, 2)
REGIMES = ("hot", "rotate")
# manifest family -> (module kind, weight packed?, NVFP4 scaling policy)
FAMILY_TARGETS = {
    "mxfp8_fused_fwd": ("mxfp8", False, None),
    "mxfp8_prequant_fwd": ("mxfp8", False, None),
    "mxfp8_weight_prequant_fwd": ("mxfp8", True, None),
    "nvfp4_dynamic_fwd": ("nvfp4", False, "current"),
    "nvfp4_jit_row_region_fwd": ("nvfp4", False, "jit_row_region"),
    "nvfp4_delayed_fwd": ("nvfp4", False, "delayed"),
    "nvfp4_weight_prequant_fwd": ("nvfp4", True, "current"),
}
# families of the reference with no schedule choice behind them here: both operands packed (the caller picks
# the kernel with the library's schedule switch) and the backward (one schedule per GEMM)
UNTUNED_FAMILIES = ("mxfp8_fully_prequant_fwd", "nvfp4_fully_prequant_fwd", "mxfp8_bwd")
L2_BYTES = 126 << 20


@dataclass(frozen=True)
class ShapeSpec:
    m: int
    n: int
    k: int
    name: str = ""

    @property
    def label(self) -> str:
        return self.name or f"m{self.m}_n{self.n}_k{self.k}"


@dataclass(frozen=True)
class Protocol:
    warmup_calls: int = 5
    samples: int = 7
    confirm_samples: int = 21

    @classmethod
    def from_dict(cls, d: Optional[Mapping[str, Any]]) -> "Protocol":
        d = d or {}
        out = cls(int(d.get("warmup_calls", 5)), int(d.get("samples", 7)), int(d.get("confirm_samples", 21)))
        if out.warmup_calls < 0 or out.samples < 1 or out.confirm_samples < 1:
            raise ValueError("protocol needs warmup_calls >= 0 and at least one sample per phase")
        return out


@dataclass(frozen=True)
class Job:
    family: str
    shapes: tuple
    regimes: tuple = ("hot",)
    promote: int = 2
    protocol: Protocol = field(default_factory=Protocol)
    tuning: Mapping[str, Any] = field(default_factory=dict)
    tags: tuple = ()


@dataclass(frozen=True)
class Manifest:
    name: str
    seed: int
    jobs: tuple

    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "Manifest":
        version = d.get("schema_version", 1)
        if version not in SUPPORTED_SCHEMA_VERSIONS:
            raise ValueError(f"manifest schema_version {version!r} is not supported")
        name = str(d.get("name") or "")
        if not name or any(c in name for c in "/\\") or ".." in name:
            raise ValueError("a manifest needs a name that is a safe path component")
        jobs = []
        for j in d.get("jobs") or ():
            family = j.get("family")
            if family not in FAMILY_TARGETS and family not in UNTUNED_FAMILIES:
                raise ValueError(f"unknown kernel family {family!r}")
            shapes = []
            for s in j.get("shapes") or ():
                m, n, k = int(s["m"]), int(s["n"]), int(s["k"])
                if min(m, n, k) < 1:
                    raise ValueError(f"shape {s!r} of family {family} has a non-positive dimension")
                shapes.append(ShapeSpec(m, n, k, str(s.get("name", ""))))
            regimes = tuple(j.get("regimes") or ("hot",))
            for r in regimes:
                if r not in REGIMES:
                    raise ValueError(f"unknown regime {r!r}; expected one of {REGIMES}")
            promote = int(j.get("promote", 2))
            if promote < 1:
                raise ValueError("promote must be at least 1")
            jobs.append(Job(family, tuple(shapes), regimes, promote, Protocol.from_dict(j.get("protocol")),
                            dict(j.get("tuning") or {}), tuple(j.get("tags") or ())))
        return cls(name, int(d.get("seed", 0)), tuple(jobs))

    @classmethod
    def load(cls, path) -> "Manifest":
        with open(path) as f:
            return cls.from_dict(json.load(f))


class Target:
    """One (family, shape, regime) to tune: the winner-store key the frontends look up, the schedule
    candidates, and a callable per candidate."""

    def __init__(self, context: KernelContext, adapter, configured, call: Callable[[Any], Callable[[], Any]],
                 output: Optional[Callable[[Any], Any]] = None):
        self.context, self.adapter, self.configured, self.call = context, adapter, configured, call
        # the output the gate compares: one call from a defined state (default: one plain call)
        self.output = output or (lambda cfg: call(cfg)())

    def candidates(self) -> Sequence[Any]:
        import dataclasses

        seen, out = set(), []
        for cand in (self.configured, *self.adapter.candidates(self.context)):
            cfg = cand if cand is self.configured else dataclasses.replace(self.configured, gemm=cand.gemm)
            key = cfg.to_key()
            if key in seen or self.adapter.rejection(cfg, self.context) is not None:
                continue
            seen.add(key)
            out.append(cfg)
        return out


def build_target(family: str, shape: ShapeSpec, regime: str, seed: int, device="cuda") -> Target:
    """Seeded synthetic operands of the shape behind the module a user of the family would build; the context
    is the module's own resolver context, so an installed winner is the one that module finds."""
    import torch

    from . import fp4 as _fp4
    from . import fp8 as _fp8

    kind, packed, scaling = FAMILY_TARGETS[family]
    gen = torch.Generator(device="cpu").manual_seed(seed)
    w = (torch.randn(shape.n, shape.k, generator=gen) / shape.k ** 0.5).to(device=device, dtype=torch.bfloat16)
    copies = 1
    if regime == "rotate":   # enough activations in rotation that none is still in L2 when its turn comes again
        copies = max(2, min(64, -(-2 * L2_BYTES // (shape.m * shape.k * 2))))
    xs = [torch.randn(shape.m, shape.k, generator=gen).to(device=device, dtype=torch.bfloat16) for _ in range(copies)]
    if kind == "mxfp8":
        mod = _fp8.MXFP8Linear(shape.k, shape.n, device=device)
        configured = _fp8._resolve_prequant(mod._forward_config_key)
    else:
        mod = _fp4.NVFP4Linear(shape.k, shape.n, device=device, scaling=scaling)
        configured = mod._dynamic_config
    with torch.no_grad():
        mod.weight.copy_(w)
    if packed:
        mod = mod.to_quantized_weight()
        configured = _fp8._resolve_prequant(mod._forward_config_key) if kind == "mxfp8" else mod._dynamic_config
    ctx = mod._resolver.context(shape.m)
    ctx = KernelContext(ctx.family, ctx.m, ctx.n, ctx.k, ctx.device_id, regime, ctx.variant)

    def call(cfg):
        runs = [mod._candidate_call(x, cfg) for x in xs]
        turn = [0]

        def run():
            turn[0] = (turn[0] + 1) % len(runs)
            return runs[turn[0]]()

        return run

    def output(cfg):
        if scaling == "delayed":
            mod.reset_delayed_scales()   # the output depends on the |max| history: compare from the same state
        return mod._candidate_call(xs[0], cfg)()

    return Target(ctx, mod._resolver.adapter, configured, call, output)


def _same_bits(a, b) -> bool:
    import torch

    if a.shape != b.shape or a.dtype != b.dtype:
        return False
    if a.dtype == torch.bfloat16:   # compare bit patterns, so that NaNs in the same places count as equal
        a, b = a.view(torch.int16), b.view(torch.int16)
    return bool(torch.equal(a, b))


def tune_target(target: Target, protocol: Protocol, promote: int, *, measure=time_call, same=_same_bits,
                record: Callable[[dict], None] = lambda r: None) -> dict:
    """Search (every candidate, `protocol.samples`), confirmation (the `promote` fastest, `confirm_samples`),
    gate (winner's output == configured schedule's output).  Returns the decision."""
    ctx, adapter = target.context, target.adapter
    base = {"family": ctx.family, "m": ctx.m, "n": ctx.n, "k": ctx.k, "regime": ctx.regime, "variant": ctx.variant}
    configured_key = target.configured.to_key()
    searched = []
    for cfg in target.candidates():
        out = measure(target.call(cfg), protocol.warmup_calls, protocol.samples)
        record({**base, "phase": "search", "config_key": cfg.to_key(), "status": out.status,
                "median_ms": out.median_ms, "detail": out.detail})
        if out.ok:
            searched.append((out.median_ms, cfg))
    if not searched:
        return {**base, "decision": "no candidate ran", "winner": None}
    searched.sort(key=lambda t: t[0])
    finalists = [cfg for _, cfg in searched[:max(1, promote)]]
    if all(cfg.to_key() != configured_key for cfg in finalists):
        finalists.append(target.configured)   # the configured schedule is always confirmed: it is the yardstick
    confirmed = []
    for cfg in finalists:
        out = measure(target.call(cfg), protocol.warmup_calls, protocol.confirm_samples)
        record({**base, "phase": "confirm", "config_key": cfg.to_key(), "status": out.status,
                "median_ms": out.median_ms, "detail": out.detail})
        if out.ok:
            confirmed.append((out.median_ms, cfg))
    if not confirmed:
        return {**base, "decision": "no finalist ran", "winner": None}
    confirmed.sort(key=lambda t: t[0])
    configured_ms = next((ms for ms, cfg in confirmed if cfg.to_key() == configured_key), None)
    reference_out = None
    for ms, cfg in confirmed:
        if cfg.to_key() != configured_key:
            if reference_out is None:
                reference_out = target.output(target.configured)
            if not same(target.output(cfg), reference_out):
                record({**base, "phase": "gate", "config_key": cfg.to_key(), "status": "rejected",
                        "median_ms": ms, "detail": "output differs from the configured schedule's"})
                continue
        return {**base, "decision": "winner", "winner": cfg, "median_ms": ms, "configured_ms": configured_ms,
                "gain": (configured_ms / ms) if configured_ms else None}
    return {**base, "decision": "every finalist failed the output gate", "winner": None}


def run_campaign(manifest: Manifest, out_dir, *, cache_dir=None, families: Optional[Iterable[str]] = None,
                 build: Callable[..., Target] = build_target, measure=time_call, same=_same_bits, min_gain: float = 1.0,
                 dry_run: bool = False, log: Callable[[str], None] = lambda s: None) -> dict:
    """Runs every job of `manifest`; installs each winner that is at least `min_gain` times as fast as the
    configured schedule (1.0: the fastest confirmed schedule is always stored, the configured one included).
    Returns the summary that is also written to `<out>/<name>/summary.json`."""
    root = Path(out_dir) / manifest.name
    root.mkdir(parents=True, exist_ok=True)
    wanted = set(families) if families else None
    summary = {"manifest": manifest.name, "seed": manifest.seed, "started": time.strftime("%Y-%m-%dT%H:%M:%S"),
               "targets": [], "skipped": []}
    trials = None if dry_run else open(root / "trials.jsonl", "a")

    def record(r: dict) -> None:
        if trials is not None:
            trials.write(json.dumps({"manifest": manifest.name, **r}, sort_keys=True) + "\n")
            trials.flush()

    try:
        for job_index, job in enumerate(manifest.jobs):
            if wanted is not None and job.family not in wanted:
                continue
            if job.family in UNTUNED_FAMILIES:
                summary["skipped"].append({"family": job.family, "shapes": len(job.shapes),
                                           "why": "one schedule per launch: nothing to choose"})
                continue
            for shape in job.shapes:
                for regime in job.regimes:
                    entry = {"family": job.family, "shape": shape.label, "m": shape.m, "n": shape.n, "k": shape.k,
                             "regime": regime}
                    if dry_run:
                        ctx = KernelContext(job.family, shape.m, shape.n, shape.k, regime=regime)
                        entry["candidates"] = [c.to_key() for c in ADAPTERS[_adapter_family(job.family)]().candidates(ctx)]
                        summary["targets"].append(entry)
                        continue
                    target = build(job.family, shape, regime, manifest.seed + 7919 * job_index)
                    decision = tune_target(target, job.protocol, job.promote, measure=measure, same=same, record=record)
                    winner = decision.pop("winner")
                    entry.update({k: decision[k] for k in ("decision", "median_ms", "configured_ms", "gain")
                                  if k in decision})
                    if winner is not None:
                        entry["winner"] = winner.to_key()
                        gain = decision.get("gain")
                        if gain is None or gain >= min_gain:
                            path = save_runtime_winner(target.context, target.adapter, winner, decision["median_ms"],
                                                       cache_dir)
                            entry["installed"] = str(path)
                    log(f"{job.family} {shape.label} {regime}: {entry.get('decision')} "
                        f"{entry.get('winner', '')[:60]} gain {entry.get('gain')}")
                    summary["targets"].append(entry)
    finally:
        if trials is not None:
            trials.close()
    with open(root / "summary.json", "w") as f:
        json.dump(summary, f, indent=1, sort_keys=True)
    return summary


def _adapter_family(family: str) -> str:
    kind, packed, _ = FAMILY_TARGETS[family]
    if kind == "mxfp8":
        return "mxfp8_prequant_fwd"
    return "nvfp4_weight_prequant_fwd" if packed else "nvfp4_dynamic_fwd"


def main(argv: Optional[Sequence[str]] = None) -> int:
    ap = argparse.ArgumentParser(prog="python -m rtx_b200.campaign", description=__doc__.split("\n\n")[0])
    ap.add_argument("manifest")
    ap.add_argument("--out", required=True, help="directory for trials.jsonl and summary.json")
    ap.add_argument("--cache-dir", default=None, help="winner store (default: the store the modules read)")
    ap.add_argument("--family", action="append", default=None, help="only these families (repeatable)")
    ap.add_argument("--min-gain", type=float, default=1.0)
    ap.add_argument("--dry-run", action="store_true", help="list targets and candidates; run nothing")
    args = ap.parse_args(argv)
    manifest = Manifest.load(args.manifest)
    summary = run_campaign(manifest, args.out, cache_dir=args.cache_dir, families=args.family, min_gain=args.min_gain,
                           dry_run=args.dry_run, log=lambda s: print(s, file=sys.stderr))
    print(json.dumps({"manifest": summary["manifest"], "targets": len(summary["targets"]),
                      "installed": sum(1 for t in summary["targets"] if "installed" in t),
                      "skipped": summary["skipped"]}))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
