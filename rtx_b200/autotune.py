"""Thin autotune boundary for the sm_100a kernels: the `KernelAdapter` protocol of the
reference (rtx/autotune/core.py:167-187), one discrete adapter per kernel family that
enumerates the legal tile / stage / CTA-group schedules, and the runtime winner cache
with the reference's key scheme (rtx/autotune/winners.py:26-45).  The search engine
(cost models, bandits, campaign CLI) is out of scope; `pick()` times the legal
candidates with the caller's evaluator and remembers the winner.
"""

from __future__ import annotations

import json
import os
from dataclasses import dataclass, field
from pathlib import Path
from typing import Any, Callable, Iterable, Optional, Protocol, Sequence, runtime_checkable

from .configs import (MXFP8BwdConfig, MXFP8GemmConfig, MXFP8PrequantConfig, MXFP8Problem, NVFP4DynamicConfig,
                      NVFP4GemmConfig, NVFP4Problem, config_from_key)

WINNER_REVISION = 1
FAMILIES = ("mxfp8_fused_fwd", "mxfp8_prequant_fwd", "mxfp8_bwd", "nvfp4_dynamic_fwd", "nvfp4_weight_prequant_fwd",
            "nvfp4_fully_prequant_fwd")


@dataclass(frozen=True)
class KernelContext:
    """What a schedule is chosen for (rtx/autotune/core.py:72-100)."""
    family: str
    m: int
    n: int
    k: int
    device_id: str = "b200"
    regime: str = "hot"
    variant: str = "default"


@dataclass(frozen=True)
class TrialOutcome:
    """rtx/autotune/outcomes.py:49-96."""
    status: str                      # ok | rejected | failed
    median_ms: Optional[float] = None
    detail: str = ""

    @property
    def ok(self) -> bool:
        return self.status == "ok" and self.median_ms is not None


@runtime_checkable
class KernelAdapter(Protocol):
    family: str

    def default(self, ctx: KernelContext) -> Any: ...
    def candidates(self, ctx: KernelContext) -> Sequence[Any]: ...
    def rejection(self, config: Any, ctx: KernelContext) -> Optional[str]: ...
    def encode(self, config: Any) -> str: ...
    def decode(self, key: str) -> Any: ...


@dataclass
class DiscreteKernelAdapter:
    """Adapter over an explicit candidate list (rtx/autotune/core.py:190-293)."""
    family: str
    default_config: Any
    space: Sequence[Any] = field(default_factory=tuple)
    problem_type: type = MXFP8Problem

    def default(self, ctx: KernelContext) -> Any:
        return self.default_config

    def candidates(self, ctx: KernelContext) -> Sequence[Any]:
        legal = [c for c in (self.default_config, *self.space) if self.rejection(c, ctx) is None]
        out, seen = [], set()
        for c in legal:
            key = self.encode(c)
            if key not in seen:
                seen.add(key)
                out.append(c)
        return out

    def rejection(self, config: Any, ctx: KernelContext) -> Optional[str]:
        problem = self.problem_type(ctx.m, ctx.n, ctx.k)
        try:
            return config.rejection(problem)
        except TypeError:
            return config.rejection()

    def encode(self, config: Any) -> str:
        return config.to_key()

    def decode(self, key: str) -> Any:
        return config_from_key(key)


def _gemm_space():
    # one candidate per built kernel; the frontends select it for the call with the library's per-thread
    # schedule switch, so a stored winner changes which kernel runs
    return tuple(MXFP8GemmConfig.for_schedule(name) for name in MXFP8GemmConfig.SCHEDULES)


def _nvfp4_gemm_space():
    return tuple(NVFP4GemmConfig.for_schedule(name) for name in NVFP4GemmConfig.SCHEDULES)


def make_mxfp8_prequant_fwd_adapter() -> DiscreteKernelAdapter:
    return DiscreteKernelAdapter("mxfp8_prequant_fwd", MXFP8PrequantConfig(),
                                 tuple(MXFP8PrequantConfig(gemm=g) for g in _gemm_space()))


def make_mxfp8_fwd_adapter() -> DiscreteKernelAdapter:
    return DiscreteKernelAdapter("mxfp8_fused_fwd", MXFP8PrequantConfig(),
                                 tuple(MXFP8PrequantConfig(gemm=g) for g in _gemm_space()))


def make_mxfp8_bwd_adapter() -> DiscreteKernelAdapter:
    return DiscreteKernelAdapter("mxfp8_bwd", MXFP8BwdConfig(),
                                 (MXFP8BwdConfig(streams="single"), MXFP8BwdConfig(streams="dual_stream")))


def make_nvfp4_dynamic_fwd_adapter() -> DiscreteKernelAdapter:
    return DiscreteKernelAdapter("nvfp4_dynamic_fwd", NVFP4DynamicConfig(),
                                 tuple(NVFP4DynamicConfig(gemm=g) for g in _nvfp4_gemm_space()),
                                 problem_type=NVFP4Problem)


ADAPTERS: dict[str, Callable[[], DiscreteKernelAdapter]] = {
    "mxfp8_fused_fwd": make_mxfp8_fwd_adapter,
    "mxfp8_prequant_fwd": make_mxfp8_prequant_fwd_adapter,
    "mxfp8_bwd": make_mxfp8_bwd_adapter,
    "nvfp4_dynamic_fwd": make_nvfp4_dynamic_fwd_adapter,
    "nvfp4_weight_prequant_fwd": make_nvfp4_dynamic_fwd_adapter,
    "nvfp4_fully_prequant_fwd": make_nvfp4_dynamic_fwd_adapter,
}


# --------------------------------------------------------------------------- winner cache

def cache_root(cache_dir: "Path | str | None" = None) -> Path:
    if cache_dir is not None:
        return Path(cache_dir)
    env = os.environ.get("RTX_AUTOTUNE_CACHE_DIR")
    return Path(env) if env else Path.home() / ".cache" / "rtx_b200" / "autotune"


def runtime_winner_path(ctx: KernelContext, cache_dir=None) -> Path:
    """runtime_winners/<family>/<device_id>/m{M}_n{N}_k{K}_{regime}_{variant}_rev{R}.json"""
    name = f"m{ctx.m}_n{ctx.n}_k{ctx.k}_{ctx.regime}_{ctx.variant}_rev{WINNER_REVISION}.json"
    return cache_root(cache_dir) / "runtime_winners" / ctx.family / ctx.device_id / name


def save_runtime_winner(ctx: KernelContext, adapter: KernelAdapter, config: Any, median_ms: float, cache_dir=None) -> Path:
    path = runtime_winner_path(ctx, cache_dir)
    path.parent.mkdir(parents=True, exist_ok=True)
    tmp = path.with_suffix(".tmp")
    payload = {"family": ctx.family, "m": ctx.m, "n": ctx.n, "k": ctx.k, "device_id": ctx.device_id,
               "regime": ctx.regime, "variant": ctx.variant, "revision": WINNER_REVISION,
               "config_key": adapter.encode(config), "median_ms": median_ms}
    with open(tmp, "w") as f:
        json.dump(payload, f, indent=1, sort_keys=True)
        f.flush()
        os.fsync(f.fileno())
    os.replace(tmp, path)
    return path


def load_runtime_winner(ctx: KernelContext, adapter: KernelAdapter, cache_dir=None):
    path = runtime_winner_path(ctx, cache_dir)
    if not path.exists():
        return None
    with open(path) as f:
        payload = json.load(f)
    if payload.get("revision") != WINNER_REVISION or payload.get("family") != ctx.family:
        return None
    config = adapter.decode(payload["config_key"])
    return config if adapter.rejection(config, ctx) is None else None


def time_call(run: Callable[[], Any], warmup: int = 2, samples: int = 5) -> TrialOutcome:
    """Median device time of `run()` over `samples` calls after `warmup` untimed ones, by CUDA events on the
    current stream; a RuntimeError from the call (an illegal schedule for the shape) is a failed trial."""
    import torch

    try:
        for _ in range(max(0, warmup)):
            run()
        times = []
        for _ in range(max(1, samples)):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            run()
            e1.record()
            e1.synchronize()
            times.append(e0.elapsed_time(e1))
    except RuntimeError as exc:
        return TrialOutcome("failed", detail=str(exc))
    return TrialOutcome("ok", median_ms=sorted(times)[len(times) // 2])


def pick(ctx: KernelContext, adapter: KernelAdapter, evaluate: Callable[[Any], TrialOutcome], *, mode: str = "cache",
         cache_dir=None):
    """Resolve the schedule for `ctx`: `off` -> the adapter default; `cache` -> the stored winner or the
    default; `balanced`/`online`/`coordinate` -> time every legal candidate with `evaluate`, store and return
    the fastest."""
    if mode == "off":
        return adapter.default(ctx)
    cached = load_runtime_winner(ctx, adapter, cache_dir)
    if cached is not None or mode == "cache":
        return cached if cached is not None else adapter.default(ctx)
    best, best_ms = adapter.default(ctx), None
    for cand in adapter.candidates(ctx):
        outcome = evaluate(cand)
        if outcome.ok and (best_ms is None or outcome.median_ms < best_ms):
            best, best_ms = cand, outcome.median_ms
    if best_ms is not None:
        save_runtime_winner(ctx, adapter, best, best_ms, cache_dir)
    return best


class ScheduleResolver:
    """Where a frontend turns its `autotune=` argument into the schedule of a call, as the reference's
    frontends do (rtx/fp8.py:804-886, 2302-2386): `off` keeps the configured schedule; `cache` uses the
    stored winner of this (family, M, N, K) when there is one; `balanced` / `online` / `coordinate`
    time every legal candidate on the first call with a new M (with the caller's evaluator), store the
    winner and use it from then on.  Only the GEMM schedule is taken from a winner: the quantizer
    settings (rounding, layouts) stay those of the configured schedule.  Resolutions are remembered per
    M, so the steady state costs one dictionary lookup."""

    def __init__(self, family: str, n: int, k: int, mode: str, cache_dir=None, *, variant: str = "default",
                 device_id: str = "b200"):
        self.family, self.n, self.k, self.mode, self.cache_dir = family, int(n), int(k), mode, cache_dir
        self.variant, self.device_id = variant, device_id
        self.adapter = ADAPTERS[family]()
        self.resolved: dict[int, Any] = {}
        self.sources: dict[int, str] = {}

    def context(self, m: int) -> KernelContext:
        return KernelContext(self.family, int(m), self.n, self.k, self.device_id, "hot", self.variant)

    def resolve(self, m: int, configured: Any, evaluate: Optional[Callable[[Any], TrialOutcome]] = None) -> Any:
        import dataclasses

        if self.mode == "off":
            return configured
        m = int(m)
        if m in self.resolved:
            return self.resolved[m]
        ctx = self.context(m)
        winner = load_runtime_winner(ctx, self.adapter, self.cache_dir)
        source = "stored winner"
        if winner is None and self.mode != "cache" and evaluate is not None:
            def trial(candidate):
                return evaluate(dataclasses.replace(configured, gemm=candidate.gemm))

            winner = pick(ctx, self.adapter, trial, mode=self.mode, cache_dir=self.cache_dir)
            source = "tuned on first use"
        if winner is None:
            chosen, source = configured, "configured (no stored winner)"
        else:
            chosen = dataclasses.replace(configured, gemm=winner.gemm)
        if chosen.rejection(self.adapter.problem_type(m, self.n, self.k)) is not None:
            chosen, source = configured, "configured (winner not legal for this schedule)"
        self.resolved[m], self.sources[m] = chosen, source
        return chosen


__all__ = ["KernelAdapter", "ScheduleResolver", "DiscreteKernelAdapter", "KernelContext", "TrialOutcome", "ADAPTERS", "pick",
           "runtime_winner_path", "save_runtime_winner", "load_runtime_winner", "FAMILIES", "time_call"]
