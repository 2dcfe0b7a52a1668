"""Schedule descriptions of the sm_100a kernels.

The public class names are the reference's (rtx/configs/mxfp8.py:18-343,
rtx/kernels/mxfp8.py:45-545, rtx/kernels/mxfp8_bwd.py:23-464,
rtx/configs/nvfp4.py); the reference's fields described SM120 schedules (99 KB
of shared memory, ldmatrix widths, warp-level MMA atoms) and are replaced by the
knobs the tcgen05 kernels have: CTA tile, pipeline stages, CTA-group size,
scale layout and rounding.  Every config is frozen, hashable, has an explicit
`rejection()` legality check returning a reason string or None, and travels
through custom ops as an interned JSON key (`to_key` / `config_from_key`).
"""

from __future__ import annotations

import functools
import json
from dataclasses import asdict, dataclass, field, fields
from typing import ClassVar, Optional

SMEM_CAPACITY_BYTES = 227 * 1024
TMEM_COLUMNS = 512
SM_COUNT = 148

_REGISTRY: dict[str, type] = {}


def _register(cls):
    _REGISTRY[cls.__name__] = cls
    return cls


class _Config:
    def to_dict(self) -> dict:
        out = {"type": type(self).__name__}
        for f in fields(self):
            v = getattr(self, f.name)
            out[f.name] = v.to_dict() if isinstance(v, _Config) else v
        return out

    def to_key(self) -> str:
        return json.dumps(self.to_dict(), sort_keys=True, separators=(",", ":"))

    @classmethod
    def from_dict(cls, d: dict):
        kwargs = {}
        for f in fields(cls):
            if f.name in d:
                v = d[f.name]
                kwargs[f.name] = _REGISTRY[v["type"]].from_dict(v) if isinstance(v, dict) and "type" in v else v
        return cls(**kwargs)


@functools.lru_cache(maxsize=1024)
def config_from_key(key: str):
    """The schedule a key names.  Configs are frozen, so one parsed instance serves every call that carries
    the key (keys ride on the launch path of every op call)."""
    d = json.loads(key)
    return _REGISTRY[d["type"]].from_dict(d)


@_register
@dataclass(frozen=True)
class MXFP8Problem(_Config):
    """Y[m,n] = X[m,k] W[n,k]^T (rtx/kernels/mxfp8.py:45-66)."""
    m: int
    n: int
    k: int

    @property
    def storage_k(self) -> int:
        return (self.k + 31) // 32 * 32

    def rejection(self) -> Optional[str]:
        if min(self.m, self.n, self.k) <= 0:
            return "m, n and k must be positive"
        if max(self.m, self.n, self.k) >= 2 ** 31:
            return "dimensions must fit in 32 bits"
        return None


@_register
@dataclass(frozen=True)
class MXFP8QuantConfig(_Config):
    """BF16 -> MXFP8 quantizer (rtx/configs/mxfp8.py:18-107)."""
    scale_layout: str = "mma128"       # row_major | mma128 (the tcgen05.cp tiling)
    scale_rounding: str = "infinity"   # infinity (default) | floor (OCP ablation)
    rows_per_tile: int = 128
    threads: int = 256

    def rejection(self, rows: int = 1, k: int = 1) -> Optional[str]:
        if self.scale_layout == "mma64":
            return "mma64 is an SM120 scale schedule; sm_100a uses row_major or mma128"
        if self.scale_layout not in ("row_major", "mma128"):
            return f"unknown scale layout {self.scale_layout!r}"
        if self.scale_rounding not in ("infinity", "floor"):
            return f"unknown scale rounding {self.scale_rounding!r}"
        if rows <= 0 or k <= 0:
            return "rows and k must be positive"
        if (self.rows_per_tile, self.threads) != (128, 256):
            return "the sm_100a quantizer is built for 128-row tiles and 256 threads"
        return None


@_register
@dataclass(frozen=True)
class MXFP8GemmConfig(_Config):
    """tcgen05 block-scaled GEMM on packed operands (rtx/configs/mxfp8.py:110-343)."""
    tile_m: int = 128
    tile_n: int = 256
    tile_k_bytes: int = 128
    stages: int = 4
    cta_group: int = 1
    accumulator_windows: int = 2       # overlapping TMEM windows [0,256) and [224,480)
    epilogue: str = "direct"           # direct vectorised stores
    raster: str = "m_fastest"
    # which built kernel runs: "auto" (the library picks by shape) or one of SCHEDULES, whose tile shape the
    # other fields must then state
    schedule: str = "auto"

    # (tile_m, tile_n, tile_k_bytes, stages, cta_group); stages 0 = ring depth chosen at launch
    # "fused_x": the pair tiling with the activation operand quantized by the GEMM's own quantizer warps (the
    # composite forwards drop their activation-quantizer launch; packed-operand GEMMs run it as "pair")
    SCHEDULES: ClassVar[dict] = {"single": (128, 256, 128, 4, 1), "pair": (256, 256, 128, 6, 2),
                                 "stream": (128, 64, 128, 0, 1), "fused_x": (256, 256, 128, 6, 2)}
    BUILT: ClassVar[tuple] = tuple(SCHEDULES.values())

    @classmethod
    def for_schedule(cls, name: str) -> "MXFP8GemmConfig":
        tm, tn, tk, st, cg = cls.SCHEDULES[name]
        return cls(tile_m=tm, tile_n=tn, tile_k_bytes=tk, stages=st, cta_group=cg, schedule=name)

    def smem_bytes(self, sf_bytes_per_stage: int = 1536) -> int:
        rows = self.tile_m // self.cta_group + self.tile_n // self.cta_group   # per CTA
        return self.stages * (rows * self.tile_k_bytes + sf_bytes_per_stage) + 1280

    def rejection(self, problem: Optional[MXFP8Problem] = None) -> Optional[str]:
        shape = (self.tile_m, self.tile_n, self.tile_k_bytes, self.stages, self.cta_group)
        if shape not in self.BUILT:
            return ("no kernel is built for this tile/stage/cta_group combination; built: "
                    + ", ".join(map(str, self.BUILT)))
        if self.schedule != "auto":
            if self.schedule not in self.SCHEDULES:
                return f"unknown GEMM schedule {self.schedule!r}; built: auto, " + ", ".join(self.SCHEDULES)
            if self.SCHEDULES[self.schedule] != shape:
                return f"schedule {self.schedule!r} has the tile shape {self.SCHEDULES[self.schedule]}, not {shape}"
            if self.schedule == "stream" and problem is not None and problem.m > 128:
                return "the streaming schedule serves M <= 128"
        if self.smem_bytes() > SMEM_CAPACITY_BYTES:
            return "pipeline does not fit 227 KB of shared memory"
        if problem is not None:
            return problem.rejection()
        return None


@_register
@dataclass(frozen=True)
class MXFP8FwdConfig(_Config):
    """Forward schedule (rtx/kernels/mxfp8.py:68-545): `pipeline` picks quantize-once +
    packed GEMM ("materialized") — the only forward pipeline built so far."""
    pipeline: str = "materialized"
    quant: MXFP8QuantConfig = field(default_factory=MXFP8QuantConfig)
    gemm: MXFP8GemmConfig = field(default_factory=MXFP8GemmConfig)
    glu_epilogue: bool = False

    def rejection(self, problem: Optional[MXFP8Problem] = None) -> Optional[str]:
        if self.pipeline != "materialized":
            return f"forward pipeline {self.pipeline!r} is not built"
        if self.quant.scale_layout != "mma128":
            return "the GEMM consumes mma128 scales"
        return self.quant.rejection() or self.gemm.rejection(problem)


@_register
@dataclass(frozen=True)
class MXFP8PrequantConfig(_Config):
    """Quantize-then-GEMM pair (rtx/fp8.py `MXFP8PrequantConfig`)."""
    quant: MXFP8QuantConfig = field(default_factory=MXFP8QuantConfig)
    gemm: MXFP8GemmConfig = field(default_factory=MXFP8GemmConfig)

    def rejection(self, problem: Optional[MXFP8Problem] = None) -> Optional[str]:
        if self.quant.scale_layout != "mma128":
            return "the GEMM consumes mma128 scales"
        return self.quant.rejection() or self.gemm.rejection(problem)


MXFP8WeightPrequantConfig = MXFP8PrequantConfig
MXFP8FullyPrequantConfig = MXFP8GemmConfig


@_register
@dataclass(frozen=True)
class MXFP8BwdMatmulConfig(_Config):
    """One backward product (rtx/kernels/mxfp8_bwd.py:23-356)."""
    gemm: MXFP8GemmConfig = field(default_factory=MXFP8GemmConfig)
    output_dtype: str = "bf16"   # bf16 (reference dtype) | f32 (data-parallel all-reduce)

    def rejection(self) -> Optional[str]:
        if self.output_dtype not in ("bf16", "f32"):
            return f"unknown output dtype {self.output_dtype!r}"
        return self.gemm.rejection()


@_register
@dataclass(frozen=True)
class MXFP8BwdConfig(_Config):
    """dX = dY W, dW = dY^T X, operands requantized along their contraction dimension
    (rtx/kernels/mxfp8_bwd.py:358-464)."""
    dx: MXFP8BwdMatmulConfig = field(default_factory=MXFP8BwdMatmulConfig)
    dw: MXFP8BwdMatmulConfig = field(default_factory=MXFP8BwdMatmulConfig)
    schedule: str = "decomposed"    # quantizers + packed GEMMs
    streams: str = "single"         # single | dual_stream (dX and dW on two streams)

    def rejection(self) -> Optional[str]:
        if self.schedule != "decomposed":
            return f"backward schedule {self.schedule!r} is not built"
        if self.streams not in ("single", "dual_stream"):
            return f"unknown stream policy {self.streams!r}"
        return self.dx.rejection() or self.dw.rejection()


@_register
@dataclass(frozen=True)
class NVFP4Problem(_Config):
    m: int
    n: int
    k: int

    @property
    def storage_k(self) -> int:
        return (self.k + 31) // 32 * 32

    def rejection(self) -> Optional[str]:
        if min(self.m, self.n, self.k) <= 0:
            return "m, n and k must be positive"
        return None


@_register
@dataclass(frozen=True)
class NVFP4QuantConfig(_Config):
    """BF16 -> NVFP4 quantizer (rtx/configs/nvfp4.py `NVFP4QuantConfig`)."""
    scale_layout: str = "mma128"
    scale_reciprocal: str = "direct"   # (1 / tensor_scale) / block_scale, two IEEE divisions
    rows_per_tile: int = 128
    threads: int = 256

    def rejection(self, rows: int = 1, k: int = 1) -> Optional[str]:
        if self.scale_layout not in ("row_major", "mma128"):
            return f"unknown scale layout {self.scale_layout!r}"
        if self.scale_reciprocal != "direct":
            return "only the reference-default 'direct' reciprocal is built (bit-exact payloads)"
        if rows <= 0 or k <= 0:
            return "rows and k must be positive"
        return None


@_register
@dataclass(frozen=True)
class NVFP4ScaleConfig(_Config):
    """Outer-scale policy (rtx/configs/nvfp4.py `NVFP4ScaleConfig`)."""
    policy: str = "current"            # current | jit_row_region | delayed | block
    tensor_scale_mode: str = "power2"  # power2 (dynamic default) | exact (offline weights)
    amax_history_len: int = 16         # delayed: |max| values kept per operand (1, 4, 16 or 64)
    amax_history_algo: str = "window_max"   # delayed: window_max | most_recent

    def rejection(self) -> Optional[str]:
        if self.policy not in ("current", "jit_row_region", "delayed", "block"):
            return f"unknown NVFP4 scaling policy {self.policy!r}"
        if self.tensor_scale_mode not in ("power2", "exact"):
            return f"unknown tensor scale mode {self.tensor_scale_mode!r}"
        if self.amax_history_len not in (1, 4, 16, 64):
            return "amax_history_len must be 1, 4, 16, or 64"
        if self.amax_history_algo not in ("most_recent", "window_max"):
            return "amax_history_algo must be most_recent or window_max"
        return None


@_register
@dataclass(frozen=True)
class NVFP4GemmConfig(_Config):
    tile_m: int = 128
    tile_n: int = 256
    tile_k_bytes: int = 128            # 256 E2M1 values
    stages: int = 4
    cta_group: int = 1
    schedule: str = "auto"             # as MXFP8GemmConfig.schedule

    SCHEDULES: ClassVar[dict] = {"single": (128, 256, 128, 4, 1), "pair": (256, 256, 128, 5, 2),
                                 "stream": (128, 64, 128, 0, 1)}

    @classmethod
    def for_schedule(cls, name: str) -> "NVFP4GemmConfig":
        tm, tn, tk, st, cg = cls.SCHEDULES[name]
        return cls(tile_m=tm, tile_n=tn, tile_k_bytes=tk, stages=st, cta_group=cg, schedule=name)

    def rejection(self, problem: Optional[NVFP4Problem] = None) -> Optional[str]:
        shape = (self.tile_m, self.tile_n, self.tile_k_bytes, self.stages, self.cta_group)
        if shape not in self.SCHEDULES.values():
            return "no kernel is built for this tile/stage/cta_group combination"
        if self.schedule != "auto":
            if self.schedule not in self.SCHEDULES:
                return f"unknown GEMM schedule {self.schedule!r}; built: auto, " + ", ".join(self.SCHEDULES)
            if self.SCHEDULES[self.schedule] != shape:
                return f"schedule {self.schedule!r} has the tile shape {self.SCHEDULES[self.schedule]}, not {shape}"
            if self.schedule == "stream" and problem is not None and problem.m > 128:
                return "the streaming schedule serves M <= 128"
        return problem.rejection() if problem is not None else None


@_register
@dataclass(frozen=True)
class NVFP4DynamicConfig(_Config):
    quant: NVFP4QuantConfig = field(default_factory=NVFP4QuantConfig)
    gemm: NVFP4GemmConfig = field(default_factory=NVFP4GemmConfig)
    scale: NVFP4ScaleConfig = field(default_factory=NVFP4ScaleConfig)
    # row-region policy: rows per outer scale of each operand; both zero for the other policies
    # (rtx/configs/nvfp4.py:325-360)
    x_scale_region_rows: int = 0
    weight_scale_region_rows: int = 0

    @property
    def jit_row_region(self) -> bool:
        return bool(self.x_scale_region_rows or self.weight_scale_region_rows)

    def rejection(self, problem: Optional[NVFP4Problem] = None) -> Optional[str]:
        if bool(self.x_scale_region_rows) != bool(self.weight_scale_region_rows):
            return "row-region scaling needs a region size for both operands"
        if self.jit_row_region and (self.x_scale_region_rows < 1 or self.weight_scale_region_rows < 1):
            return "region rows must be positive"
        if self.jit_row_region != (self.scale.policy == "jit_row_region"):
            return "region sizes go with the jit_row_region policy and only with it"
        return self.quant.rejection() or self.scale.rejection() or self.gemm.rejection(problem)


NVFP4WeightPrequantConfig = NVFP4DynamicConfig
NVFP4FullyPrequantConfig = NVFP4GemmConfig

DEFAULT_MXFP8_PREQUANT_CONFIG = MXFP8PrequantConfig()
DEFAULT_MXFP8_INFERENCE_CONFIG = MXFP8PrequantConfig()
DEFAULT_MXFP8_BWD_CONFIG = MXFP8BwdConfig()
DEFAULT_FUSED_MXFP8_BWD_CONFIG = MXFP8BwdConfig()
DEFAULT_NVFP4_QUANT_CONFIG = NVFP4QuantConfig()
DEFAULT_NVFP4_DYNAMIC_CONFIG = NVFP4DynamicConfig()
