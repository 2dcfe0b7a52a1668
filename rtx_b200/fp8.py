"""MXFP8 frontend: `MXFP8Linear`, `mxfp8_linear`, `quantize_mxfp8` and the `rtx::mxfp8_*`
custom ops, with the reference's signatures (rtx/fp8.py:745-793, :2019-2193,
:2389-2775, ops at :498-680, :1016-1074, :1269-1366) on top of the sm_100a kernels.

Routing follows the reference: operand state (dynamic / weight-prequantized /
fully-prequantized), leading dimensions flattened, autograd through the training
op.  `backend="materialized"` and `"auto"` are the quantize-once + packed tcgen05 GEMM
pipeline; `backend="fused"` selects the GEMM that quantizes the activations in the kernel
(the reference's fused forward; several times slower on compute-bound shapes, same bits).
Schedules travel through the ops as interned JSON keys (rtx/fp8.py:376-415).
"""

from __future__ import annotations

import functools
from pathlib import Path
from threading import RLock
from typing import Optional

import torch
from torch import nn

from ._oplib import custom_op
from . import _native as N
from . import ops
from . import weight_cache as _weight_cache
from .configs import (DEFAULT_MXFP8_INFERENCE_CONFIG, DEFAULT_MXFP8_PREQUANT_CONFIG, MXFP8BwdConfig, MXFP8FwdConfig, MXFP8GemmConfig,
                      MXFP8PrequantConfig, MXFP8Problem, MXFP8QuantConfig, config_from_key)
from .formats import (PACKED_OPERAND_SCHEMA_VERSION, SCALE_LAYOUT_CODES, SCALE_LAYOUT_NAMES, MXFP8Tensor,
                      make_mxfp8_tensor, mxfp8_matrix_shape, mxfp8_qdata_2d, mxfp8_scale_layout,
                      mxfp8_scales_for_kernel, reject_packed_dtype_conversion, scales_row_major_to_mma128)
from .runtime import BoundedCache, runner_cache_limit
from .types import AutotuneMode, MXFP8Backend

_LOCK = RLock()
_WORKSPACES: BoundedCache = BoundedCache(runner_cache_limit("prequant", namespace="MXFP8"))
_LAYOUT_CODE = {"row_major": N.SCALE_ROW_MAJOR, "mma128": N.SCALE_MMA128}


def _intern(config) -> str:
    return config.to_key()


def _normalize_backend(backend: str) -> str:
    if backend not in ("auto", "fused", "materialized"):
        raise ValueError(f"unknown MXFP8 backend {backend!r}; expected auto, fused or materialized")
    return backend


def _autotune_mode(autotune) -> str:
    if autotune is None or autotune is False:
        return "off"
    if autotune is True:
        return "cache"
    if autotune not in ("off", "cache", "balanced", "online", "coordinate"):
        raise ValueError(f"unknown autotune mode {autotune!r}")
    return autotune


def _check_inputs(x: torch.Tensor, weight: torch.Tensor) -> None:
    """rtx/fp8.py:480-495."""
    if x.device.type != "cuda" or weight.device.type != "cuda":
        raise ValueError("MXFP8 linear requires CUDA tensors")
    if x.device != weight.device:
        raise ValueError("x and weight must share one device")
    if x.dtype is not torch.bfloat16 or weight.dtype is not torch.bfloat16:
        raise TypeError(f"MXFP8 linear requires BF16 operands, got {x.dtype} and {weight.dtype}")
    if x.ndim != 2 or weight.ndim != 2:
        raise ValueError("kernel operands must be two-dimensional")
    if x.shape[1] != weight.shape[1]:
        raise ValueError(f"K mismatch: x has {x.shape[1]}, weight has {weight.shape[1]}")


def _workspace(device: torch.device) -> ops.Workspace:
    """One scratch buffer per (device, stream): launches on a stream are ordered, so one
    in-flight use at a time (rtx/fp8.py:954-970)."""
    index = device.index if device.index is not None else torch._C._cuda_getDevice()
    key = (index, torch._C._cuda_getCurrentRawStream(index))
    with _LOCK:
        ws = _WORKSPACES.get(key)
        if ws is None:
            ws = ops.Workspace(device)
            _WORKSPACES[key] = ws
        return ws


def _clear_runtime_caches() -> dict:
    stats = _WORKSPACES.stats()
    _WORKSPACES.clear()
    return {"workspaces": stats}


@functools.lru_cache(maxsize=1024)
def _resolve_prequant(config_key: str) -> MXFP8PrequantConfig:
    cfg = config_from_key(config_key)
    if isinstance(cfg, MXFP8FwdConfig):
        cfg = MXFP8PrequantConfig(quant=cfg.quant, gemm=cfg.gemm)
    if not isinstance(cfg, MXFP8PrequantConfig):
        raise RuntimeError(f"config key does not name an MXFP8 forward schedule: {type(cfg).__name__}")
    return cfg


def _rounding(cfg: MXFP8PrequantConfig) -> int:
    return N.ROUND_INFINITY if cfg.quant.scale_rounding == "infinity" else N.ROUND_FLOOR


# --------------------------------------------------------------------------- quantize

def quantize_mxfp8(tensor: torch.Tensor, *, config: Optional[MXFP8QuantConfig] = None) -> MXFP8Tensor:
    """Prequantize BF16 once and return the packed MX tensor (rtx/fp8.py:745-793)."""
    if tensor.ndim < 1:
        raise ValueError("MXFP8 quantization requires at least one dimension")
    if tensor.device.type != "cuda":
        raise ValueError("MXFP8 quantization requires a CUDA tensor")
    if tensor.dtype is not torch.bfloat16:
        raise TypeError(f"MXFP8 quantization requires BF16, got {tensor.dtype}")
    leading_shape = tuple(int(v) for v in tensor.shape)
    source = tensor.reshape(-1, tensor.shape[-1])
    source = source if source.is_contiguous() else source.contiguous()
    selected = config or MXFP8QuantConfig()
    rejection = selected.rejection(int(source.shape[0]), int(source.shape[1]))
    if rejection is not None:
        raise RuntimeError(f"MXFP8 operand cannot be quantized: {rejection}")
    q, s = ops.mxfp8_quantize(source, layout=_LAYOUT_CODE[selected.scale_layout],
                              rounding=N.ROUND_INFINITY if selected.scale_rounding == "infinity" else N.ROUND_FLOOR)
    # launches are asynchronous: keep the BF16 source alive until the outputs are ready
    q._base_inputs = (source,)
    s._base_inputs = (source,)
    return make_mxfp8_tensor(q, s, leading_shape, selected.scale_layout)


# --------------------------------------------------------------------------- custom ops

@custom_op("rtx::mxfp8_linear_fwd", mutates_args=(), device_types="cuda")
def mxfp8_linear_fwd(x: torch.Tensor, weight: torch.Tensor, config_key: str) -> torch.Tensor:
    _check_inputs(x, weight)
    cfg = _resolve_prequant(config_key)
    problem = MXFP8Problem(int(x.shape[0]), int(weight.shape[0]), int(x.shape[1]))
    rejection = cfg.rejection(problem)
    if rejection is not None:
        raise RuntimeError(f"illegal MXFP8 forward schedule: {rejection}")
    x = x if x.is_contiguous() else x.contiguous()
    weight = weight if weight.is_contiguous() else weight.contiguous()
    with ops.schedule_of(cfg.gemm):
        return ops.mxfp8_linear_fwd(x, weight, _workspace(x.device), rounding=_rounding(cfg))


@mxfp8_linear_fwd.register_fake
def _(x, weight, config_key):
    return x.new_empty((x.shape[0], weight.shape[0]), dtype=torch.bfloat16)


@custom_op("rtx::mxfp8_linear_prequant", mutates_args=(), device_types="cuda")
def mxfp8_linear_prequant(x: torch.Tensor, weight: torch.Tensor, config_key: str) -> torch.Tensor:
    """Materialized pipeline: quantize both operands once, then the packed GEMM (rtx/fp8.py:1016-1030)."""
    return mxfp8_linear_fwd.fn(x, weight, config_key)   # the implementation itself: one dispatch per call, not two


@mxfp8_linear_prequant.register_fake
def _(x, weight, config_key):
    return x.new_empty((x.shape[0], weight.shape[0]), dtype=torch.bfloat16)


def _kernel_scales(scales: torch.Tensor, rows: int, k: int, layout: str) -> torch.Tensor:
    nb = (k + 31) // 32
    if layout == "mma128":
        return scales.reshape(-1).view(torch.uint8)
    if layout == "row_major":
        return scales_row_major_to_mma128(scales, rows, nb, (nb + 3) // 4)
    raise RuntimeError(f"MXFP8 scale layout {layout!r} cannot feed the sm_100a GEMM")


# Launch-only variants writing into a caller-provided [M, N] BF16 tensor (rtx/fp8.py:648-680, :1043-1075)
_OUT_LIBRARY = torch.library.Library("rtx", "FRAGMENT")
_OUT_LIBRARY.define("mxfp8_linear_fwd_out(Tensor x, Tensor weight, str config_key, Tensor(a!) out) -> ()")
_OUT_LIBRARY.define("mxfp8_linear_prequant_out(Tensor x, Tensor weight, str config_key, Tensor(a!) out) -> ()")


def _fwd_out(x, weight, config_key, out):
    _check_inputs(x, weight)
    cfg = _resolve_prequant(config_key)
    rejection = cfg.rejection(MXFP8Problem(int(x.shape[0]), int(weight.shape[0]), int(x.shape[1])))
    if rejection is not None:
        raise RuntimeError(f"illegal MXFP8 forward schedule: {rejection}")
    if tuple(out.shape) != (x.shape[0], weight.shape[0]) or out.dtype is not torch.bfloat16 or not out.is_contiguous():
        raise ValueError("out must be a contiguous BF16 [M, N] tensor")
    with ops.schedule_of(cfg.gemm):
        ops.mxfp8_linear_fwd(x if x.is_contiguous() else x.contiguous(),
                             weight if weight.is_contiguous() else weight.contiguous(), _workspace(x.device), out=out,
                             rounding=_rounding(cfg))


torch.library.impl("rtx::mxfp8_linear_fwd_out", "cuda")(_fwd_out)
torch.library.impl("rtx::mxfp8_linear_prequant_out", "cuda")(_fwd_out)


@torch.library.register_fake("rtx::mxfp8_linear_fwd_out")
def _(x, weight, config_key, out):
    return None


@torch.library.register_fake("rtx::mxfp8_linear_prequant_out")
def _(x, weight, config_key, out):
    return None


@custom_op("rtx::mxfp8_linear_dynamic_x_prequant_w", mutates_args=(), device_types="cuda")
def mxfp8_linear_dynamic_x_prequant_w(x: torch.Tensor, weight_data: torch.Tensor, weight_scales: torch.Tensor, n: int,
                                      k: int, weight_scale_layout: str, config_key: str) -> torch.Tensor:
    """BF16 activations, packed weight (rtx/fp8.py:1269-1302)."""
    if x.dtype is not torch.bfloat16 or x.ndim != 2 or x.shape[1] != k:
        raise TypeError("x must be BF16 [M, K]")
    cfg = _resolve_prequant(config_key)
    x = x if x.is_contiguous() else x.contiguous()
    sw = _kernel_scales(weight_scales, n, k, weight_scale_layout)
    if cfg.gemm.schedule == "fused_x":
        # one launch: the GEMM's quantizer warps encode X (the reference's fused kernel for this operand state)
        return ops.mxfp8_linear_fwd_fused_x(x, weight_data.view(torch.uint8), sw, n, rounding=_rounding(cfg))
    qx, sx = ops.mxfp8_quantize(x, rounding=_rounding(cfg))
    with ops.schedule_of(cfg.gemm):
        return ops.mxfp8_gemm(qx, sx, weight_data.view(torch.uint8), sw, int(x.shape[0]), n, k)


@mxfp8_linear_dynamic_x_prequant_w.register_fake
def _(x, weight_data, weight_scales, n, k, weight_scale_layout, config_key):
    return x.new_empty((x.shape[0], n), dtype=torch.bfloat16)


@custom_op("rtx::mxfp8_linear_prequantized", mutates_args=(), device_types="cuda")
def mxfp8_linear_prequantized(x_data: torch.Tensor, weight_data: torch.Tensor, x_scales: torch.Tensor,
                              weight_scales: torch.Tensor, m: int, n: int, k: int, x_scale_layout: str,
                              weight_scale_layout: str, config_key: str) -> torch.Tensor:
    """Both operands packed (rtx/fp8.py:1305-1366)."""
    sx = _kernel_scales(x_scales, m, k, x_scale_layout)
    sw = _kernel_scales(weight_scales, n, k, weight_scale_layout)
    with ops.schedule_of(_resolve_prequant(config_key).gemm):
        return ops.mxfp8_gemm(x_data.view(torch.uint8), sx, weight_data.view(torch.uint8), sw, m, n, k)


@mxfp8_linear_prequantized.register_fake
def _(x_data, weight_data, x_scales, weight_scales, m, n, k, x_scale_layout, weight_scale_layout, config_key):
    return x_data.new_empty((m, n), dtype=torch.bfloat16)


# --------------------------------------------------------------------------- functional

_FUNCTIONAL_RESOLVERS: dict = {}


def _stored_winner_key(fwd_key: str, m: int, n: int, k: int, cache_dir, packed: bool) -> str:
    from .autotune import ScheduleResolver

    slot = (n, k, str(cache_dir), packed)
    with _LOCK:
        resolver = _FUNCTIONAL_RESOLVERS.get(slot)
        if resolver is None:
            resolver = ScheduleResolver("mxfp8_prequant_fwd", n, k, "cache", cache_dir,
                                        variant="weight_prequant" if packed else "default")
            _FUNCTIONAL_RESOLVERS[slot] = resolver
        return _intern(resolver.resolve(m, _resolve_prequant(fwd_key)))


@torch._dynamo.assume_constant_result
def _select_keys(forward_config, config, dynamic_config, prequant_config, backward_config, packed: bool,
                 backend: str = "auto"):
    """Interned (forward, backward) schedule keys; a constant under torch.compile.  `backend="fused"` names the
    reference's one-kernel forward (rtx/fp8.py:292-312): unless the config already names a schedule, it selects
    the GEMM that quantizes the activations in its own quantizer warps (`fused_x`); `auto` and `materialized`
    are the quantize-once pipeline, which is what the reference's `auto` resolves to on these shapes."""
    if config is not None and forward_config is not None:
        raise ValueError("pass only forward_config, not both config aliases")
    if prequant_config is not None and dynamic_config is not None:
        raise ValueError("pass only dynamic_config, not both materialized config aliases")
    fwd = forward_config if forward_config is not None else config
    pre = dynamic_config if dynamic_config is not None else prequant_config
    if pre is None:
        if fwd is not None:
            pre = MXFP8PrequantConfig(quant=fwd.quant, gemm=fwd.gemm)
        else:
            pre = DEFAULT_MXFP8_INFERENCE_CONFIG if packed else DEFAULT_MXFP8_PREQUANT_CONFIG
    if backend == "fused" and pre.gemm.schedule == "auto":
        import dataclasses

        pre = dataclasses.replace(pre, gemm=MXFP8GemmConfig.for_schedule("fused_x"))
    bwd = backward_config or MXFP8BwdConfig()
    return _intern(pre), _intern(bwd)


def mxfp8_linear(x, weight, *, forward_config: Optional[MXFP8FwdConfig] = None, config: Optional[MXFP8FwdConfig] = None,
                 autotune: "AutotuneMode | bool | None" = None, tuning_policy: object = None,
                 autotune_cache_dir: "Path | str | None" = None, backend: MXFP8Backend = "auto",
                 dynamic_config: Optional[MXFP8PrequantConfig] = None,
                 prequant_config: Optional[MXFP8PrequantConfig] = None,
                 backward_config: Optional[MXFP8BwdConfig] = None) -> torch.Tensor:
    """Apply MXFP8 linear in dynamic or prequantized states (rtx/fp8.py:2019-2193).  Leading
    activation dimensions are flattened for the kernel and restored in the output."""
    _normalize_backend(backend)
    mode = _autotune_mode(autotune)
    x_packed, w_packed = isinstance(x, MXFP8Tensor), isinstance(weight, MXFP8Tensor)
    fwd_key, bwd_key = _select_keys(forward_config, config, dynamic_config, prequant_config, backward_config, w_packed,
                                    backend)
    if mode != "off" and not x_packed and not torch.compiler.is_compiling():
        # functional calls use stored winners only; first-use tuning belongs to the module, which owns its state
        n_w, k_w = mxfp8_matrix_shape(weight) if w_packed else (int(weight.shape[0]), int(weight.shape[-1]))
        fwd_key = _stored_winner_key(fwd_key, int(x.numel() // max(int(x.shape[-1]), 1)), n_w, k_w, autotune_cache_dir,
                                     w_packed)
    if x_packed and not w_packed:
        raise ValueError("a packed activation requires a packed weight")
    if w_packed:
        n, k = mxfp8_matrix_shape(weight)
        wq = mxfp8_qdata_2d(weight)
        ws = mxfp8_scales_for_kernel(weight)
        if x_packed:
            m, kx = mxfp8_matrix_shape(x)
            if kx != k:
                raise ValueError(f"K mismatch: x has {kx}, weight has {k}")
            out = torch.ops.rtx.mxfp8_linear_prequantized(mxfp8_qdata_2d(x), wq, mxfp8_scales_for_kernel(x), ws, m, n, k,
                                                          "mma128", "mma128", fwd_key)
            return out.reshape(*x._rtx_logical_shape[:-1], n)
        if x.shape[-1] != k:
            raise ValueError(f"K mismatch: x has {x.shape[-1]}, weight has {k}")
        if x.requires_grad:
            raise RuntimeError("a prequantized MXFP8 weight is inference-only; keep the BF16 master weight to train")
        x2d = x.reshape(-1, k)
        out = torch.ops.rtx.mxfp8_linear_dynamic_x_prequant_w(x2d, wq, ws, n, k, "mma128", fwd_key)
        return out.reshape(*x.shape[:-1], n)
    if x.shape[-1] != weight.shape[-1]:
        raise ValueError(f"K mismatch: x has {x.shape[-1]}, weight has {weight.shape[-1]}")
    x2d = x.reshape(-1, x.shape[-1])
    _check_inputs(x2d, weight)
    if torch.is_grad_enabled() and (x.requires_grad or weight.requires_grad):
        from . import fp8_bwd  # registers rtx::mxfp8_linear_train

        out = torch.ops.rtx.mxfp8_linear_train(x2d, weight, fwd_key, bwd_key)
    else:
        out = torch.ops.rtx.mxfp8_linear_prequant(x2d, weight, fwd_key)
    return out.reshape(*x.shape[:-1], weight.shape[0])


# --------------------------------------------------------------------------- module

class MXFP8Linear(nn.Module):
    """No-bias BF16-master linear with MXFP8 forward and backward GEMMs (rtx/fp8.py:2389-2775).

    Dynamic modules expose only `weight` (BF16) so BF16 / MXFP8 / NVFP4 models share checkpoints;
    packed modules store `weight_data`, `weight_scales`, `weight_packing_meta =
    [schema, layout code, in_features, storage_k]` (rtx/fp8.py:2500-2517).
    """

    __constants__ = ["in_features", "out_features", "backend", "weight_mode"]

    def __init__(self, in_features: int, out_features: int, bias: bool = False, *, device=None,
                 dtype: torch.dtype = torch.bfloat16, forward_config: Optional[MXFP8FwdConfig] = None,
                 config: Optional[MXFP8FwdConfig] = None, autotune: "AutotuneMode | bool | None" = None,
                 tuning_policy: object = None, autotune_cache_dir: "Path | str | None" = None,
                 backend: MXFP8Backend = "auto", dynamic_config: Optional[MXFP8PrequantConfig] = None,
                 prequant_config: Optional[MXFP8PrequantConfig] = None,
                 backward_config: Optional[MXFP8BwdConfig] = None,
                 packed_weight: Optional[MXFP8Tensor] = None) -> None:
        super().__init__()
        if bias:
            raise NotImplementedError("MXFP8Linear is a no-bias linear layer; pass bias=False")
        if dtype is not torch.bfloat16:
            raise TypeError(f"MXFP8Linear parameters must be BF16, got {dtype}")
        if config is not None and forward_config is not None:
            raise ValueError("pass only forward_config, not both config aliases")
        if prequant_config is not None and dynamic_config is not None:
            raise ValueError("pass only dynamic_config, not both materialized config aliases")
        self.in_features = int(in_features)
        self.out_features = int(out_features)
        self.forward_config = forward_config if forward_config is not None else config
        self.config = self.forward_config
        self.dynamic_config = dynamic_config if dynamic_config is not None else prequant_config
        self.prequant_config = self.dynamic_config
        self.backward_config = backward_config
        self.autotune = autotune
        self.tuning_policy = tuning_policy
        self.autotune_cache_dir = autotune_cache_dir
        self.backend = _normalize_backend(backend)
        self.weight_mode = "prequantized" if packed_weight is not None else "dynamic"
        from .autotune import ScheduleResolver

        self._resolver = ScheduleResolver("mxfp8_prequant_fwd", self.out_features, self.in_features,
                                          _autotune_mode(autotune), autotune_cache_dir,
                                          variant="weight_prequant" if packed_weight is not None else "default")
        # schedules travel as interned strings so that a compiled graph sees constants (rtx/fp8.py:376-415)
        self._forward_config_key, self._backward_config_key = _select_keys(
            self.forward_config, None, self.dynamic_config, None, backward_config, packed_weight is not None,
            self.backend)
        if packed_weight is None:
            weight = torch.empty(self.out_features, self.in_features, device=device, dtype=torch.bfloat16)
            self.weight = nn.Parameter(weight)
            self.reset_parameters()
        else:
            n, k = mxfp8_matrix_shape(packed_weight)
            if (n, k) != (self.out_features, self.in_features):
                raise ValueError(f"packed weight is {n}x{k}, module is {self.out_features}x{self.in_features}")
            layout = mxfp8_scale_layout(packed_weight)
            self._weight_scale_layout = layout
            self.register_parameter("weight", None)
            self.register_buffer("weight_data", mxfp8_qdata_2d(packed_weight).view(torch.uint8))
            self.register_buffer("weight_scales", packed_weight.scale.reshape(-1).view(torch.uint8))
            self.register_buffer("weight_packing_meta", torch.tensor(
                [PACKED_OPERAND_SCHEMA_VERSION, SCALE_LAYOUT_CODES[layout], self.in_features,
                 int(packed_weight.qdata.shape[-1])], dtype=torch.int64))

    def reset_parameters(self) -> None:
        nn.init.kaiming_uniform_(self.weight, a=5 ** 0.5)

    # -- conversion -----------------------------------------------------------------
    @classmethod
    def from_float(cls, module: nn.Linear, **kwargs) -> "MXFP8Linear":
        if module.bias is not None:
            raise NotImplementedError("MXFP8Linear is a no-bias linear layer")
        out = cls(module.in_features, module.out_features, device=module.weight.device, **kwargs)
        with torch.no_grad():
            out.weight.copy_(module.weight.to(torch.bfloat16))
        return out

    def to_quantized_weight(self, *, config: Optional[MXFP8QuantConfig] = None) -> "MXFP8Linear":
        """Inference copy with the weight packed once (rtx/fp8.py:2598-2629)."""
        if self.weight_mode == "prequantized":
            return self
        packed = quantize_mxfp8(self.weight.detach(), config=config)
        return MXFP8Linear(self.in_features, self.out_features, device=self.weight.device, backend=self.backend,
                           dynamic_config=self.dynamic_config, packed_weight=packed)

    def packed_weight(self) -> MXFP8Tensor:
        if self.weight_mode != "prequantized":
            raise RuntimeError("module holds a BF16 weight; call to_quantized_weight() first")
        layout = SCALE_LAYOUT_NAMES[int(self.weight_packing_meta[1])]
        return make_mxfp8_tensor(self.weight_data, self.weight_scales, (self.out_features, self.in_features), layout)

    def explain(self, m: Optional[int] = None) -> dict:
        """What forward() will run for this module; with `m` (token rows of a call) the schedule that
        `autotune=` resolves for that shape (a stored winner when one exists)."""
        key = self._forward_config_key
        out = {"format": "mxfp8", "weight_mode": self.weight_mode, "backend": self.backend,
               "pipeline": "quantize once + tcgen05 block-scaled GEMM (sm_100a)", "autotune": self._resolver.mode,
               "forward_key": key}
        if m is not None:
            cfg = self._resolver.resolve(int(m), _resolve_prequant(key))
            out.update(forward_key=_intern(cfg), gemm_schedule=cfg.gemm.schedule,
                       schedule_source=self._resolver.sources.get(int(m), "configured"))
        return out

    def _tuned_forward_key(self, x2d: torch.Tensor) -> str:
        """The forward schedule key of this call: the configured one, or what `autotune=` resolves for
        this M (stored winner / tuned on first use).  Constant under torch.compile (no tuning while tracing)."""
        if self._resolver.mode == "off" or torch.compiler.is_compiling():
            return self._forward_config_key
        m = int(x2d.shape[0])
        cfg = self._resolver.resolved.get(m)
        if cfg is None:
            cfg = self._resolver.resolve(m, _resolve_prequant(self._forward_config_key), self._evaluator(x2d))
        return _intern(cfg)

    def _candidate_call(self, x2d: torch.Tensor, cfg):
        """A zero-argument callable that runs this module's forward on `x2d` with the schedule `cfg`."""
        key = _intern(cfg)

        def run():
            with torch.no_grad():
                if self.weight_mode == "prequantized":
                    return torch.ops.rtx.mxfp8_linear_dynamic_x_prequant_w(
                        x2d, self.weight_data, self.weight_scales, self.out_features, self.in_features,
                        self._weight_scale_layout, key)
                return torch.ops.rtx.mxfp8_linear_prequant(x2d, self.weight, key)

        return run

    def _evaluator(self, x2d: torch.Tensor, warmup: int = 2, samples: int = 5):
        """Times one candidate schedule on this call's own operands (first-hit tuning)."""
        from .autotune import time_call

        return lambda cfg: time_call(self._candidate_call(x2d, cfg), warmup, samples)

    def to(self, *args, **kwargs):
        if self.weight_mode == "prequantized":
            reject_packed_dtype_conversion(args, kwargs, format_name="MXFP8")
        return super().to(*args, **kwargs)

    def extra_repr(self) -> str:
        return (f"in_features={self.in_features}, out_features={self.out_features}, bias=False, "
                f"weight_mode={self.weight_mode}, backend={self.backend}")

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        k, n = self.in_features, self.out_features
        if x.shape[-1] != k:
            raise ValueError(f"K mismatch: x has {x.shape[-1]}, weight has {k}")
        x2d = x.reshape(-1, k)
        fwd_key = self._tuned_forward_key(x2d)
        if self.weight_mode == "prequantized":
            if x.requires_grad and torch.is_grad_enabled():
                raise RuntimeError("a prequantized MXFP8 weight is inference-only; keep the BF16 master weight to train")
            out = torch.ops.rtx.mxfp8_linear_dynamic_x_prequant_w(x2d, self.weight_data, self.weight_scales, n, k,
                                                                  self._weight_scale_layout, fwd_key)
        elif (cache := _weight_cache.active()) is not None:
            # inside a quantized_weight_cache() scope: the weight operands come from the step's cache
            _check_inputs(x2d, self.weight)
            rounding = _rounding(_resolve_prequant(self._forward_config_key))
            if torch.is_grad_enabled() and (x.requires_grad or self.weight.requires_grad):
                out = _weight_cache.MXFP8CachedLinearFunction.apply(x2d, self.weight, cache, rounding)
            else:
                qw, sw = _weight_cache.mxfp8_rows(cache, self.weight, rounding)
                x2d = x2d if x2d.is_contiguous() else x2d.contiguous()
                qx, sx = ops.mxfp8_quantize(x2d, rounding=rounding)
                out = ops.mxfp8_gemm(qx, sx, qw, sw, int(x2d.shape[0]), n, k)
        elif torch.is_grad_enabled() and (x.requires_grad or self.weight.requires_grad):
            from . import fp8_bwd  # noqa: F401  (registers rtx::mxfp8_linear_train)

            out = torch.ops.rtx.mxfp8_linear_train(x2d, self.weight, fwd_key, self._backward_config_key)
        else:
            out = torch.ops.rtx.mxfp8_linear_prequant(x2d, self.weight, fwd_key)
        return out.reshape(*x.shape[:-1], n)


__all__ = ["MXFP8Linear", "mxfp8_linear", "quantize_mxfp8", "MXFP8PrequantConfig", "DEFAULT_MXFP8_PREQUANT_CONFIG",
           "DEFAULT_MXFP8_INFERENCE_CONFIG"]


# Inductor lowerings of the ops above (skipped quietly when Inductor's internals are unavailable)
from . import inductor as _inductor  # noqa: E402

_inductor.register_mxfp8_lowerings()
