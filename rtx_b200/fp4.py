"""NVFP4 frontend: `NVFP4Linear`, `nvfp4_linear`, `quantize_nvfp4` and the `rtx::nvfp4_*`
custom ops, with the reference's signatures (rtx/fp4.py:1501-1540, :1543-1973,
:2676-2942, :2945-3642) on top of the sm_100a kernels.

Numerics (PRECISION_POLICY of the reference): NVFP4 forward — E2M1 payload, E4M3
scale per 16 values, FP32 per-tensor outer scale — and MXFP8 backward on the saved
BF16 operands (rtx/fp4.py:1772-1794).  Scaling policies built for sm_100a:
`jit_row_region` (the default for dynamic operands: one outer scale per region of
rows, from the region's present |max|), `current` (outer scale from the tensor's
present |max|; power-of-two for dynamic operands, exact `amax/2688` for offline
weights), `delayed` (outer scale from the |max| history of earlier steps; the
current |max| is only observed, in the same pass that quantizes) and `block`
(outer scale 1).
"""

from __future__ import annotations

import functools
from pathlib import Path
from typing import Optional

import torch
from torch import nn

from ._oplib import custom_op
from . import _native as N
from . import fp8 as _fp8
from . import ops
from . import weight_cache as _weight_cache
from .configs import (DEFAULT_NVFP4_QUANT_CONFIG, MXFP8BwdConfig, NVFP4DynamicConfig, NVFP4Problem, NVFP4QuantConfig,
                      NVFP4ScaleConfig, config_from_key)
from .formats import (PACKED_OPERAND_SCHEMA_VERSION, SCALE_LAYOUT_CODES, SCALE_LAYOUT_NAMES, NVFP4Tensor,
                      make_nvfp4_tensor, nvfp4_matrix_shape, nvfp4_qdata_2d, nvfp4_scale_layout,
                      nvfp4_scales_for_kernel, nvfp4_storage_k, reject_packed_dtype_conversion)
from .types import AutotuneMode

DEFAULT_NVFP4_X_SCALE_REGION_ROWS = 5
DEFAULT_NVFP4_WEIGHT_SCALE_REGION_ROWS = 4
_LAYOUT_CODE = {"row_major": N.SCALE_ROW_MAJOR, "mma128": N.SCALE_MMA128}
_SCALE_MODE = {"exact": N.TENSOR_SCALE_EXACT, "power2": N.TENSOR_SCALE_POWER2}


@custom_op("rtx::nvfp4_outer_scale", mutates_args=(), device_types="cuda")
def nvfp4_outer_scale(x: torch.Tensor, mode: str) -> torch.Tensor:
    """FP32[1] outer decode scale of a BF16 matrix: one device pass (|max| reduction + scale rule),
    no host synchronisation.  The reference computes it with PyTorch reductions (rtx/fp4.py:343-365)."""
    if mode not in _SCALE_MODE:
        raise ValueError(f"unknown NVFP4 tensor scale mode {mode!r}")
    x = x if x.is_contiguous() else x.contiguous()
    return ops.nvfp4_tensor_scale(x, _SCALE_MODE[mode])


@nvfp4_outer_scale.register_fake
def _(x, mode):
    return x.new_empty((1,), dtype=torch.float32)


def _current_tensor_scale(tensor: torch.Tensor) -> torch.Tensor:
    """Exact two-level decode scale amax / (448 * 6); 1.0 for an all-zero tensor (rtx/fp4.py:343-350)."""
    return torch.ops.rtx.nvfp4_outer_scale(tensor.detach().reshape(-1, tensor.shape[-1]), "exact")


def _outer_tensor_scale(tensor: torch.Tensor, mode: str) -> torch.Tensor:
    """Outer decode scale consumed by the quantizer (rtx/fp4.py:354-365): `exact` or `power2`
    = 2^ceil(log2(max(amax/2688, FLT_MIN))), evaluated with the integer exponent rule of
    rtx/kernels/nvfp4_quant.py:117-143."""
    if mode not in _SCALE_MODE:
        raise ValueError(f"unknown NVFP4 tensor scale mode {mode!r}")
    return torch.ops.rtx.nvfp4_outer_scale(tensor.detach().reshape(-1, tensor.shape[-1]), mode)


def _check_bf16_cuda(t: torch.Tensor, name: str) -> None:
    if t.device.type != "cuda":
        raise ValueError(f"NVFP4 {name} must be a CUDA tensor")
    if t.dtype is not torch.bfloat16:
        raise TypeError(f"NVFP4 {name} must be BF16, got {t.dtype}")


def quantize_nvfp4(tensor: torch.Tensor, *, tensor_scale: Optional[torch.Tensor] = None,
                   config: Optional[NVFP4QuantConfig] = None) -> NVFP4Tensor:
    """Prequantize BF16 into the packed NVFP4 tensor (rtx/fp4.py:1501-1540); the default outer scale
    is the exact `amax / 2688`."""
    if tensor.ndim < 1 or tensor.dtype is not torch.bfloat16:
        raise TypeError("NVFP4 quantization requires a BF16 tensor")
    if tensor.device.type != "cuda":
        raise ValueError("NVFP4 quantization requires a CUDA tensor")
    source = tensor.reshape(-1, tensor.shape[-1])
    source = source if source.is_contiguous() else source.contiguous()
    rows, k = int(source.shape[0]), int(source.shape[1])
    selected = config or DEFAULT_NVFP4_QUANT_CONFIG
    rejection = selected.rejection(rows, k)
    if rejection is not None:
        raise RuntimeError(f"NVFP4 operand cannot be quantized: {rejection}")
    scale = _current_tensor_scale(source) if tensor_scale is None else tensor_scale
    if scale.dtype is not torch.float32 or scale.numel() != 1:
        raise TypeError("NVFP4 tensor_scale must be one FP32 value")
    if scale.device != source.device:
        raise ValueError("NVFP4 tensor_scale and source must share one device")
    q, s = ops.nvfp4_quantize(source, scale.reshape(1), layout=_LAYOUT_CODE[selected.scale_layout])
    q._base_inputs = (source, scale)
    s._base_inputs = (source, scale)
    return make_nvfp4_tensor(q, s, scale.reshape(()), tuple(int(v) for v in tensor.shape), selected.scale_layout)


@functools.lru_cache(maxsize=1024)
def _resolve_dynamic(key: str) -> NVFP4DynamicConfig:
    cfg = config_from_key(key)
    if not isinstance(cfg, NVFP4DynamicConfig):
        raise RuntimeError(f"config key does not name an NVFP4 forward schedule: {type(cfg).__name__}")
    rejection = cfg.rejection()
    if rejection is not None:
        raise RuntimeError(f"illegal NVFP4 forward schedule: {rejection}")
    return cfg


def _materialized_forward(x, weight, x_scale, weight_scale, output_scale):
    x = x if x.is_contiguous() else x.contiguous()
    weight = weight if weight.is_contiguous() else weight.contiguous()
    m, k = x.shape
    n = weight.shape[0]
    qx, sx = ops.nvfp4_quantize(x, x_scale)
    qw, sw = ops.nvfp4_quantize(weight, weight_scale)
    return ops.nvfp4_gemm(qx, sx, qw, sw, int(m), int(n), int(k), output_scale)


# --------------------------------------------------------------------------- custom ops

@custom_op("rtx::nvfp4_linear_materialized_fwd", mutates_args=(), device_types="cuda")
def nvfp4_linear_materialized_fwd(x: torch.Tensor, weight: torch.Tensor, x_scale: torch.Tensor,
                                  weight_scale: torch.Tensor, output_scale: torch.Tensor, key: str) -> torch.Tensor:
    """`current` policy: outer scales computed by the caller, dual quantize, GEMM x output_scale
    (rtx/fp4.py:1260-1313, _DynamicRunner :404-454)."""
    with ops.schedule_of(_resolve_dynamic(key).gemm):
        return _materialized_forward(x, weight, x_scale, weight_scale, output_scale)


@nvfp4_linear_materialized_fwd.register_fake
def _(x, weight, x_scale, weight_scale, output_scale, key):
    return x.new_empty((x.shape[0], weight.shape[0]), dtype=torch.bfloat16)


@custom_op("rtx::nvfp4_linear_materialized_train", mutates_args=(), device_types="cuda")
def nvfp4_linear_materialized_train(x: torch.Tensor, weight: torch.Tensor, x_scale: torch.Tensor,
                                    weight_scale: torch.Tensor, output_scale: torch.Tensor, key: str,
                                    bwd_key: str) -> torch.Tensor:
    with ops.schedule_of(_resolve_dynamic(key).gemm):
        return _materialized_forward(x, weight, x_scale, weight_scale, output_scale)


@nvfp4_linear_materialized_train.register_fake
def _(x, weight, x_scale, weight_scale, output_scale, key, bwd_key):
    return x.new_empty((x.shape[0], weight.shape[0]), dtype=torch.bfloat16)


def _nv_train_setup(ctx, inputs, output):
    ctx.save_for_backward(inputs[0], inputs[1])
    ctx.bwd_key = inputs[-1]
    ctx.n_inputs = len(inputs)


def _nv_train_backward(ctx, grad_output):
    """Backward of every NVFP4 op is the MXFP8 backward on the saved BF16 operands (rtx/fp4.py:1772-1794)."""
    from . import fp8_bwd  # noqa: F401  (registers the backward ops)

    x, weight = ctx.saved_tensors
    need_dx, need_dw = ctx.needs_input_grad[0], ctx.needs_input_grad[1]
    grad_output = grad_output.contiguous()
    dx = dw = None
    if need_dx and need_dw:
        dx, dw = torch.ops.rtx.mxfp8_linear_bwd(grad_output, x, weight, ctx.bwd_key)
    elif need_dx:
        dx = torch.ops.rtx.mxfp8_linear_dx(grad_output, x, weight, ctx.bwd_key)
    elif need_dw:
        dw = torch.ops.rtx.mxfp8_linear_dw(grad_output, x, weight, ctx.bwd_key)
    return (dx, dw) + (None,) * (ctx.n_inputs - 2)


nvfp4_linear_materialized_train.register_autograd(_nv_train_backward, setup_context=_nv_train_setup)


@custom_op("rtx::nvfp4_linear_block_fwd", mutates_args=(), device_types="cuda")
def nvfp4_linear_block_fwd(x: torch.Tensor, weight: torch.Tensor, key: str) -> torch.Tensor:
    """`block` policy: outer scale 1 folded out of both kernels (rtx/fp4.py:859-875)."""
    with ops.schedule_of(_resolve_dynamic(key).gemm):
        return _materialized_forward(x, weight, None, None, None)


@nvfp4_linear_block_fwd.register_fake
def _(x, weight, key):
    return x.new_empty((x.shape[0], weight.shape[0]), dtype=torch.bfloat16)


@custom_op("rtx::nvfp4_linear_block_train", mutates_args=(), device_types="cuda")
def nvfp4_linear_block_train(x: torch.Tensor, weight: torch.Tensor, key: str, bwd_key: str) -> torch.Tensor:
    with ops.schedule_of(_resolve_dynamic(key).gemm):
        return _materialized_forward(x, weight, None, None, None)


@nvfp4_linear_block_train.register_fake
def _(x, weight, key, bwd_key):
    return x.new_empty((x.shape[0], weight.shape[0]), dtype=torch.bfloat16)


nvfp4_linear_block_train.register_autograd(_nv_train_backward, setup_context=_nv_train_setup)


def _jit_row_region_forward(x, weight, key):
    cfg = _resolve_dynamic(key)
    if not cfg.jit_row_region:
        raise RuntimeError("the forward schedule carries no region geometry")
    x = x if x.is_contiguous() else x.contiguous()
    weight = weight if weight.is_contiguous() else weight.contiguous()
    with ops.schedule_of(cfg.gemm):
        return ops.nvfp4_linear_fwd_regions(x, weight, _fp8._workspace(x.device), cfg.x_scale_region_rows,
                                            cfg.weight_scale_region_rows,
                                            scale_mode=_SCALE_MODE[cfg.scale.tensor_scale_mode])


@custom_op("rtx::nvfp4_linear_jit_row_region_fwd", mutates_args=(), device_types="cuda")
def nvfp4_linear_jit_row_region_fwd(x: torch.Tensor, weight: torch.Tensor, key: str) -> torch.Tensor:
    """`jit_row_region` policy: per-region outer scales observed and applied inside the call
    (rtx/fp4.py:1604-1626, _JITRegionDynamicRunner :522-560); region sizes travel in the config key."""
    return _jit_row_region_forward(x, weight, key)


@nvfp4_linear_jit_row_region_fwd.register_fake
def _(x, weight, key):
    return x.new_empty((x.shape[0], weight.shape[0]), dtype=torch.bfloat16)


@custom_op("rtx::nvfp4_linear_jit_row_region_train", mutates_args=(), device_types="cuda")
def nvfp4_linear_jit_row_region_train(x: torch.Tensor, weight: torch.Tensor, key: str, bwd_key: str) -> torch.Tensor:
    return _jit_row_region_forward(x, weight, key)


@nvfp4_linear_jit_row_region_train.register_fake
def _(x, weight, key, bwd_key):
    return x.new_empty((x.shape[0], weight.shape[0]), dtype=torch.bfloat16)


nvfp4_linear_jit_row_region_train.register_autograd(_nv_train_backward, setup_context=_nv_train_setup)


@custom_op("rtx::nvfp4_linear_train_delayed",
                         mutates_args=("next_x_amax_state", "next_weight_amax_state"), device_types="cuda")
def nvfp4_linear_train_delayed(x: torch.Tensor, weight: torch.Tensor, x_amax_state: torch.Tensor,
                               weight_amax_state: torch.Tensor, next_x_amax_state: torch.Tensor,
                               next_weight_amax_state: torch.Tensor, forward_config_key: str,
                               materialized_config_key: str, backward_config_key: str) -> torch.Tensor:
    """`delayed` policy (rtx/fp4.py:1931-1957, _DelayedDynamicRunner :462-517): outer scales from the prior
    |max| histories, successor histories written into the `next_*` tensors (index 0 = this call's |max|)."""
    cfg = _resolve_dynamic(forward_config_key)
    if x_amax_state.data_ptr() == next_x_amax_state.data_ptr():
        raise ValueError("delayed x amax generations must not alias")
    if weight_amax_state.data_ptr() == next_weight_amax_state.data_ptr():
        raise ValueError("delayed weight amax generations must not alias")
    x = x if x.is_contiguous() else x.contiguous()
    weight = weight if weight.is_contiguous() else weight.contiguous()
    with ops.schedule_of(cfg.gemm):
        return ops.nvfp4_linear_fwd_delayed(x, weight, _fp8._workspace(x.device), x_amax_state, weight_amax_state,
                                            next_x_amax_state, next_weight_amax_state,
                                            window_max=cfg.scale.amax_history_algo == "window_max",
                                            scale_mode=_SCALE_MODE[cfg.scale.tensor_scale_mode])


@nvfp4_linear_train_delayed.register_fake
def _(x, weight, x_amax_state, weight_amax_state, next_x_amax_state, next_weight_amax_state, forward_config_key,
      materialized_config_key, backward_config_key):
    return x.new_empty((x.shape[0], weight.shape[0]), dtype=torch.bfloat16)


class _NVFP4DelayedAutograd(torch.autograd.Function):
    """Autograd shell around the state-mutating delayed forward (rtx/fp4.py:2635-2673): the histories are
    plain buffers, gradients flow to x and weight through the MXFP8 backward."""

    @staticmethod
    def forward(ctx, x, weight, x_state, w_state, next_x_state, next_w_state, key, materialized_key, bwd_key):
        ctx.save_for_backward(x, weight)
        ctx.bwd_key = bwd_key
        ctx.n_inputs = 9
        return torch.ops.rtx.nvfp4_linear_train_delayed(x, weight, x_state, w_state, next_x_state, next_w_state, key,
                                                        materialized_key, bwd_key)

    @staticmethod
    def backward(ctx, grad_output):
        return _nv_train_backward(ctx, grad_output)


def _delayed_amax_state(tensor: torch.Tensor, values: int) -> torch.Tensor:
    """History bootstrapped from the tensor's present |max|, no host synchronisation (rtx/fp4.py:368-373)."""
    amax = torch.amax(torch.abs(tensor.detach().float())).reshape(1)
    return amax.expand(values).clone()


@custom_op("rtx::nvfp4_linear_dynamic_x_prequant_w", mutates_args=(), device_types="cuda")
def nvfp4_linear_dynamic_x_prequant_w(x: torch.Tensor, weight_data: torch.Tensor, weight_block_scales: torch.Tensor,
                                      x_scale: torch.Tensor, output_scale: torch.Tensor, n: int, k: int, layout: str,
                                      key: str) -> torch.Tensor:
    """Packed weight, BF16 activations quantized on the fly (rtx/fp4.py:1628-1686)."""
    if x.dtype is not torch.bfloat16 or x.ndim != 2 or x.shape[1] != k:
        raise TypeError("x must be BF16 [M, K]")
    x = x if x.is_contiguous() else x.contiguous()
    qx, sx = ops.nvfp4_quantize(x, x_scale)
    sw = _kernel_block_scales(weight_block_scales, n, k, layout)
    with ops.schedule_of(_resolve_dynamic(key).gemm):
        return ops.nvfp4_gemm(qx, sx, weight_data.view(torch.uint8), sw, int(x.shape[0]), n, k, output_scale)


@nvfp4_linear_dynamic_x_prequant_w.register_fake
def _(x, weight_data, weight_block_scales, x_scale, output_scale, n, k, layout, key):
    return x.new_empty((x.shape[0], n), dtype=torch.bfloat16)


@custom_op("rtx::nvfp4_linear_prequant_w_current", mutates_args=(), device_types="cuda")
def nvfp4_linear_prequant_w_current(x: torch.Tensor, weight_data: torch.Tensor, weight_block_scales: torch.Tensor,
                                    weight_tensor_scale: torch.Tensor, n: int, k: int, layout: str,
                                    key: str) -> torch.Tensor:
    """Packed weight, BF16 activations with their exact current outer scale, all inside one call: what
    `NVFP4Linear.forward` does for a packed weight (rtx/fp4.py:3421-3446 `_current_tensor_scale` followed by
    `nvfp4_linear_dynamic_x_prequant_w`), without the separate scale op and product.  Decode-sized inputs
    take one kernel (M <= 4) or three chained launches; the bits equal the two-op route."""
    if x.dtype is not torch.bfloat16 or x.ndim != 2 or x.shape[1] != k:
        raise TypeError("x must be BF16 [M, K]")
    x = x if x.is_contiguous() else x.contiguous()
    sw = _kernel_block_scales(weight_block_scales, n, k, layout)
    with ops.schedule_of(_resolve_dynamic(key).gemm):
        return ops.nvfp4_linear_fwd_prequant_w(x, weight_data.view(torch.uint8), sw, weight_tensor_scale, n,
                                               _fp8._workspace(x.device), scale_mode=N.TENSOR_SCALE_EXACT)


@nvfp4_linear_prequant_w_current.register_fake
def _(x, weight_data, weight_block_scales, weight_tensor_scale, n, k, layout, key):
    return x.new_empty((x.shape[0], n), dtype=torch.bfloat16)


@custom_op("rtx::nvfp4_linear_prequantized", mutates_args=(), device_types="cuda")
def nvfp4_linear_prequantized(x_data: torch.Tensor, weight_data: torch.Tensor, x_block_scales: torch.Tensor,
                              weight_block_scales: torch.Tensor, output_scale: torch.Tensor, m: int, n: int, k: int,
                              x_layout: str, weight_layout: str, key: str) -> torch.Tensor:
    """Both operands packed (rtx/fp4.py:1689-1760)."""
    sx = _kernel_block_scales(x_block_scales, m, k, x_layout)
    sw = _kernel_block_scales(weight_block_scales, n, k, weight_layout)
    with ops.schedule_of(_resolve_dynamic(key).gemm):
        return ops.nvfp4_gemm(x_data.view(torch.uint8), sx, weight_data.view(torch.uint8), sw, m, n, k, output_scale)


@nvfp4_linear_prequantized.register_fake
def _(x_data, weight_data, x_block_scales, weight_block_scales, output_scale, m, n, k, x_layout, weight_layout, key):
    return x_data.new_empty((m, n), dtype=torch.bfloat16)


def _kernel_block_scales(scales: torch.Tensor, rows: int, k: int, layout: str) -> torch.Tensor:
    if layout == "mma128":
        return scales.reshape(-1).view(torch.uint8)
    from .formats.common import scales_row_major_to_mma128
    from .formats.nvfp4 import nvfp4_scale_chunks

    storage_k = nvfp4_storage_k(k)
    if layout == "row_major":
        return scales_row_major_to_mma128(scales, rows, storage_k // 16, nvfp4_scale_chunks(storage_k))
    raise RuntimeError(f"NVFP4 scale layout {layout!r} cannot feed the sm_100a GEMM")


# --------------------------------------------------------------------------- functional

@torch._dynamo.assume_constant_result
def _bwd_key(backward_config):
    return (backward_config or MXFP8BwdConfig()).to_key()


def _resolve_scale_region_rows(shared, x_rows, weight_rows):
    """The shared override or the asymmetric defaults X = 5, W = 4 (rtx/fp4.py:61-86)."""
    if shared is not None and shared <= 0:
        raise ValueError("scale_region_rows must be positive")
    rx = x_rows if x_rows is not None else shared if shared is not None else DEFAULT_NVFP4_X_SCALE_REGION_ROWS
    rw = (weight_rows if weight_rows is not None else shared if shared is not None
          else DEFAULT_NVFP4_WEIGHT_SCALE_REGION_ROWS)
    if rx <= 0 or rw <= 0:
        raise ValueError("X and weight scale-region rows must be positive")
    return int(rx), int(rw)


@torch._dynamo.assume_constant_result
def _dynamic_key(dynamic_config, scale_config, scaling, region_rows=(0, 0)):
    region = scaling == "jit_row_region"
    if scale_config is not None and scale_config.policy != scaling:
        # the policy is chosen by `scaling`; a scale_config contributes the scale mode and history settings
        import dataclasses
        scale_config = dataclasses.replace(scale_config, policy=scaling)
    cfg = dynamic_config or NVFP4DynamicConfig(
        scale=scale_config or NVFP4ScaleConfig(policy=scaling,
                                               tensor_scale_mode="exact" if scaling == "block" else "power2"),
        x_scale_region_rows=region_rows[0] if region else 0,
        weight_scale_region_rows=region_rows[1] if region else 0)
    rejection = cfg.rejection()
    if rejection is not None:
        raise RuntimeError(f"illegal NVFP4 forward schedule: {rejection}")
    return cfg, cfg.to_key()


def nvfp4_linear(x, weight, *, scale_config: Optional[NVFP4ScaleConfig] = None,
                 backward_config: Optional[MXFP8BwdConfig] = None, scaling: Optional[str] = None,
                 scale_region_rows: Optional[int] = None, x_scale_region_rows: Optional[int] = None,
                 weight_scale_region_rows: Optional[int] = None, backend: str = "auto",
                 autotune: "AutotuneMode | bool | None" = None, tuning_policy: object = None,
                 autotune_cache_dir: "Path | str | None" = None, dynamic_config: Optional[NVFP4DynamicConfig] = None,
                 weight_prequant_config=None, fully_prequant_config=None) -> torch.Tensor:
    """Apply NVFP4 forward and MXFP8 backward to BF16 or packed operands (rtx/fp4.py:2676-2942)."""
    w_packed, x_packed = isinstance(weight, NVFP4Tensor), isinstance(x, NVFP4Tensor)
    if scaling is None:
        # dynamic BF16 operands default to the row-region policy; a packed weight to current activation
        # scaling (rtx/fp4.py:2730-2760: JIT regions need both operands dynamic)
        scaling = (scale_config.policy if scale_config is not None
                   else "current" if w_packed else "jit_row_region")
    if scaling not in ("current", "jit_row_region", "block"):
        raise ValueError("functional NVFP4 scaling must be current, jit_row_region, or block")
    if scaling == "jit_row_region" and w_packed:
        raise ValueError("jit_row_region scaling requires dynamic BF16 X and W; a packed weight uses current scaling")
    _fp8._normalize_backend(backend)
    mode = _fp8._autotune_mode(autotune)
    if x_packed and not w_packed:
        raise ValueError("a packed activation requires a packed weight")
    bwd_key = _bwd_key(backward_config)
    region_rows = (_resolve_scale_region_rows(scale_region_rows, x_scale_region_rows, weight_scale_region_rows)
                   if scaling == "jit_row_region" else (0, 0))
    cfg, key = _dynamic_key(dynamic_config, scale_config, scaling, region_rows)
    if mode != "off" and not x_packed and not torch.compiler.is_compiling():
        # functional calls use stored winners only (first-use tuning belongs to the module, which owns its state):
        # the family and variant a module of the same operand state and policy would look up
        n_w, k_w = nvfp4_matrix_shape(weight) if w_packed else (int(weight.shape[0]), int(weight.shape[-1]))
        cfg = _stored_winner_config(cfg, int(x.numel() // max(int(x.shape[-1]), 1)), n_w, k_w, autotune_cache_dir,
                                    w_packed, scaling)
        key = cfg.to_key()
    if w_packed:
        n, k = nvfp4_matrix_shape(weight)
        wq, wscales = nvfp4_qdata_2d(weight), nvfp4_scales_for_kernel(weight)
        w_scale = weight.per_tensor_scale.reshape(1).float()
        if x_packed:
            m, kx = nvfp4_matrix_shape(x)
            if kx != k:
                raise ValueError(f"K mismatch: x has {kx}, weight has {k}")
            out_scale = x.per_tensor_scale.reshape(1).float() * w_scale
            out = torch.ops.rtx.nvfp4_linear_prequantized(nvfp4_qdata_2d(x), wq, nvfp4_scales_for_kernel(x), wscales,
                                                          out_scale, m, n, k, "mma128", "mma128", key)
            return out.reshape(*x._rtx_logical_shape[:-1], n)
        _check_bf16_cuda(x, "activation")
        if x.shape[-1] != k:
            raise ValueError(f"K mismatch: x has {x.shape[-1]}, weight has {k}")
        if x.requires_grad:
            raise RuntimeError("a prequantized NVFP4 weight is inference-only; keep the BF16 master weight to train")
        x2d = x.reshape(-1, k)
        # rtx/fp4.py:3421-3446: exact current scale of the activations for packed weights
        out = torch.ops.rtx.nvfp4_linear_prequant_w_current(x2d, wq, wscales, w_scale, n, k, "mma128", key)
        return out.reshape(*x.shape[:-1], n)
    _check_bf16_cuda(x, "activation")
    _check_bf16_cuda(weight, "weight")
    if x.shape[-1] != weight.shape[-1]:
        raise ValueError(f"K mismatch: x has {x.shape[-1]}, weight has {weight.shape[-1]}")
    x2d = x.reshape(-1, x.shape[-1])
    train = torch.is_grad_enabled() and (x.requires_grad or weight.requires_grad)
    if train:
        from . import fp8_bwd  # noqa: F401
    if cfg.scale.policy == "block":
        out = (torch.ops.rtx.nvfp4_linear_block_train(x2d, weight, key, bwd_key) if train
               else torch.ops.rtx.nvfp4_linear_block_fwd(x2d, weight, key))
    elif cfg.scale.policy == "jit_row_region":
        out = (torch.ops.rtx.nvfp4_linear_jit_row_region_train(x2d, weight, key, bwd_key) if train
               else torch.ops.rtx.nvfp4_linear_jit_row_region_fwd(x2d, weight, key))
    else:
        mode = cfg.scale.tensor_scale_mode
        x_scale = _outer_tensor_scale(x2d.detach(), mode)
        w_scale = _outer_tensor_scale(weight.detach(), mode)
        output_scale = x_scale * w_scale                # rtx/fp4.py:2919-2921
        out = (torch.ops.rtx.nvfp4_linear_materialized_train(x2d, weight, x_scale, w_scale, output_scale, key, bwd_key)
               if train else
               torch.ops.rtx.nvfp4_linear_materialized_fwd(x2d, weight, x_scale, w_scale, output_scale, key))
    return out.reshape(*x.shape[:-1], weight.shape[0])


_FUNCTIONAL_RESOLVERS: dict = {}


def _stored_winner_config(cfg: NVFP4DynamicConfig, m: int, n: int, k: int, cache_dir, packed: bool, scaling: str):
    from .autotune import ScheduleResolver

    slot = (n, k, str(cache_dir), packed, scaling)
    resolver = _FUNCTIONAL_RESOLVERS.get(slot)
    if resolver is None:
        resolver = ScheduleResolver("nvfp4_weight_prequant_fwd" if packed else "nvfp4_dynamic_fwd", n, k, "cache",
                                    cache_dir, variant=scaling)
        _FUNCTIONAL_RESOLVERS[slot] = resolver
    return resolver.resolve(m, cfg)


# --------------------------------------------------------------------------- module

class NVFP4Linear(nn.Module):
    """No-bias BF16-master linear with NVFP4 forward and MXFP8 backward (rtx/fp4.py:2945-3642).
    Packed modules store `weight_data`, `weight_block_scales`, `weight_tensor_scale`,
    `weight_packing_meta = [schema, layout code, in_features, storage_k]` (rtx/fp4.py:3176-3196)."""

    __constants__ = ["in_features", "out_features", "scaling", "weight_mode"]

    def __init__(self, in_features: int, out_features: int, bias: bool = False, *, device=None,
                 dtype: torch.dtype = torch.bfloat16, scale_config: Optional[NVFP4ScaleConfig] = None,
                 backward_config: Optional[MXFP8BwdConfig] = None, scaling: Optional[str] = None,
                 scale_region_rows: Optional[int] = None, x_scale_region_rows: Optional[int] = None,
                 weight_scale_region_rows: Optional[int] = None, backend: str = "auto",
                 packed_weight: Optional[NVFP4Tensor] = None, autotune: "AutotuneMode | bool | None" = None,
                 tuning_policy: object = None, autotune_cache_dir: "Path | str | None" = None,
                 dynamic_config: Optional[NVFP4DynamicConfig] = None, weight_prequant_config=None,
                 fully_prequant_config=None) -> None:
        super().__init__()
        if bias:
            raise NotImplementedError("NVFP4Linear is a no-bias linear layer; pass bias=False")
        if dtype is not torch.bfloat16:
            raise TypeError(f"NVFP4Linear parameters must be BF16, got {dtype}")
        if scaling is None:
            # rtx/fp4.py:3010-3040: dynamic BF16 operands default to the row-region policy, a packed weight to
            # current activation scaling (JIT regions need both operands dynamic)
            scaling = (scale_config.policy if scale_config is not None
                       else "current" if packed_weight is not None else "jit_row_region")
        if scaling not in ("delayed", "current", "jit_row_region", "block"):
            raise ValueError("NVFP4 scaling must be delayed, current, jit_row_region, or block")
        if scaling in ("jit_row_region", "delayed") and packed_weight is not None:
            raise ValueError(f"{scaling} scaling requires dynamic BF16 X and W; a packed weight uses current scaling")
        self.in_features, self.out_features = int(in_features), int(out_features)
        self.scaling = scaling
        self.scale_config = scale_config
        self.backward_config = backward_config
        self.backend = _fp8._normalize_backend(backend)
        self.autotune = autotune
        self.tuning_policy = tuning_policy
        self.autotune_cache_dir = autotune_cache_dir
        self.dynamic_config = dynamic_config
        self.x_scale_region_rows, self.weight_scale_region_rows = _resolve_scale_region_rows(
            scale_region_rows, x_scale_region_rows, weight_scale_region_rows)
        self.weight_mode = "prequantized" if packed_weight is not None else "dynamic"
        self._dynamic_config, self._forward_key = _dynamic_key(
            dynamic_config, scale_config, scaling, (self.x_scale_region_rows, self.weight_scale_region_rows))
        self._backward_key = _bwd_key(backward_config)
        from .autotune import ScheduleResolver

        # `autotune=`: stored winners of the call's (M, N, K), or first-use tuning (rtx/fp4.py:1065-1207)
        self._resolver = ScheduleResolver(
            "nvfp4_weight_prequant_fwd" if packed_weight is not None else "nvfp4_dynamic_fwd", self.out_features,
            self.in_features, _fp8._autotune_mode(autotune), autotune_cache_dir, variant=scaling)
        self._delayed_initialized = False
        self._delayed_problem = None
        self._x_amax_state = self._weight_amax_state = None
        self._next_x_amax_state = self._next_weight_amax_state = None
        if packed_weight is None:
            self.weight = nn.Parameter(torch.empty(self.out_features, self.in_features, device=device,
                                                   dtype=torch.bfloat16))
            nn.init.kaiming_uniform_(self.weight, a=5 ** 0.5)
        else:
            n, k = nvfp4_matrix_shape(packed_weight)
            if (n, k) != (self.out_features, self.in_features):
                raise ValueError(f"packed weight is {n}x{k}, module is {self.out_features}x{self.in_features}")
            layout = nvfp4_scale_layout(packed_weight)
            self._weight_scale_layout = layout
            self.register_parameter("weight", None)
            self.register_buffer("weight_data", nvfp4_qdata_2d(packed_weight))
            self.register_buffer("weight_block_scales", packed_weight.scale.reshape(-1).view(torch.uint8))
            self.register_buffer("weight_tensor_scale", packed_weight.per_tensor_scale.reshape(1).float())
            self.register_buffer("weight_packing_meta", torch.tensor(
                [PACKED_OPERAND_SCHEMA_VERSION, SCALE_LAYOUT_CODES[layout], self.in_features,
                 nvfp4_storage_k(self.in_features)], dtype=torch.int64))

    @classmethod
    def from_float(cls, module: nn.Linear, **kwargs) -> "NVFP4Linear":
        if module.bias is not None:
            raise NotImplementedError("NVFP4Linear is a no-bias linear layer")
        out = cls(module.in_features, module.out_features, device=module.weight.device, **kwargs)
        with torch.no_grad():
            out.weight.copy_(module.weight.to(torch.bfloat16))
        return out

    def to_quantized_weight(self, *, config: Optional[NVFP4QuantConfig] = None) -> "NVFP4Linear":
        if self.weight_mode == "prequantized":
            return self
        packed = quantize_nvfp4(self.weight.detach(), config=config)
        return NVFP4Linear(self.in_features, self.out_features, device=self.weight.device, scaling="current",
                           packed_weight=packed)

    def packed_weight(self) -> NVFP4Tensor:
        if self.weight_mode != "prequantized":
            raise RuntimeError("module holds a BF16 weight; call to_quantized_weight() first")
        layout = SCALE_LAYOUT_NAMES[int(self.weight_packing_meta[1])]
        return make_nvfp4_tensor(self.weight_data, self.weight_block_scales, self.weight_tensor_scale.reshape(()),
                                 (self.out_features, self.in_features), layout)

    def reset_delayed_scales(self) -> None:
        """Drop the |max| histories of the delayed policy; the next forward re-initialises them from its
        own operands (rtx/fp4.py:3269-3283).  Called after state loading and when training is re-entered."""
        self._delayed_initialized = False
        self._delayed_problem = None

    def _load_from_state_dict(self, *args, **kwargs):
        super()._load_from_state_dict(*args, **kwargs)
        self.reset_delayed_scales()

    def train(self, mode: bool = True):
        if mode and not self.training:
            self.reset_delayed_scales()
        return super().train(mode)

    def _forward_delayed(self, x2d: torch.Tensor, key: Optional[str] = None) -> torch.Tensor:
        """History handling of the delayed policy (rtx/fp4.py:3452-3535): (re)initialise from current data when
        the problem (device, stream, shape) changes, run, then swap the two generations.  The policy is a
        forward one: eval / no_grad consume and publish histories exactly like training."""
        problem = (x2d.device.type, x2d.device.index, torch.cuda.current_stream(x2d.device).cuda_stream,
                   int(x2d.shape[0]), self.out_features, self.in_features)
        if not self._delayed_initialized or self._delayed_problem != problem:
            with torch.no_grad():
                values = self._dynamic_config.scale.amax_history_len
                self._x_amax_state = _delayed_amax_state(x2d, values)
                self._weight_amax_state = _delayed_amax_state(self.weight, values)
                self._next_x_amax_state = torch.empty_like(self._x_amax_state)
                self._next_weight_amax_state = torch.empty_like(self._weight_amax_state)
            self._delayed_initialized, self._delayed_problem = True, problem
        args = (x2d, self.weight, self._x_amax_state, self._weight_amax_state, self._next_x_amax_state,
                self._next_weight_amax_state, key or self._forward_key, key or self._forward_key, self._backward_key)
        if torch.is_grad_enabled() and (x2d.requires_grad or self.weight.requires_grad):
            from . import fp8_bwd  # noqa: F401  (registers the backward ops)
            out = _NVFP4DelayedAutograd.apply(*args)
        else:
            out = torch.ops.rtx.nvfp4_linear_train_delayed(*args)
        self._x_amax_state, self._next_x_amax_state = self._next_x_amax_state, self._x_amax_state
        self._weight_amax_state, self._next_weight_amax_state = self._next_weight_amax_state, self._weight_amax_state
        return out

    def explain(self, m: Optional[int] = None) -> dict:
        """What forward() runs; with `m` (token rows of a call) also the GEMM schedule `autotune=` resolves for it."""
        out = {"format": "nvfp4", "weight_mode": self.weight_mode, "scaling": self.scaling,
               "x_scale_region_rows": self.x_scale_region_rows if self.scaling == "jit_row_region" else 0,
               "weight_scale_region_rows": self.weight_scale_region_rows if self.scaling == "jit_row_region" else 0,
               "pipeline": "outer scale(s) + quantize once + tcgen05 mxf4nvf4 GEMM (sm_100a)", "backward": "mxfp8",
               "autotune": self._resolver.mode, "forward_key": self._forward_key}
        if m is not None:
            cfg = self._resolver.resolve(int(m), self._dynamic_config)
            out.update(forward_key=cfg.to_key(), gemm_schedule=cfg.gemm.schedule,
                       schedule_source=self._resolver.sources.get(int(m), "configured"))
        return out

    def _tuned_forward_key(self, x2d: torch.Tensor) -> str:
        """The forward schedule key of this call: the configured one, or what `autotune=` resolves for this M.
        The delayed policy carries state from call to call, so it is never re-run for timing: it uses stored
        winners only.  Constant while torch.compile traces."""
        if self._resolver.mode == "off" or torch.compiler.is_compiling():
            return self._forward_key
        m = int(x2d.shape[0])
        cfg = self._resolver.resolved.get(m)
        if cfg is None:
            evaluate = None if self.scaling == "delayed" else self._evaluator(x2d)
            cfg = self._resolver.resolve(m, self._dynamic_config, evaluate)
        return cfg.to_key()

    def _candidate_call(self, x2d: torch.Tensor, cfg):
        """A zero-argument callable that runs this module's forward on `x2d` with the schedule `cfg`
        (the configured schedule is put back after every call)."""

        def run():
            saved = self._forward_key, self._dynamic_config, self._resolver.mode
            self._forward_key, self._dynamic_config, self._resolver.mode = cfg.to_key(), cfg, "off"
            try:
                with torch.no_grad():
                    return self.forward(x2d)
            finally:
                self._forward_key, self._dynamic_config, self._resolver.mode = saved

        return run

    def _evaluator(self, x2d: torch.Tensor, warmup: int = 2, samples: int = 5):
        from .autotune import time_call

        return lambda cfg: time_call(self._candidate_call(x2d, cfg), warmup, samples)

    def to(self, *args, **kwargs):
        if self.weight_mode == "prequantized":
            reject_packed_dtype_conversion(args, kwargs, format_name="NVFP4")
        return super().to(*args, **kwargs)

    def extra_repr(self) -> str:
        return (f"in_features={self.in_features}, out_features={self.out_features}, bias=False, "
                f"weight_mode={self.weight_mode}, scaling={self.scaling}")

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        k, n = self.in_features, self.out_features
        if x.shape[-1] != k:
            raise ValueError(f"K mismatch: x has {x.shape[-1]}, weight has {k}")
        x2d = x.reshape(-1, k)
        key, bwd_key = self._tuned_forward_key(x2d), self._backward_key
        if self.weight_mode == "prequantized":
            if x.requires_grad and torch.is_grad_enabled():
                raise RuntimeError("a prequantized NVFP4 weight is inference-only; keep the BF16 master weight to train")
            # exact current outer scale of the activations (rtx/fp4.py:3421-3446), computed inside the call
            out = torch.ops.rtx.nvfp4_linear_prequant_w_current(
                x2d, self.weight_data, self.weight_block_scales, self.weight_tensor_scale, n, k,
                self._weight_scale_layout, key)
            return out.reshape(*x.shape[:-1], n)
        if self._dynamic_config.scale.policy == "delayed":
            return self._forward_delayed(x2d, key).reshape(*x.shape[:-1], n)
        train = torch.is_grad_enabled() and (x.requires_grad or self.weight.requires_grad)
        if train:
            from . import fp8_bwd  # noqa: F401  (registers the backward ops)
        if self._dynamic_config.scale.policy == "block":
            out = (torch.ops.rtx.nvfp4_linear_block_train(x2d, self.weight, key, bwd_key) if train
                   else torch.ops.rtx.nvfp4_linear_block_fwd(x2d, self.weight, key))
        elif self._dynamic_config.scale.policy == "jit_row_region":
            cache = _weight_cache.active()
            if cache is not None:
                # inside a quantized_weight_cache() scope: weight payload, block and region scales are reused
                _check_bf16_cuda(x2d, "activation")
                cfg = self._dynamic_config
                args = (cfg.x_scale_region_rows, cfg.weight_scale_region_rows, _SCALE_MODE[cfg.scale.tensor_scale_mode])
                out = (_weight_cache.NVFP4CachedRegionLinearFunction.apply(x2d, self.weight, cache, *args) if train
                       else _weight_cache.nvfp4_linear_regions_cached(cache, x2d, self.weight, *args))
            else:
                out = (torch.ops.rtx.nvfp4_linear_jit_row_region_train(x2d, self.weight, key, bwd_key) if train
                       else torch.ops.rtx.nvfp4_linear_jit_row_region_fwd(x2d, self.weight, key))
        else:
            mode = self._dynamic_config.scale.tensor_scale_mode
            x_scale = torch.ops.rtx.nvfp4_outer_scale(x2d.detach(), mode)
            w_scale = torch.ops.rtx.nvfp4_outer_scale(self.weight.detach(), mode)
            output_scale = x_scale * w_scale                                   # rtx/fp4.py:2919-2921
            out = (torch.ops.rtx.nvfp4_linear_materialized_train(x2d, self.weight, x_scale, w_scale, output_scale, key,
                                                                 bwd_key) if train else
                   torch.ops.rtx.nvfp4_linear_materialized_fwd(x2d, self.weight, x_scale, w_scale, output_scale, key))
        return out.reshape(*x.shape[:-1], n)


def _clear_runtime_caches() -> dict:
    return {}


__all__ = ["NVFP4Linear", "nvfp4_linear", "quantize_nvfp4", "DEFAULT_NVFP4_X_SCALE_REGION_ROWS",
           "DEFAULT_NVFP4_WEIGHT_SCALE_REGION_ROWS"]


# Inductor lowerings of the ops above (skipped quietly when Inductor's internals are unavailable)
from . import inductor as _inductor  # noqa: E402

_inductor.register_nvfp4_lowerings()
