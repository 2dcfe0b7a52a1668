"""MXFP8 backward frontend (rtx/fp8_bwd.py:1016-1248, :1481-1738).

    dX[M,K] = dY[M,N] W[N,K]     operands requantized in 32-blocks along N
    dW[N,K] = dY^T[N,M] X[M,K]   operands requantized in 32-blocks along M

Both outputs are BF16 as in the reference; the accumulation is FP32 in TMEM over
the whole contraction (no split-K workspace or reduce pass is needed).  The
data-parallel path asks for FP32 dW through `dw_dtype` so that partial dW of
different ranks are summed in FP32 before the one BF16 rounding.
"""

from __future__ import annotations

from pathlib import Path
from typing import Optional, Tuple

import torch

from ._oplib import custom_op
from . import fp8 as _fp8
from . import ops
from .configs import MXFP8BwdConfig, config_from_key

_ALIGN = 8  # elements; the packed result keeps dW 16-byte aligned behind dX (rtx/fp8_bwd.py:1251-1267)


def _bwd_config(key: str) -> MXFP8BwdConfig:
    cfg = config_from_key(key)
    if not isinstance(cfg, MXFP8BwdConfig):
        raise RuntimeError(f"config key does not name an MXFP8 backward schedule: {type(cfg).__name__}")
    rejection = cfg.rejection()
    if rejection is not None:
        raise RuntimeError(f"illegal MXFP8 backward schedule: {rejection}")
    return cfg


def _check_bwd(grad_output, x, weight) -> None:
    for name, t in (("grad_output", grad_output), ("x", x), ("weight", weight)):
        if t is None:
            continue
        if t.device.type != "cuda":
            raise ValueError(f"{name} must be a CUDA tensor")
        if t.dtype is not torch.bfloat16:
            raise TypeError(f"{name} must be BF16, got {t.dtype}")
        if t.ndim != 2:
            raise ValueError(f"{name} must be two-dimensional")
    if x is not None and grad_output.shape[0] != x.shape[0]:
        raise ValueError("grad_output and x disagree on M")
    if weight is not None and grad_output.shape[1] != weight.shape[0]:
        raise ValueError("grad_output and weight disagree on N")
    if x is not None and weight is not None and x.shape[1] != weight.shape[1]:
        raise ValueError("x and weight disagree on K")


def _contig(t):
    return t if t is None or t.is_contiguous() else t.contiguous()


def _run(grad_output, x, weight, need_dx, need_dw, dw_dtype=torch.bfloat16):
    _check_bwd(grad_output, x if need_dw else None, weight if need_dx else None)
    return ops.mxfp8_linear_bwd(_contig(grad_output), _contig(x) if need_dw else None,
                                _contig(weight) if need_dx else None, _fp8._workspace(grad_output.device),
                                need_dx=need_dx, need_dw=need_dw, dw_dtype=dw_dtype)


@custom_op("rtx::mxfp8_linear_bwd", mutates_args=(), device_types="cuda")
def mxfp8_linear_bwd(grad_output: torch.Tensor, x: torch.Tensor, weight: torch.Tensor,
                     config_key: str) -> Tuple[torch.Tensor, torch.Tensor]:
    _bwd_config(config_key)
    dx, dw = _run(grad_output, x, weight, True, True)
    return dx, dw


@mxfp8_linear_bwd.register_fake
def _(grad_output, x, weight, config_key):
    return torch.empty_like(x), torch.empty_like(weight)


@custom_op("rtx::mxfp8_linear_bwd_packed", mutates_args=(), device_types="cuda")
def mxfp8_linear_bwd_packed(grad_output: torch.Tensor, x: torch.Tensor, weight: torch.Tensor,
                            config_key: str) -> torch.Tensor:
    """One flat allocation `[dX | pad to 8 elements | dW]` (rtx/fp8_bwd.py:1040-1094)."""
    _bwd_config(config_key)
    dx, dw = _run(grad_output, x, weight, True, True)
    dx_n = dx.numel()
    dw_off = (dx_n + _ALIGN - 1) // _ALIGN * _ALIGN
    flat = torch.empty(dw_off + dw.numel(), dtype=torch.bfloat16, device=dx.device)
    flat[:dx_n].copy_(dx.reshape(-1))
    flat[dw_off:].copy_(dw.reshape(-1))
    return flat


@mxfp8_linear_bwd_packed.register_fake
def _(grad_output, x, weight, config_key):
    dx_n = x.numel()
    dw_off = (dx_n + _ALIGN - 1) // _ALIGN * _ALIGN
    return x.new_empty((dw_off + weight.numel(),), dtype=torch.bfloat16)


def unpack_bwd(flat: torch.Tensor, x_shape, w_shape):
    dx_n = x_shape[0] * x_shape[1]
    dw_off = (dx_n + _ALIGN - 1) // _ALIGN * _ALIGN
    return flat[:dx_n].view(x_shape), flat[dw_off:dw_off + w_shape[0] * w_shape[1]].view(w_shape)


@custom_op("rtx::mxfp8_linear_dx", mutates_args=(), device_types="cuda")
def mxfp8_linear_dx(grad_output: torch.Tensor, x: torch.Tensor, weight: torch.Tensor,
                    config_key: str) -> torch.Tensor:
    """dX only; `x` gives the result's shape, as in the reference (rtx/fp8_bwd.py:1097-1118)."""
    _bwd_config(config_key)
    return _run(grad_output, None, weight, True, False)[0]


@mxfp8_linear_dx.register_fake
def _(grad_output, x, weight, config_key):
    return torch.empty_like(x)


@custom_op("rtx::mxfp8_linear_dw", mutates_args=(), device_types="cuda")
def mxfp8_linear_dw(grad_output: torch.Tensor, x: torch.Tensor, weight: torch.Tensor,
                    config_key: str) -> torch.Tensor:
    """dW only; `weight` gives the result's shape (rtx/fp8_bwd.py:1121-1142)."""
    _bwd_config(config_key)
    return _run(grad_output, x, None, False, True)[1]


@mxfp8_linear_dw.register_fake
def _(grad_output, x, weight, config_key):
    return torch.empty_like(weight)


# Launch-only overloads writing into caller-provided tensors (rtx/fp8_bwd.py:1145-1248): compiled graphs
# allocate the results in their memory planner and call these.
_OUT_LIBRARY = torch.library.Library("rtx", "FRAGMENT")
_OUT_TAGS = (torch.Tag.out,) if hasattr(torch.Tag, "out") else ()
_OUT_LIBRARY.define("mxfp8_linear_bwd.out(Tensor grad_output, Tensor x, Tensor weight, str config_key, *, "
                    "Tensor(a!) grad_x, Tensor(b!) grad_weight) -> (Tensor(a!), Tensor(b!))", tags=_OUT_TAGS)
_OUT_LIBRARY.define("mxfp8_linear_dx.out(Tensor grad_output, Tensor x, Tensor weight, str config_key, *, "
                    "Tensor(a!) grad_x) -> Tensor(a!)", tags=_OUT_TAGS)
_OUT_LIBRARY.define("mxfp8_linear_dw.out(Tensor grad_output, Tensor x, Tensor weight, str config_key, *, "
                    "Tensor(a!) grad_weight) -> Tensor(a!)", tags=_OUT_TAGS)


def _run_out(grad_output, x, weight, need_dx, need_dw, grad_x=None, grad_weight=None):
    ops.mxfp8_linear_bwd(_contig(grad_output), _contig(x) if need_dw else None, _contig(weight) if need_dx else None,
                         _fp8._workspace(grad_output.device), need_dx=need_dx, need_dw=need_dw, dx_out=grad_x,
                         dw_out=grad_weight)


@torch.library.impl("rtx::mxfp8_linear_bwd.out", "cuda")
def _bwd_out(grad_output, x, weight, config_key, *, grad_x, grad_weight):
    _bwd_config(config_key)
    _run_out(grad_output, x, weight, True, True, grad_x, grad_weight)
    return grad_x, grad_weight


@torch.library.impl("rtx::mxfp8_linear_dx.out", "cuda")
def _dx_out(grad_output, x, weight, config_key, *, grad_x):
    _bwd_config(config_key)
    _run_out(grad_output, x, weight, True, False, grad_x=grad_x)
    return grad_x


@torch.library.impl("rtx::mxfp8_linear_dw.out", "cuda")
def _dw_out(grad_output, x, weight, config_key, *, grad_weight):
    _bwd_config(config_key)
    _run_out(grad_output, x, weight, False, True, grad_weight=grad_weight)
    return grad_weight


@torch.library.register_fake("rtx::mxfp8_linear_bwd.out")
def _(grad_output, x, weight, config_key, *, grad_x, grad_weight):
    return grad_x, grad_weight


@torch.library.register_fake("rtx::mxfp8_linear_dx.out")
def _(grad_output, x, weight, config_key, *, grad_x):
    return grad_x


@torch.library.register_fake("rtx::mxfp8_linear_dw.out")
def _(grad_output, x, weight, config_key, *, grad_weight):
    return grad_weight


@custom_op("rtx::mxfp8_linear_dw_f32", mutates_args=(), device_types="cuda")
def mxfp8_linear_dw_f32(grad_output: torch.Tensor, x: torch.Tensor, config_key: str) -> torch.Tensor:
    """FP32 dW for the data-parallel all-reduce (no counterpart in the single-GPU reference)."""
    _bwd_config(config_key)
    return _run(grad_output, x, None, False, True, dw_dtype=torch.float32)[1]


@mxfp8_linear_dw_f32.register_fake
def _(grad_output, x, config_key):
    return grad_output.new_empty((grad_output.shape[1], x.shape[1]), dtype=torch.float32)


# --------------------------------------------------------------------------- training op

@custom_op("rtx::mxfp8_linear_train", mutates_args=(), device_types="cuda")
def mxfp8_linear_train(x: torch.Tensor, weight: torch.Tensor, fwd_key: str, bwd_key: str) -> torch.Tensor:
    """Forward of the differentiable op (rtx/fp8_bwd.py:1481-1494); saves BF16 (x, weight)."""
    return torch.ops.rtx.mxfp8_linear_prequant(x, weight, fwd_key)


@mxfp8_linear_train.register_fake
def _(x, weight, fwd_key, bwd_key):
    return x.new_empty((x.shape[0], weight.shape[0]), dtype=torch.bfloat16)


def _train_setup(ctx, inputs, output):
    x, weight, _fwd_key, bwd_key = inputs
    ctx.save_for_backward(x, weight)
    ctx.bwd_key = bwd_key


def _train_backward(ctx, grad_output):
    """rtx/fp8_bwd.py:1577-1593: both grads -> one packed op; one grad -> dx / dw op."""
    x, weight = ctx.saved_tensors
    need_dx, need_dw = ctx.needs_input_grad[0], ctx.needs_input_grad[1]
    grad_output = grad_output.contiguous()
    if need_dx and need_dw:
        dx, dw = torch.ops.rtx.mxfp8_linear_bwd(grad_output, x, weight, ctx.bwd_key)
        return dx, dw, None, None
    if need_dx:
        return torch.ops.rtx.mxfp8_linear_dx(grad_output, x, weight, ctx.bwd_key), None, None, None
    if need_dw:
        return None, torch.ops.rtx.mxfp8_linear_dw(grad_output, x, weight, ctx.bwd_key), None, None
    return None, None, None, None


mxfp8_linear_train.register_autograd(_train_backward, setup_context=_train_setup)


# --------------------------------------------------------------------------- functional

def mxfp8_linear_backward(grad_output: torch.Tensor, x: torch.Tensor, weight: torch.Tensor, *,
                          config: Optional[MXFP8BwdConfig] = None, autotune=None, tuning_policy=None,
                          autotune_cache_dir: "Path | str | None" = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """Compute BF16 dX and dW using independently quantized MXFP8 GEMMs (rtx/fp8_bwd.py:1603-1738).
    Leading dimensions of `x` and `grad_output` are flattened into the token dimension."""
    _fp8._autotune_mode(autotune)
    key = (config or MXFP8BwdConfig()).to_key()
    k = x.shape[-1]
    n = grad_output.shape[-1]
    g2d, x2d = grad_output.reshape(-1, n), x.reshape(-1, k)
    dx, dw = torch.ops.rtx.mxfp8_linear_bwd(g2d, x2d, weight, key)
    return dx.reshape(x.shape), dw


def _clear_runtime_caches() -> dict:
    return {}


DEFAULT_MXFP8_BWD_CONFIG = MXFP8BwdConfig()
DEFAULT_FUSED_MXFP8_BWD_CONFIG = MXFP8BwdConfig()

__all__ = ["mxfp8_linear_backward", "MXFP8BwdConfig", "DEFAULT_MXFP8_BWD_CONFIG", "DEFAULT_FUSED_MXFP8_BWD_CONFIG"]


# Inductor lowerings of the ops above (skipped quietly when Inductor's internals are unavailable)
from . import inductor as _inductor  # noqa: E402

_inductor.register_mxfp8_train_lowering()
_inductor.register_mxfp8_backward_lowerings()
