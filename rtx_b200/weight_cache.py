"""Step-scoped cache of quantized weights.

A BF16 master weight changes once per optimizer step, yet a dynamic `MXFP8Linear` /
`NVFP4Linear` requantizes it in every forward and again (transposed) in every backward
(rtx/fp8.py:292-312 `_PrequantRunner`, rtx/fp8_bwd.py:229-325 `_BwdRunner`).  With several
micro-batches per step, or several calls of a shared module, that work repeats on an
operand that has not changed: 0.35 GB of memory traffic per call for a 28672 x 4096 weight.

    with rtx_b200.quantized_weight_cache():
        for micro_batch in step:                 # gradient accumulation
            model(micro_batch).backward()
    optimizer.step()                             # outside: the next step requantizes

Inside the scope a dynamic module quantizes its weight on first use and reuses the payload
and scales while the parameter is unchanged (same storage, same autograd version counter;
optimizers bump the counter, writes through `.data` do not, which is why the scope ends
before the optimizer runs).  The kernels are the ones the uncached path launches, so
outputs and gradients are bit-identical to it.  Nothing is cached under `torch.compile`
tracing: a compiled graph keeps the uncached ops.
"""

from __future__ import annotations

import threading
from dataclasses import dataclass, field
from typing import Optional

import torch

from . import _native as N
from . import ops

_tls = threading.local()


@dataclass
class _Entry:
    ptr: int
    version: int
    shape: tuple
    parts: dict = field(default_factory=dict)


class quantized_weight_cache:
    """Context manager; scopes nest (an inner scope shares the outer cache).  `stats` counts
    quantizer launches saved (`hits`) and made (`misses`)."""

    def __init__(self):
        self.entries: dict = {}
        self.stats = {"hits": 0, "misses": 0}
        self.alive = False
        self._outer = None

    def __enter__(self):
        self._outer = getattr(_tls, "cache", None)
        if self._outer is None:
            _tls.cache = self
            self.alive = True
        return self._outer or self

    def __exit__(self, *exc):
        if self._outer is None:
            _tls.cache = None
            self.alive = False
            self.entries.clear()
        return False

    # -- lookup ---------------------------------------------------------------------
    def _entry(self, weight: torch.Tensor) -> _Entry:
        # keyed by storage, not object identity: autograd may hand the same parameter over as another
        # Python object.  The entry keeps the tensor alive, so its address cannot be reused under it.
        key = (weight.data_ptr(), tuple(weight.shape), tuple(weight.stride()))
        entry = self.entries.get(key)
        if entry is None or entry.version != weight._version:
            entry = _Entry(key[0], weight._version, key[1])
            entry.keep = weight
            self.entries[key] = entry
        return entry

    def get(self, weight: torch.Tensor, part: str, make):
        entry = self._entry(weight)
        value = entry.parts.get(part)
        if value is None:
            self.stats["misses"] += 1
            value = entry.parts[part] = make()
        else:
            self.stats["hits"] += 1
        return value


def active() -> Optional[quantized_weight_cache]:
    """The cache of the enclosing scope, or None (also None while torch.compile traces)."""
    if torch.compiler.is_compiling():
        return None
    return getattr(_tls, "cache", None)


# ------------------------------------------------------------------------------- MXFP8

def mxfp8_rows(cache, weight: torch.Tensor, rounding: int = N.ROUND_INFINITY):
    """W [N, K] quantized in blocks along K: the forward's B operand."""
    w = weight.detach()
    return cache.get(weight, f"mx_rows_{rounding}",
                     lambda: ops.mxfp8_quantize(w if w.is_contiguous() else w.contiguous(), rounding=rounding))


def mxfp8_transposed(cache, weight: torch.Tensor):
    """W^T [K, N] quantized in blocks along N: dX's B operand."""
    w = weight.detach()
    return cache.get(weight, "mx_transposed",
                     lambda: ops.mxfp8_quantize_transposed(w if w.is_contiguous() else w.contiguous()))


def _cached_backward(ctx, grad_output):
    """dX and dW as the uncached backward computes them (rtx/fp8_bwd.py:530-541), with W^T from the cache.
    Runs on autograd's worker thread, so the scope is checked on the cache object, not the thread."""
    x2d, weight = ctx.saved_tensors
    need_dx, need_dw = ctx.needs_input_grad[0], ctx.needs_input_grad[1]
    dy = grad_output if grad_output.is_contiguous() else grad_output.contiguous()
    m, n = dy.shape
    k = weight.shape[1]
    dx = dw = None
    if need_dx and need_dw:
        q_rows, s_rows, q_t, s_t = ops.mxfp8_quantize_dual(dy)
    elif need_dx:
        q_rows, s_rows = ops.mxfp8_quantize(dy)
    elif need_dw:
        q_t, s_t = ops.mxfp8_quantize_transposed(dy)
    if need_dx:
        # a scope that ended between forward and backward: quantize as the uncached path does
        qwt, swt = (mxfp8_transposed(ctx.cache, weight) if ctx.cache.alive
                    else ops.mxfp8_quantize_transposed(weight.detach().contiguous()))
        dx = ops.mxfp8_gemm(q_rows, s_rows, qwt, swt, int(m), int(k), int(n))
    if need_dw:
        qxt, sxt = ops.mxfp8_quantize_transposed(x2d)
        dw = ops.mxfp8_gemm(q_t, s_t, qxt, sxt, int(n), int(k), int(m))
    return dx, dw


class MXFP8CachedLinearFunction(torch.autograd.Function):
    """`rtx::mxfp8_linear_train` with the weight operands of forward and dX taken from the cache: launch
    for launch the uncached composition minus the weight quantizers."""

    @staticmethod
    def forward(ctx, x2d, weight, cache, rounding):
        n, k = weight.shape
        qw, sw = mxfp8_rows(cache, weight, rounding)
        x2d = x2d if x2d.is_contiguous() else x2d.contiguous()
        qx, sx = ops.mxfp8_quantize(x2d, rounding=rounding)
        ctx.save_for_backward(x2d, weight)
        ctx.cache = cache
        return ops.mxfp8_gemm(qx, sx, qw, sw, int(x2d.shape[0]), int(n), int(k))

    @staticmethod
    def backward(ctx, grad_output):
        return (*_cached_backward(ctx, grad_output), None, None)


def mxfp8_glu_mlp_cached(cache, x2d, w_gate_up, w_down):
    """The fused SwiGLU forward (quantize X, gate/up GEMM whose epilogue emits H as MXFP8, down GEMM) with
    both weights from the cache: two launches instead of five once the cache is warm."""
    inter, k = w_gate_up.shape[0] // 2, w_gate_up.shape[1]
    q_gu, s_gu = mxfp8_rows(cache, w_gate_up)
    q_dn, s_dn = mxfp8_rows(cache, w_down)
    x2d = x2d if x2d.is_contiguous() else x2d.contiguous()
    m = int(x2d.shape[0])
    qx, sx = ops.mxfp8_quantize(x2d)
    qh, sh, _ = ops.mxfp8_gemm_glu_mx(qx, sx, q_gu, s_gu, m, int(inter), int(k))
    return ops.mxfp8_gemm(qh, sh, q_dn, s_dn, m, int(w_down.shape[0]), int(inter))


# ------------------------------------------------------------------------------- NVFP4

def nvfp4_regions(cache, weight: torch.Tensor, region_rows: int, scale_mode: int):
    """W quantized under the row-region policy: (payload, block scales, region scales, effective rows)."""
    def make():
        w = weight.detach()
        w = w if w.is_contiguous() else w.contiguous()
        rows = ops.nvfp4_effective_region_rows(int(w.shape[0]), int(region_rows))
        scales = ops.nvfp4_region_scales(w, rows, scale_mode)
        q, s = ops.nvfp4_quantize_regions(w, scales, rows)
        return q, s, scales, rows

    return cache.get(weight, f"nv_regions_{region_rows}_{scale_mode}", make)


def nvfp4_linear_regions_cached(cache, x2d, weight, x_region_rows: int, w_region_rows: int, scale_mode: int):
    """`jit_row_region` forward with the weight side from the cache."""
    qw, sw, w_scales, w_rows = nvfp4_regions(cache, weight, w_region_rows, scale_mode)
    x2d = x2d if x2d.is_contiguous() else x2d.contiguous()
    m, k = int(x2d.shape[0]), int(x2d.shape[1])
    x_rows = ops.nvfp4_effective_region_rows(m, int(x_region_rows))
    x_scales = ops.nvfp4_region_scales(x2d, x_rows, scale_mode)
    qx, sx = ops.nvfp4_quantize_regions(x2d, x_scales, x_rows)
    return ops.nvfp4_gemm_regions(qx, sx, qw, sw, m, int(weight.shape[0]), k, x_scales, x_rows, w_scales, w_rows)


class NVFP4CachedRegionLinearFunction(torch.autograd.Function):
    """`rtx::nvfp4_linear_jit_row_region_train` with cached weight operands: NVFP4 forward, MXFP8 backward
    (rtx/fp4.py:1772-1794)."""

    @staticmethod
    def forward(ctx, x2d, weight, cache, x_region_rows, w_region_rows, scale_mode):
        x2d = x2d if x2d.is_contiguous() else x2d.contiguous()
        ctx.save_for_backward(x2d, weight)
        ctx.cache = cache
        return nvfp4_linear_regions_cached(cache, x2d, weight, x_region_rows, w_region_rows, scale_mode)

    @staticmethod
    def backward(ctx, grad_output):
        return (*_cached_backward(ctx, grad_output), None, None, None, None)


__all__ = ["quantized_weight_cache", "active"]
