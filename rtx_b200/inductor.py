"""Inductor lowerings of the forward and backward ops: inside a `torch.compile`d graph the op becomes an extern kernel
that writes into a buffer Inductor owns, called through a launcher bound to the (immutable) config key.

Mirrors the reference's entry points (rtx/fp8.py:207-230 and :683-721 launcher registries and lowerings;
rtx/fp4.py:2037-2604): `register_lowering(op)` returns an `ir.ExternKernelOut` with a fixed BF16 [m, n]
row-major layout whose `python_kernel_name` is an expression that looks the launcher up in a registry
attached to the `torch` module, so wrappers that Inductor re-loads from its disk cache find (and lazily
re-create) their launchers.  Launcher convention: `launcher(*inputs, out=buffer) -> None`.

The backward ops (rtx/fp8_bwd.py:1387-1478) lower the same way: dX-only and dW-only become one extern
kernel each; the two-output op becomes ONE extern kernel that writes `[dX | pad to 8 elements | dW]`
into a flat buffer (the layout of the reference's packed op) followed by two views, so the gradient is
still read once for its two quantizations.

Without the lowering the ops still compile (they carry fake implementations); the lowering removes the
dispatcher round trip and the allocation inside the op from the steady-state path.  Registration is
attempted once at import of the frontends and is skipped quietly if Inductor's internals are not there.
"""

from __future__ import annotations

import threading
from typing import Callable, Dict

import torch

_LOCK = threading.RLock()
CALLS: Dict[str, int] = {}          # launcher family -> calls, for tests and diagnostics


class LauncherRegistry(dict):
    """config key -> launcher, created on first use (also by wrappers loaded from Inductor's cache)."""

    def __init__(self, family: str, factory: Callable[[str], Callable]):
        super().__init__()
        self.family, self.factory = family, factory

    def __missing__(self, key: str):
        with _LOCK:
            launcher = self.get(key)
            if launcher is None:
                launcher = self.factory(key)
                self[key] = launcher
        return launcher


def _count(family: str) -> None:
    CALLS[family] = CALLS.get(family, 0) + 1


def _mxfp8_fwd_launcher(key: str):
    from . import fp8, ops

    cfg = fp8._resolve_prequant(key)
    rounding = fp8._rounding(cfg)

    def launch(x, weight, *, out):
        _count("mxfp8_fwd")
        with ops.schedule_of(cfg.gemm):
            ops.mxfp8_linear_fwd(x, weight, fp8._workspace(x.device), out=out, rounding=rounding)

    return launch


def _nvfp4_region_launcher(key: str):
    from . import fp4, fp8, ops

    cfg = fp4._resolve_dynamic(key)
    mode = fp4._SCALE_MODE[cfg.scale.tensor_scale_mode]

    def launch(x, weight, *, out):
        _count("nvfp4_jit_row_region_fwd")
        with ops.schedule_of(cfg.gemm):
            ops.nvfp4_linear_fwd_regions(x, weight, fp8._workspace(x.device), cfg.x_scale_region_rows,
                                         cfg.weight_scale_region_rows, out=out, scale_mode=mode)

    return launch


def _nvfp4_block_launcher(key: str):
    from . import fp4, ops

    cfg = fp4._resolve_dynamic(key)

    def launch(x, weight, *, out):
        _count("nvfp4_block_fwd")
        qx, sx = ops.nvfp4_quantize(x, None)
        qw, sw = ops.nvfp4_quantize(weight, None)
        with ops.schedule_of(cfg.gemm):
            ops.nvfp4_gemm(qx, sx, qw, sw, int(x.shape[0]), int(weight.shape[0]), int(x.shape[1]), None, out=out)

    return launch


def _nvfp4_materialized_launcher(key: str):
    from . import fp4, ops

    cfg = fp4._resolve_dynamic(key)

    def launch(x, weight, x_scale, weight_scale, output_scale, *, out):
        _count("nvfp4_materialized_fwd")
        qx, sx = ops.nvfp4_quantize(x, x_scale)
        qw, sw = ops.nvfp4_quantize(weight, weight_scale)
        with ops.schedule_of(cfg.gemm):
            ops.nvfp4_gemm(qx, sx, qw, sw, int(x.shape[0]), int(weight.shape[0]), int(x.shape[1]), output_scale,
                           out=out)

    return launch


def _mxfp8_bwd_launcher(spec):
    """spec = (backward config key, "dx" | "dw" | "packed")."""
    from . import fp8, fp8_bwd, ops

    key, kind = spec
    fp8_bwd._bwd_config(key)

    def launch(grad_output, x, weight, *, out):
        _count("mxfp8_bwd")
        ws = fp8._workspace(grad_output.device)
        if kind == "dx":
            ops.mxfp8_linear_bwd(grad_output, None, weight, ws, need_dw=False, dx_out=out)
        elif kind == "dw":
            ops.mxfp8_linear_bwd(grad_output, x, None, ws, need_dx=False, dw_out=out)
        else:
            dx_n = x.numel()
            off = (dx_n + 7) // 8 * 8
            ops.mxfp8_linear_bwd(grad_output, x, weight, ws, dx_out=out[:dx_n].view(x.shape),
                                 dw_out=out[off:off + weight.numel()].view(weight.shape))

    return launch


REGISTRIES = {
    "mxfp8_bwd": LauncherRegistry("mxfp8_bwd", _mxfp8_bwd_launcher),
    "mxfp8_fwd": LauncherRegistry("mxfp8_fwd", _mxfp8_fwd_launcher),
    "nvfp4_jit_row_region_fwd": LauncherRegistry("nvfp4_jit_row_region_fwd", _nvfp4_region_launcher),
    "nvfp4_block_fwd": LauncherRegistry("nvfp4_block_fwd", _nvfp4_block_launcher),
    "nvfp4_materialized_fwd": LauncherRegistry("nvfp4_materialized_fwd", _nvfp4_materialized_launcher),
}


def _inductor():
    try:
        from torch._inductor import ir
        from torch._inductor.lowering import register_lowering
    except Exception:
        return None
    torch._rtx_b200_launchers = REGISTRIES
    return ir, register_lowering


def _extern(ir, family: str, key: str, tensors, m, n):
    inputs = [ir.ExternKernel.require_contiguous(ir.ExternKernel.realize_input(t)) for t in tensors]
    layout = ir.FixedLayout(device=tensors[0].get_device(), dtype=torch.bfloat16, size=[m, n], stride=[n, 1])
    return ir.TensorBox.create(ir.ExternKernelOut(
        layout=layout, inputs=inputs, python_kernel_name=f"torch._rtx_b200_launchers[{family!r}][{key!r}]"))


def _register(group: str, entries) -> bool:
    """entries: (op overload, launcher family, number of leading tensor arguments).  The config key follows
    the tensors; the `*_train` overloads carry a backward key after it, which the forward launcher ignores."""
    with _LOCK:
        if group in _DONE:
            return _DONE[group]
        found = _inductor()
        ok = found is not None
        if ok:
            ir, register_lowering = found
            try:
                for op, family, n_tensors in entries:
                    def lower(*args, _family=family, _n=n_tensors):
                        tensors, key = args[:_n], args[_n]
                        return _extern(ir, _family, key, tensors, tensors[0].get_size()[0], tensors[1].get_size()[0])
                    register_lowering(op, type_promotion_kind=None)(lower)
            except Exception:
                ok = False
        _DONE[group] = ok
        return ok


_DONE: Dict[str, bool] = {}


def register_mxfp8_lowerings() -> bool:
    """Forward ops defined in fp8.py (call after they exist).  False when Inductor is unavailable."""
    ops_ns = torch.ops.rtx
    return _register("mxfp8", [(ops_ns.mxfp8_linear_fwd.default, "mxfp8_fwd", 2),
                               (ops_ns.mxfp8_linear_prequant.default, "mxfp8_fwd", 2)])


def register_mxfp8_train_lowering() -> bool:
    return _register("mxfp8_train", [(torch.ops.rtx.mxfp8_linear_train.default, "mxfp8_fwd", 2)])


def register_mxfp8_backward_lowerings() -> bool:
    """rtx::mxfp8_linear_bwd / _bwd_packed / _dx / _dw (call after fp8_bwd.py defined them)."""
    with _LOCK:
        if "mxfp8_bwd" in _DONE:
            return _DONE["mxfp8_bwd"]
        found = _inductor()
        ok = found is not None
        if ok:
            ir, register_lowering = found
            try:
                from torch._inductor.lowering import lowerings

                aten = torch.ops.aten

                def extern(kind, key, grad_output, x, weight, size):
                    inputs = [ir.ExternKernel.require_contiguous(ir.ExternKernel.realize_input(t))
                              for t in (grad_output, x, weight)]
                    stride = [size[1], 1] if len(size) == 2 else [1]
                    layout = ir.FixedLayout(device=x.get_device(), dtype=torch.bfloat16, size=list(size), stride=stride)
                    return ir.TensorBox.create(ir.ExternKernelOut(
                        layout=layout, inputs=inputs,
                        python_kernel_name=f"torch._rtx_b200_launchers['mxfp8_bwd'][{(key, kind)!r}]"))

                def packed(grad_output, x, weight, key):
                    xs, wsz = x.get_size(), weight.get_size()
                    off = (xs[0] * xs[1] + 7) // 8 * 8
                    return extern("packed", key, grad_output, x, weight, [off + wsz[0] * wsz[1]]), off

                @register_lowering(torch.ops.rtx.mxfp8_linear_bwd_packed.default, type_promotion_kind=None)
                def lower_packed(grad_output, x, weight, key):
                    return packed(grad_output, x, weight, key)[0]

                @register_lowering(torch.ops.rtx.mxfp8_linear_bwd.default, type_promotion_kind=None)
                def lower_both(grad_output, x, weight, key):
                    flat, off = packed(grad_output, x, weight, key)
                    xs, wsz = x.get_size(), weight.get_size()
                    view, cut = lowerings[aten.view.default], lowerings[aten.slice.Tensor]
                    dx = view(cut(flat, 0, 0, xs[0] * xs[1]), list(xs))
                    dw = view(cut(flat, 0, off, off + wsz[0] * wsz[1]), list(wsz))
                    return dx, dw

                @register_lowering(torch.ops.rtx.mxfp8_linear_dx.default, type_promotion_kind=None)
                def lower_dx(grad_output, x, weight, key):
                    return extern("dx", key, grad_output, x, weight, x.get_size())

                @register_lowering(torch.ops.rtx.mxfp8_linear_dw.default, type_promotion_kind=None)
                def lower_dw(grad_output, x, weight, key):
                    return extern("dw", key, grad_output, x, weight, weight.get_size())
            except Exception:
                ok = False
        _DONE["mxfp8_bwd"] = ok
        return ok


def register_nvfp4_lowerings() -> bool:
    ops_ns = torch.ops.rtx
    return _register("nvfp4", [
        (ops_ns.nvfp4_linear_jit_row_region_fwd.default, "nvfp4_jit_row_region_fwd", 2),
        (ops_ns.nvfp4_linear_jit_row_region_train.default, "nvfp4_jit_row_region_fwd", 2),
        (ops_ns.nvfp4_linear_block_fwd.default, "nvfp4_block_fwd", 2),
        (ops_ns.nvfp4_linear_block_train.default, "nvfp4_block_fwd", 2),
        (ops_ns.nvfp4_linear_materialized_fwd.default, "nvfp4_materialized_fwd", 5),
        (ops_ns.nvfp4_linear_materialized_train.default, "nvfp4_materialized_fwd", 5),
    ])
