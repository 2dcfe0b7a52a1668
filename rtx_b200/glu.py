"""SwiGLU MLP forward with the activation fused into the gate/up GEMM epilogue.

The reference computes `F.silu(gate) * up` with PyTorch on the BF16 output of one
fused gate_up linear (rtx/models/decoder.py:349-384).  Here the gate/up GEMM keeps
gate and up of the same output columns in one accumulator tile, applies
`silu(g) * u` to the FP32 accumulators and rounds once to BF16, which removes a
470 MB write and read at the benchmark shape.  Forward only (inference and
activation-recompute use); training modules use `MXFP8Linear` for both projections.
"""

from __future__ import annotations

import torch
from torch import nn

from ._oplib import custom_op
from . import fp8 as _fp8
from . import ops
from . import weight_cache as _weight_cache


@custom_op("rtx::mxfp8_glu_mlp_fwd", mutates_args=(), device_types="cuda")
def mxfp8_glu_mlp_fwd(x: torch.Tensor, w_gate_up: torch.Tensor, w_down: torch.Tensor) -> torch.Tensor:
    """x [M, K], w_gate_up [2*I, K] (gate rows first, I a multiple of 128), w_down [N, I] -> y [M, N]:
    three quantizer launches, the gate/up GEMM whose epilogue emits H = silu(g) * u already MXFP8-encoded,
    the down GEMM.  Forward only (no sm_120 counterpart: the reference applies SiLU * up in PyTorch,
    rtx/models/decoder.py:382-384)."""
    _fp8._check_inputs(x, w_gate_up)
    inter = w_gate_up.shape[0] // 2
    if w_gate_up.shape[0] != 2 * inter or inter % 128 or w_down.shape[1] != inter:
        raise ValueError("w_gate_up must be [2*I, K] with I a multiple of 128, w_down [N, I]")
    _, y = ops.mxfp8_glu_mlp_fwd(x if x.is_contiguous() else x.contiguous(), w_gate_up.contiguous(),
                                 w_down.contiguous(), _fp8._workspace(x.device), want_hidden=False)
    return y


@mxfp8_glu_mlp_fwd.register_fake
def _(x, w_gate_up, w_down):
    return x.new_empty((x.shape[0], w_down.shape[0]), dtype=torch.bfloat16)


class SwiGLU(nn.Module):
    """SwiGLU feed-forward block with a fused gate/up projection, the caller of the hot path in the
    reference's decoder (rtx/models/decoder.py:349-384: `gate_up_proj` [2*I, H], `down_proj` [H, I], both
    no-bias low-precision linears; forward `down(silu(gate) * up)`).  Parameter names and shapes match, so
    checkpoints interchange.  `linear` picks the projection modules: "mxfp8", "nvfp4" or "bf16".

    With MXFP8 projections and no gradient required the forward is the fused pipeline above (the BF16
    gate/up output and the BF16 H never reach memory); training, NVFP4 and BF16 run the two projections
    as modules with SiLU * up between them, as the reference does."""

    def __init__(self, hidden_size: int, intermediate_size: int, *, linear: str = "mxfp8", device=None, **linear_kwargs):
        super().__init__()
        if linear not in ("mxfp8", "nvfp4", "bf16"):
            raise ValueError("linear must be mxfp8, nvfp4 or bf16")
        self.hidden_size, self.intermediate_size, self.linear = int(hidden_size), int(intermediate_size), linear
        if linear == "mxfp8":
            make = lambda i, o: _fp8.MXFP8Linear(i, o, device=device, **linear_kwargs)
        elif linear == "nvfp4":
            from .fp4 import NVFP4Linear
            make = lambda i, o: NVFP4Linear(i, o, device=device, **linear_kwargs)
        else:
            make = lambda i, o: nn.Linear(i, o, bias=False, device=device, dtype=torch.bfloat16)
        self.gate_up_proj = make(self.hidden_size, 2 * self.intermediate_size)
        self.down_proj = make(self.intermediate_size, self.hidden_size)

    def _fused_ok(self, x: torch.Tensor) -> bool:
        if self.linear != "mxfp8" or self.intermediate_size % 128:
            return False
        if getattr(self.gate_up_proj, "weight_mode", "") != "dynamic" or self.down_proj.weight_mode != "dynamic":
            return False
        needs_grad = torch.is_grad_enabled() and (x.requires_grad or self.gate_up_proj.weight.requires_grad
                                                  or self.down_proj.weight.requires_grad)
        return not needs_grad

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if self._fused_ok(x):
            cache = _weight_cache.active()
            if cache is not None:
                x2d = x.reshape(-1, self.hidden_size)
                _fp8._check_inputs(x2d, self.gate_up_proj.weight)
                y = _weight_cache.mxfp8_glu_mlp_cached(cache, x2d, self.gate_up_proj.weight, self.down_proj.weight)
                return y.reshape(*x.shape[:-1], self.hidden_size)
            y = torch.ops.rtx.mxfp8_glu_mlp_fwd(x.reshape(-1, self.hidden_size), self.gate_up_proj.weight,
                                                self.down_proj.weight)
            return y.reshape(*x.shape[:-1], self.hidden_size)
        gate, up = self.gate_up_proj(x).chunk(2, dim=-1)
        return self.down_proj(torch.nn.functional.silu(gate) * up)


def mxfp8_glu_mlp(x: torch.Tensor, w_gate_up: torch.Tensor, w_down: torch.Tensor, *, return_hidden: bool = False):
    """x [..., K] bf16, w_gate_up [2*I, K] (gate rows first), w_down [N, I] -> y [..., N] bf16."""
    k = x.shape[-1]
    x2d = x.reshape(-1, k)
    _fp8._check_inputs(x2d, w_gate_up)
    inter = w_gate_up.shape[0] // 2
    if w_gate_up.shape[0] != 2 * inter or w_down.shape[1] != inter:
        raise ValueError("w_gate_up must be [2*I, K] and w_down [N, I]")
    x2d = x2d if x2d.is_contiguous() else x2d.contiguous()
    if inter % 128 == 0:
        h, y = ops.mxfp8_glu_mlp_fwd(x2d, w_gate_up.contiguous(), w_down.contiguous(), _fp8._workspace(x.device))
    else:
        # the fused epilogue pairs 128-column gate/up blocks; other widths take the unfused composition
        ws = _fp8._workspace(x.device)
        y_gu = ops.mxfp8_linear_fwd(x2d, w_gate_up.contiguous(), ws)
        gate, up = y_gu.chunk(2, dim=-1)
        h = torch.nn.functional.silu(gate) * up
        y = ops.mxfp8_linear_fwd(h.contiguous(), w_down.contiguous(), ws)
    y = y.reshape(*x.shape[:-1], w_down.shape[0])
    return (y, h.reshape(*x.shape[:-1], inter)) if return_hidden else y
