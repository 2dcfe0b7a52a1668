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

from . import fp8 as _fp8
from . import ops


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
