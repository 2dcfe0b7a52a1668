"""The reference's CPU path, timed as the CPU baseline.  TEST / BENCH INFRASTRUCTURE ONLY.

"TorchAO-style encode + FP32 dequantized matmul": the formulation of
rtx/autotune/legacy.py:783-806 (`_torch_mxfp8_reference`) — amax, integer E8M0
rule, divide, clamp, cast to float8_e4m3fn, dequantize, FP32 matmul, one BF16
rounding — written with whole-tensor torch CPU ops so that it uses every host
thread torch is given.  tests/test_oracle_pins.py checks it bit for bit
against mx_oracle.py (which is pinned to the reference's vectors).

Only bench.py's `cpu_baseline` leg and `--impl reference` arm call this.
"""

from __future__ import annotations

import torch


def mx_quantize(value: torch.Tensor):
    shape = value.shape
    k = shape[-1]
    kp = (k + 31) // 32 * 32
    if kp != k:
        value = torch.nn.functional.pad(value, (0, kp - k))
    blocks = value.reshape(*shape[:-1], kp // 32, 32)
    amax = blocks.abs().amax(dim=-1, keepdim=True).float()
    amax_bits = amax.view(torch.int32)
    exponent = ((amax_bits >> 23) & 0xFF) - 127 - 8
    exponent += (amax_bits & 0x7FFFFF) > 0x600000
    scale_code = (exponent.clamp(-127, 128) + 127).to(torch.uint8)
    scale_code = torch.where(torch.isnan(amax), torch.full_like(scale_code, 255), scale_code)
    scale = (scale_code.int() << 23).view(torch.float32).clamp_min(2 ** -126)
    quantized = (blocks.float() / scale).clamp(-448, 448)
    return quantized.to(torch.float8_e4m3fn).reshape(*shape[:-1], kp), scale_code.squeeze(-1)


def mx_dequantize(q: torch.Tensor, scale_code: torch.Tensor) -> torch.Tensor:
    scale = (scale_code.int() << 23).view(torch.float32).clamp_min(2 ** -126)
    return q.float() * scale.repeat_interleave(32, dim=-1)


def mx_linear_f32(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    qx, sx = mx_quantize(x)
    qw, sw = mx_quantize(w)
    return mx_dequantize(qx, sx) @ mx_dequantize(qw, sw).t()


def mx_linear(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    return mx_linear_f32(x, w).bfloat16()


def mx_glu_mlp(x, w_gate_up, w_down):
    """SwiGLU MLP of rtx/models/decoder.py:382-384 on the MXFP8 linear above; the
    activation is applied to the FP32 accumulators and rounded once (the fused
    epilogue's contract)."""
    inter = w_gate_up.shape[0] // 2
    acc = mx_linear_f32(x, w_gate_up)
    g, u = acc[:, :inter], acc[:, inter:]
    h = (g / (1.0 + torch.exp(-g)) * u).bfloat16()
    return h, mx_linear(h, w_down)


def mlp_flops(m: int, k: int, inter: int, n_out: int) -> float:
    return 2.0 * m * (2 * inter) * k + 2.0 * m * n_out * inter
