"""Deterministic synthetic inputs with the shapes and value distributions of the
five benchmark configurations.  Every rank draws the identical global tensors
(seed 0 for configuration 1, seed = configuration number otherwise; never
seeded by rank) and slices its own contiguous block of token rows.
"""

from __future__ import annotations

import math
from typing import Dict

import torch

CONFIG_NAMES = {
    1: "mxfp8_linear_fwd_256x1024x1024",
    2: "mxfp8_glu_mlp_fwd_m8192_k4096_i14336",
    3: "nvfp4_linear_fwd_m16384_n28672_k8192",
    4: "mxfp8_linear_bwd_m16384_n4096_k4096",
    5: "nvfp4_decode_prequant_w_k8192",
}


def _randn(gen, *shape):
    return torch.randn(*shape, generator=gen, dtype=torch.float32)


def make_inputs(config: int, scale: float = 1.0, **dims) -> Dict[str, torch.Tensor]:
    """CPU BF16 tensors for configuration 1..5.  `scale` < 1 shrinks every large
    dimension (kept at multiples of 128) for CPU-sized parity cases; explicit
    keyword dimensions override the defaults."""

    def d(name, default):
        v = dims.get(name, default)
        if name in dims or scale == 1.0:
            return v
        return max(128, int(round(v * scale / 128)) * 128)

    gen = torch.Generator().manual_seed(0 if config == 1 else config)
    if config == 1:
        m, k, n = dims.get("m", 256), dims.get("k", 1024), dims.get("n", 1024)
        x = _randn(gen, m, k)
        w = _randn(gen, n, k) / math.sqrt(k)
        return {"x": x.bfloat16(), "w": w.bfloat16()}
    if config == 2:
        m, k, inter = d("m", 8192), d("k", 4096), d("inter", 14336)
        x = _randn(gen, m, k)
        mask = torch.rand(m, k, generator=gen) < 0.001
        x = torch.where(mask, x * 50.0, x)           # 0.1 % outliers scaled x50
        w_gu = _randn(gen, 2 * inter, k) / math.sqrt(k)   # gate rows first, then up rows
        w_down = _randn(gen, k, inter) / math.sqrt(inter)
        return {"x": x.bfloat16(), "w_gate_up": w_gu.bfloat16(), "w_down": w_down.bfloat16()}
    if config == 3:
        m, k, n = d("m", 16384), d("k", 8192), d("n", 28672)
        z = _randn(gen, m, k)
        chi = sum(_randn(gen, m, k) ** 2 for _ in range(4))
        x = z / torch.sqrt(chi / 4.0)                # Student-t with 4 degrees of freedom
        w = _randn(gen, n, k) / math.sqrt(k)
        return {"x": x.bfloat16(), "w": w.bfloat16()}
    if config == 4:
        m, k, n = d("m", 16384), d("k", 4096), d("n", 4096)
        x = _randn(gen, m, k)
        w = _randn(gen, n, k) / math.sqrt(k)
        dy = _randn(gen, m, n) * 0.1
        return {"x": x.bfloat16(), "w": w.bfloat16(), "dy": dy.bfloat16()}
    if config == 5:
        m, k, n = dims.get("m", 8), d("k", 8192), d("n", 8192)
        w = _randn(gen, n, k) / math.sqrt(k)
        x = _randn(gen, m, k)
        return {"x": x.bfloat16(), "w": w.bfloat16()}
    raise ValueError(f"unknown configuration {config}")


def shard_rows(t: torch.Tensor, rank: int, world: int) -> torch.Tensor:
    """Contiguous row block of the global tensor owned by `rank` (M-sharding)."""
    rows = t.shape[0]
    if rows % world:
        raise ValueError(f"{rows} rows do not split evenly over {world} ranks")
    per = rows // world
    return t[rank * per:(rank + 1) * per].contiguous()
