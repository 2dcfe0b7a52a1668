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


_CHUNK_ROWS = 4096


def _rows(gen, m, k, keep, draw):
    """The FP32 [m, k] matrix `draw(gen, m, k)` would give, produced in chunks of rows so that only the rows
    in keep = (lo, hi) are held (all of them for keep = None).  The generator advances exactly as for the whole
    matrix (a chunk is a whole multiple of the generator's vector width), so a rank that keeps only its own block
    of a large global tensor gets the values a rank that drew everything and sliced would get."""
    lo, hi = keep if keep is not None else (0, m)
    parts = []
    for r0 in range(0, m, _CHUNK_ROWS):
        r1 = min(r0 + _CHUNK_ROWS, m)
        t = draw(gen, r1 - r0, k)
        a, b = max(lo, r0), min(hi, r1)
        if a < b:
            parts.append(t[a - r0:b - r0].clone() if (a, b) != (r0, r1) else t)
    return torch.cat(parts) if parts else torch.empty(0, k)


def make_inputs(config: int, scale: float = 1.0, rows=None, **dims) -> Dict[str, torch.Tensor]:
    """CPU BF16 tensors for configuration 1..5.  `scale` < 1 shrinks every large
    dimension (kept at multiples of 128) for CPU-sized parity cases; explicit
    keyword dimensions override the defaults.  `rows = (lo, hi)` (configurations 2 and 4) keeps only
    that block of the token rows of X / dY — the values are those of the full draw — so that a rank
    of a weak-scaling run never holds the other ranks' rows."""

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
        if rows is None:
            x = _randn(gen, m, k)
            mask = torch.rand(m, k, generator=gen) < 0.001
        else:
            # the same draws (all of X, then all of the mask), only the kept block held
            x = _rows(gen, m, k, rows, _randn)
            mask = _rows(gen, m, k, rows, lambda g, r, c: torch.rand(r, c, generator=g)) < 0.001
        x = torch.where(mask, x * 50.0, x).bfloat16()           # 0.1 % outliers scaled x50
        w_gu = _randn(gen, 2 * inter, k) / math.sqrt(k)   # gate rows first, then up rows
        w_down = _randn(gen, k, inter) / math.sqrt(inter)
        return {"x": x, "w_gate_up": w_gu.bfloat16(), "w_down": w_down.bfloat16()}
    if config == 3:
        m, k, n = d("m", 16384), d("k", 8192), d("n", 28672)
        z = _randn(gen, m, k)
        chi = sum(_randn(gen, m, k) ** 2 for _ in range(4))
        x = z / torch.sqrt(chi / 4.0)                # Student-t with 4 degrees of freedom
        w = _randn(gen, n, k) / math.sqrt(k)
        return {"x": x.bfloat16(), "w": w.bfloat16()}
    if config == 4:
        m, k, n = d("m", 16384), d("k", 4096), d("n", 4096)
        x = _randn(gen, m, k) if rows is None else _rows(gen, m, k, rows, _randn)
        w = _randn(gen, n, k) / math.sqrt(k)
        dy = (_randn(gen, m, n) if rows is None else _rows(gen, m, n, rows, _randn)) * 0.1
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
