"""Shared metadata of packed low-precision operands (rtx/formats/common.py:11-18).

Layout codes, the schema version stored in `weight_packing_meta`, and the
operand-state names are kept byte for byte so packed checkpoints interchange.
"""

from __future__ import annotations

from math import prod
from typing import Literal

import torch

ScaleLayout = Literal["row_major", "mma64", "mma128"]
Orientation = Literal["row_major", "transpose"]
LinearOperandState = Literal["dynamic", "weight_prequantized", "fully_prequantized"]
PACKED_OPERAND_SCHEMA_VERSION = 3
SCALE_LAYOUT_CODES = {"row_major": 0, "mma64": 1, "mma128": 2}
SCALE_LAYOUT_NAMES = {v: k for k, v in SCALE_LAYOUT_CODES.items()}


def flattened_matrix_shape(shape: tuple[int, ...]) -> tuple[int, int]:
    if not shape:
        raise ValueError("a packed operand must have at least one dimension")
    return (prod(shape[:-1]) if len(shape) > 1 else 1), shape[-1]


def reject_packed_dtype_conversion(args, kwargs, *, format_name: str) -> None:
    """`Module.to(dtype)` on a packed module would cast heterogeneous raw buffers."""
    _device, dtype, _non_blocking, _memory_format = torch._C._nn._parse_to(*args, **kwargs)
    if dtype is not None:
        raise TypeError(
            f"a prequantized {format_name} module cannot be cast to {dtype}; move it with .to(device=...) and "
            "requantize from the BF16 master weight to change numeric formats")


def scale_tile_index(rows: int, blocks: int, chunks: int, device) -> torch.Tensor:
    """Flat byte index of (row, block) inside 128-row scale tiles with `chunks` 512-byte tiles per
    row block: ((row//128)*chunks + block//4)*512 + (row%32)*16 + ((row//32)%4)*4 + block%4
    (rtx/kernels/mxfp8_quant.py:341-354, rtx/kernels/nvfp4_quant.py:299-310)."""
    r = torch.arange(rows, device=device).unsqueeze(1)
    b = torch.arange(blocks, device=device).unsqueeze(0)
    return ((r // 128) * chunks + b // 4) * 512 + (r % 32) * 16 + ((r // 32) % 4) * 4 + b % 4


def scales_row_major_to_mma128(scales: torch.Tensor, rows: int, blocks: int, chunks: int) -> torch.Tensor:
    """Re-tile row-major scale codes [rows, blocks] (any 1-byte dtype) into the tcgen05 layout."""
    src = scales.reshape(rows, blocks).view(torch.uint8)
    out = torch.zeros(((rows + 127) // 128) * chunks * 512, dtype=torch.uint8, device=scales.device)
    out[scale_tile_index(rows, blocks, chunks, scales.device).reshape(-1)] = src.reshape(-1)
    return out


def scales_mma128_to_row_major(tiles: torch.Tensor, rows: int, blocks: int, chunks: int) -> torch.Tensor:
    flat = tiles.reshape(-1).view(torch.uint8)
    return flat[scale_tile_index(rows, blocks, chunks, tiles.device).reshape(-1)].reshape(rows, blocks)
