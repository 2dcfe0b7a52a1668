"""Data parallelism over token rows (M-sharding) for the linear path.

Token rows of X, dY, Y and dX are split contiguously over ranks; weights (and
their quantized copies) are replicated.  Forward and dX need no collective.
dW is a sum over token rows, so each rank computes its partial
`dW_r = dY_r^T X_r` in FP32 and one all-reduce(sum) over NCCL (NVLink/NVSwitch)
combines them before the single BF16 rounding.  MX blocks of the dW operands run
along M, so shards must hold a multiple of 32 rows: block membership — and hence
every quantized payload — is then identical to the single-GPU computation, and
only the FP32 summation order differs.

The reference is single-GPU and only states DDP compatibility
(docs/runtime_contract.md:59-64); this module is the sm_100a path's addition.
"""

from __future__ import annotations

import os
from typing import Optional, Tuple

import torch
import torch.distributed as dist

MX_BLOCK = 32


def shard_bounds(rows: int, rank: int, world: int) -> Tuple[int, int]:
    """Contiguous row block of `rank`; every shard is a multiple of 32 rows."""
    if rows % (world * MX_BLOCK):
        raise ValueError(f"{rows} token rows cannot be split into {world} shards of whole 32-row MX blocks")
    per = rows // world
    return rank * per, (rank + 1) * per


def shard_rows(t: torch.Tensor, rank: int, world: int) -> torch.Tensor:
    lo, hi = shard_bounds(t.shape[0], rank, world)
    return t[lo:hi].contiguous()


def all_reduce_dw(dw_partial_f32: torch.Tensor, group: Optional[dist.ProcessGroup] = None,
                  async_op: bool = False):
    """Sum FP32 partial dW over ranks in place.  With `async_op` the work handle is returned so the
    caller can overlap the collective with the dX GEMM."""
    if dw_partial_f32.dtype is not torch.float32:
        raise TypeError("partial dW must be FP32 so that ranks are summed before the BF16 rounding")
    if not dist.is_initialized() or dist.get_world_size(group) == 1:
        return None
    return dist.all_reduce(dw_partial_f32, op=dist.ReduceOp.SUM, group=group, async_op=async_op)


# SMs the kernels of the backward leave to the NCCL all-reduce that runs beside them, and the number of
# CTAs NCCL is asked to stay within (`nccl_options`).  The GEMMs are persistent and otherwise hold every
# SM until they finish, which pushes the collective behind them; a collective whose CTAs only partly
# fit finishes no earlier than one that does not fit at all (its last channels still wait for the GEMM).
# 20 SMs is what a band of dW leaves free anyway: 64 pair tiles of 256 x 256 on 128 of the 148 SMs.
OVERLAP_SM_MARGIN = int(os.environ.get("RTXB_OVERLAP_SM_MARGIN", "20"))
NCCL_MAX_CTAS = int(os.environ.get("RTXB_NCCL_MAX_CTAS", "16"))
# dW is produced and reduced in bands of rows (multiples of 256, the pair-tile height): the all-reduce of
# a band starts as soon as the GEMM has written it and runs beside the next band's GEMM, the remaining
# quantizer and dX.  0 = as many rows as give one wave of pair tiles on the SMs left to the GEMM.
DW_BAND_ROWS = int(os.environ.get("RTXB_DW_BAND_ROWS", "0"))


def nccl_options(max_ctas: Optional[int] = None):
    """`pg_options` for `dist.init_process_group("nccl", ...)` that keep NCCL's kernels within
    `max_ctas` CTAs, so that they fit the SMs the backward leaves free (OVERLAP_SM_MARGIN)."""
    opts = dist.ProcessGroupNCCL.Options()
    opts.config.max_ctas = int(max_ctas if max_ctas is not None else NCCL_MAX_CTAS)
    opts.config.min_ctas = min(opts.config.max_ctas, 4)
    return opts


def dw_bands(n: int, k: int, band_rows: int = 0, sms: int = 148, margin: Optional[int] = None):
    """Row bands [lo, hi) of the [n, k] dW: multiples of 256 rows (last band: the rest).  With
    band_rows == 0 a band is one wave: as many 256-row tile rows as fit the CTA pairs left to the GEMM."""
    margin = OVERLAP_SM_MARGIN if margin is None else margin
    if band_rows <= 0:
        pairs = max((sms - margin) // 2, 1)
        col_tiles = (k + 255) // 256
        band_rows = 256 * max(pairs // col_tiles, 1)
    band = max(256, band_rows // 256 * 256)
    return [(lo, min(lo + band, n)) for lo in range(0, n, band)]


def _banded_backward(grad_output: torch.Tensor, x: torch.Tensor, weight: torch.Tensor, group):
    """sm_100a path with more than one rank: dY is quantized once for both products, dW leaves the GEMM
    band by band in FP32 and every band's all-reduce is enqueued right behind its GEMM."""
    from . import _native as N
    from . import ops

    m, n = grad_output.shape
    k = x.shape[1]
    q_dy, s_dy, q_dyt, s_dyt = ops.mxfp8_quantize_dual(grad_output)     # dY rows (for dX) and dY^T (for dW)
    q_xt, s_xt = ops.mxfp8_quantize_transposed(x)                       # X^T [K, M], blocks along M
    dw = torch.empty(n, k, dtype=torch.float32, device=x.device)
    chunks = ops.mxfp8_scale_numel(128, m, N.SCALE_MMA128)              # scale bytes of one 128-row block of dY^T
    handles = []
    with ops.sm_margin(OVERLAP_SM_MARGIN):
        for lo, hi in dw_bands(n, k, DW_BAND_ROWS):
            ops.mxfp8_gemm(q_dyt[lo:hi], s_dyt[(lo // 128) * chunks:], q_xt, s_xt, hi - lo, k, m, out=dw[lo:hi])
            handles.append(all_reduce_dw(dw[lo:hi], group, async_op=True))
        q_wt, s_wt = ops.mxfp8_quantize_transposed(weight)              # W^T [K, N], blocks along N
        dx = ops.mxfp8_gemm(q_dy, s_dy, q_wt, s_wt, m, k, n)
    for h in handles:
        if h is not None:
            h.wait()
    return dx, dw


def data_parallel_linear_backward(grad_output: torch.Tensor, x: torch.Tensor, weight: torch.Tensor, *,
                                  group: Optional[dist.ProcessGroup] = None, compute=None):
    """dX (local rows, BF16) and dW (summed over ranks, BF16) for this rank's row shard.

    `compute(grad_output, x, weight) -> (dx_bf16, dw_f32)` defaults to the sm_100a MXFP8 backward;
    tests pass a CPU stand-in to exercise the sharding and the collective with gloo.  With one rank
    (or no process group) the sm_100a path is the plain backward: one call, dW rounded to BF16 in the
    GEMM epilogue.
    """
    if grad_output.shape[0] % MX_BLOCK:
        raise ValueError("a rank's token-row shard must be a multiple of 32 rows")
    alone = not dist.is_initialized() or dist.get_world_size(group) == 1
    if compute is not None:
        dx, dw = compute(grad_output, x, weight)
        handle = all_reduce_dw(dw, group, async_op=True)
        if handle is not None:
            handle.wait()
        return dx, dw.to(torch.bfloat16)
    from . import fp8 as _fp8
    from . import ops

    if alone:
        return ops.mxfp8_linear_bwd(grad_output, x, weight, _fp8._workspace(grad_output.device))
    dx, dw = _banded_backward(grad_output, x, weight, group)
    return dx, dw.to(torch.bfloat16)
