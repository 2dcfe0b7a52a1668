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


# SMs the dX kernels leave to the NCCL all-reduce that runs beside them.  The GEMMs are persistent and
# otherwise hold every SM until they finish, which pushes the collective behind them.  Measured on two
# B200s (67 MB FP32 dW): margins up to 24 change nothing (the collective's CTAs still do not fit), 32
# takes the step from 0.69 to 0.62 ms, larger margins only slow the GEMM.
OVERLAP_SM_MARGIN = int(os.environ.get("RTXB_OVERLAP_SM_MARGIN", "32"))


def data_parallel_linear_backward(grad_output: torch.Tensor, x: torch.Tensor, weight: torch.Tensor, *,
                                  group: Optional[dist.ProcessGroup] = None, compute=None):
    """dX (local rows, BF16) and dW (summed over ranks, BF16) for this rank's row shard.

    `compute(grad_output, x, weight) -> (dx_bf16, dw_f32)` defaults to the sm_100a MXFP8 backward;
    tests pass a CPU stand-in to exercise the sharding and the collective with gloo.
    dW is launched first and its all-reduce runs while dX is computed (on OVERLAP_SM_MARGIN fewer SMs).
    """
    if grad_output.shape[0] % MX_BLOCK:
        raise ValueError("a rank's token-row shard must be a multiple of 32 rows")
    if compute is None:
        from . import fp8 as _fp8
        from . import ops

        ws = _fp8._workspace(grad_output.device)
        _, dw = ops.mxfp8_linear_bwd(grad_output, x, None, ws, need_dx=False, dw_dtype=torch.float32)
        handle = all_reduce_dw(dw, group, async_op=True)
        with ops.sm_margin(OVERLAP_SM_MARGIN if handle is not None else 0):
            dx, _ = ops.mxfp8_linear_bwd(grad_output, None, weight, ws, need_dw=False)
    else:
        dx, dw = compute(grad_output, x, weight)
        handle = all_reduce_dw(dw, group, async_op=True)
    if handle is not None:
        handle.wait()
    return dx, dw.to(torch.bfloat16)
