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


# NCCL route (used where the peer-memory route below cannot be): SMs the persistent kernels leave to the
# NCCL all-reduce that runs beside dX, and the number of CTAs NCCL is asked to stay within (`nccl_options`).
# The GEMMs otherwise hold every SM until they finish, which pushes the collective behind them; a collective
# whose CTAs only partly fit finishes no earlier than one that does not fit at all.  Measured (67 MB FP32 dW,
# 16384 rows per GPU): 32 SMs / 32 CTAs gives 0.627 ms on two GPUs and 0.634 ms on four; 16 CTAs are enough
# on two GPUs (0.632 ms with bands) but not on four (0.907 ms).
OVERLAP_SM_MARGIN = 32
NCCL_MAX_CTAS = 32
# SMs left free on the peer-memory route for its small kernels (flag barriers, the owner's sum)
PEER_ROUTE_SM_MARGIN = 4
# NCCL route: dW may be produced and reduced in bands of rows (multiples of 256), each band's all-reduce
# enqueued right behind its GEMM.  0 = one band (the whole dW): bands pay only when the collective fits in
# the SMs a band's GEMM leaves free anyway.
DW_BAND_ROWS = 0


def nccl_options(max_ctas: Optional[int] = None):
    """`pg_options` for `dist.init_process_group("nccl", ...)` that keep NCCL's kernels within
    `max_ctas` CTAs, so that they fit the SMs the backward leaves free (OVERLAP_SM_MARGIN)."""
    opts = dist.ProcessGroupNCCL.Options()
    opts.config.max_ctas = int(max_ctas if max_ctas is not None else NCCL_MAX_CTAS)
    opts.config.min_ctas = min(opts.config.max_ctas, 4)
    return opts


def dw_bands(n: int, k: int, band_rows: int = 0, sms: int = 148, margin: Optional[int] = None):
    """Row bands [lo, hi) of the [n, k] dW: multiples of 256 rows (last band: the rest).  band_rows == 0:
    one band; band_rows < 0: a band is one wave, as many 256-row tile rows as fit the CTA pairs left to the GEMM."""
    margin = OVERLAP_SM_MARGIN if margin is None else margin
    if band_rows < 0:
        pairs = max((sms - margin) // 2, 1)
        col_tiles = (k + 255) // 256
        band_rows = 256 * max(pairs // col_tiles, 1)
    elif band_rows == 0:
        band_rows = max(n, 256)
    band = max(256, (band_rows + 255) // 256 * 256)
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


# ---------------------------------------------------------------------------------------------------------
# dW reduce-scatter through peer memory
# ---------------------------------------------------------------------------------------------------------
# Every rank owns a contiguous block of N / world rows of dW.  A rank's dW GEMM for block o writes its FP32
# partial straight into slot [rank] of owner o's staging buffer: the GEMM epilogue's TMA stores go over NVLink,
# so the "reduce-scatter" traffic IS the GEMM's output traffic and overlaps the MMAs tile by tile (no NCCL
# kernel, no SMs taken from the GEMM).  Once every rank's GEMMs are done (a flag barrier through peer memory,
# rtxb_peer_barrier) the owner sums its `world` slots in rank order, rounds once to BF16
# (rtxb_sum_parts_f32_to_bf16) into a buffer its peers can read, and after a second barrier every rank copies
# the other owners' BF16 blocks into its dW with plain device copies: 2 bytes per element cross NVLink in the
# second phase instead of 4, beside the dX GEMM, and no collective kernel competes with the GEMM for SMs
# (an NCCL all-gather kept within 16 CTAs ran at about 100 GB/s on four GPUs and was the slowest link).
# Peer buffers come from torch.distributed's symmetric memory (plain peer mappings; NVLink multicast is not
# bound).  Shapes whose rows do not split into whole 256-row tiles per rank, and processes where symmetric
# memory is not available, take the banded NCCL all-reduce above.

P2P_REDUCE_SCATTER = True     # module attribute: set False to force the NCCL route
_P2P_STATES: dict = {}


class _PeerReduceScatter:
    """Staging slots of one (device, N, K, group): `slots[s]` on this rank receives rank s's partial of
    the block this rank owns; `peer_slot[o]` is this rank's slot in owner o's buffer."""

    def __init__(self, n: int, k: int, device: torch.device, group):
        import torch.distributed._symmetric_memory as symm

        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        self.group = group if group is not None else dist.group.WORLD
        self.world, self.rank = dist.get_world_size(self.group), dist.get_rank(self.group)
        self.rows = n // self.world
        self.n, self.k = n, k
        block = self.rows * k
        self.stage = symm.empty(self.world * block, dtype=torch.float32, device=device)
        self.handle = symm.rendezvous(self.stage, self.group)
        self.slots = self.stage.view(self.world, self.rows, k)
        self.peer_slot = [self.handle.get_buffer(o, (self.rows, k), torch.float32, self.rank * block)
                          for o in range(self.world)]
        # reduced BF16 blocks, pulled by every rank: `result[o]` here is the block this rank would own as rank o;
        # only `result[rank]` is ever written (by this rank) and read (by everyone)
        self.result = symm.empty(n * k, dtype=torch.bfloat16, device=device)
        self.result_handle = symm.rendezvous(self.result, self.group)
        self.my_result = self.result.view(self.world, self.rows, k)[self.rank]
        self.peer_result = [self.result_handle.get_buffer(o, (self.rows, k), torch.bfloat16, o * block)
                            for o in range(self.world)]
        # flag words for the node barrier kernel (rtxb_peer_barrier): eight int32 per rank, zero before first use
        self.flags = symm.empty(8, dtype=torch.int32, device=device)
        self.flags.zero_()
        self.flags_handle = symm.rendezvous(self.flags, self.group)
        self.flag_views = [self.flags_handle.get_buffer(o, (8,), torch.int32, 0) for o in range(self.world)]
        self.flag_ptrs = [v.data_ptr() for v in self.flag_views]
        self.epoch_counter = torch.zeros(1, dtype=torch.int32, device=device)   # advanced by the barrier kernel
        torch.cuda.synchronize(device)
        dist.barrier(group=self.group, device_ids=[device.index])   # every rank's flags are zero before anyone signals
        self.comm = torch.cuda.Stream(device)
        # the reduced blocks come from world - 1 different peers: a few streams let those copies run at once
        self.fan = [torch.cuda.Stream(device) for _ in range(max(0, min(3, self.world - 2)))]


def _node_barrier(st: "_PeerReduceScatter") -> None:
    """Orders the ranks on the current stream with the flag kernel (a few microseconds) instead of a one-word
    NCCL all-reduce (20-40 us on the stream); a rank that never arrives shows up in the status word."""
    from . import ops

    ops.peer_barrier(st.flag_ptrs, st.rank, st.epoch_counter)


def p2p_block_rows(n: int, world: int) -> int:
    """Rows of dW each rank owns for the peer-memory reduce-scatter, or 0 when N does not split into
    whole 256-row tiles per rank (or over more than the eight blocks one GEMM launch addresses)."""
    return n // world if 1 < world <= 8 and n % (256 * world) == 0 else 0


def _peer_state(n: int, k: int, device: torch.device, group):
    key = (device.index, n, k, id(group))
    state = _P2P_STATES.get(key)
    if state is None:
        try:
            state = _PeerReduceScatter(n, k, device, group)
        except Exception as exc:   # symmetric memory unavailable here: remember and use NCCL
            state = exc
        # the route is a collective decision: if the set-up failed on any rank, every rank takes the NCCL route
        ok = torch.tensor([0.0 if isinstance(state, Exception) else 1.0], device=device)
        dist.all_reduce(ok, op=dist.ReduceOp.MIN, group=group)
        if float(ok.item()) == 0.0 and not isinstance(state, Exception):
            state = RuntimeError("peer-memory set-up failed on another rank")
        _P2P_STATES[key] = state
    return None if isinstance(state, Exception) else state


def _peer_backward(grad_output: torch.Tensor, x: torch.Tensor, weight: torch.Tensor, st: "_PeerReduceScatter",
                   marks: Optional[dict] = None):
    """`marks`: a dict that receives one timing event per phase, recorded on the stream the phase runs on
    (`python bench_configs.py --config 8` prints them); None on the product path."""
    from . import _native as N
    from . import ops

    def mark(name, stream):
        if marks is not None:
            marks[name] = torch.cuda.Event(enable_timing=True)
            marks[name].record(stream)

    m, n = grad_output.shape
    k = x.shape[1]
    main = torch.cuda.current_stream(x.device)
    mark("start", main)
    q_dy, s_dy, q_dyt, s_dyt = ops.mxfp8_quantize_dual(grad_output)
    q_xt, s_xt = ops.mxfp8_quantize_transposed(x)
    mark("quantized_dy_and_xt", main)
    rows, world, rank = st.rows, st.world, st.rank
    # ONE dW GEMM over all rows: every 256-row tile goes to the slot of the rank that owns its block, the tile
    # order starting at this rank's neighbour.  Output traffic of a wave of tiles overlaps the next wave's MMAs.
    ops.mxfp8_gemm_row_blocks(q_dyt, s_dyt, q_xt, s_xt, n, k, m, st.peer_slot, first_block=(rank + 1) % world)
    mark("dw_gemm", main)
    done = torch.cuda.Event()
    done.record(main)
    dw = torch.empty(n, k, dtype=torch.bfloat16, device=x.device)
    st.comm.wait_event(done)
    with torch.cuda.stream(st.comm):
        _node_barrier(st)                                     # every rank's partials have landed everywhere
        mark("barrier_partials_landed", st.comm)
        ops.sum_parts_f32_to_bf16(st.slots, st.my_result)
        mark("owner_sum", st.comm)
        _node_barrier(st)                                     # every owner's block is reduced
        mark("barrier_blocks_reduced", st.comm)
        reduced = torch.cuda.Event()
        reduced.record(st.comm)
        lanes = [st.comm] + st.fan
        for s in st.fan:
            s.wait_event(reduced)
        for i in range(world):
            o = (rank + i) % world
            with torch.cuda.stream(lanes[i % len(lanes)]):
                dw[o * rows:(o + 1) * rows].copy_(st.peer_result[o], non_blocking=True)   # plain copies over NVLink
        for s in st.fan:
            st.comm.wait_stream(s)
        mark("blocks_copied", st.comm)
    with ops.sm_margin(PEER_ROUTE_SM_MARGIN):
        q_wt, s_wt = ops.mxfp8_quantize_transposed(weight)
        mark("quantized_wt", main)
        dx = ops.mxfp8_gemm(q_dy, s_dy, q_wt, s_wt, m, k, n)
        mark("dx_gemm", main)
    # dw was allocated on the main stream and is written on the comm and fan streams; the main stream waits for
    # all of them here, before anything later on it, so the allocator may hand the block out again (on the main
    # stream) as soon as the caller drops it.  No record_stream: that would park every step's block until the
    # side streams' events are polled and make a host that runs ahead allocate fresh memory step after step.
    main.wait_stream(st.comm)
    mark("end", main)
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
    n, k = grad_output.shape[1], x.shape[1]
    if P2P_REDUCE_SCATTER and p2p_block_rows(n, dist.get_world_size(group)):
        state = _peer_state(n, k, grad_output.device, group)
        if state is not None:
            return _peer_backward(grad_output, x, weight, state)
    dx, dw = _banded_backward(grad_output, x, weight, group)
    return dx, dw.to(torch.bfloat16)


def backward_collective(n: int, k: int, device: torch.device, group=None) -> str:
    """Which route `data_parallel_linear_backward` takes for an [n, k] dW on this process (for reports)."""
    if not dist.is_initialized() or dist.get_world_size(group) == 1:
        return "none (one rank)"
    if P2P_REDUCE_SCATTER and p2p_block_rows(n, dist.get_world_size(group)) and _peer_state(n, k, device, group):
        return ("reduce-scatter in the dW GEMM epilogue (FP32 TMA stores into the owner's slots over NVLink), "
                "owner sums and rounds once, peers copy the BF16 blocks beside dX; ranks ordered by two flag barriers through "
                "peer memory (no NCCL kernel in the step)")
    why = ""
    if P2P_REDUCE_SCATTER and p2p_block_rows(n, dist.get_world_size(group)):
        failed = _P2P_STATES.get((device.index, n, k, id(group)))
        if isinstance(failed, Exception):
            why = f" (peer memory unavailable: {type(failed).__name__}: {failed})"[:300]
    return "NCCL all-reduce(sum) of FP32 dW per band of rows behind the dW GEMM" + why
