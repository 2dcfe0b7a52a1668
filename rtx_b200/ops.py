"""Tensor-level launchers over the C ABI.

Each function mirrors one launch callable the reference obtains from its
`compile_*` factories (rtx/kernels/*.py) — same operand order, contiguous CUDA
tensors, asynchronous on the current stream — but runs the sm_100a kernels of
librtxb.  PyTorch is used only for device memory and the stream handle.
"""

from __future__ import annotations

import threading
from typing import Optional, Tuple

import torch

from . import _native as N

_status_lock = threading.Lock()
_status_words: dict[int, torch.Tensor] = {}


def _stream_ptr() -> int:
    """Raw handle of the current stream of the current device (no Stream object is built: this sits on the
    launch path of microsecond-scale decode steps)."""
    return torch._C._cuda_getCurrentRawStream(torch._C._cuda_getDevice())


class _NoSwitch:
    def __enter__(self):
        return self

    def __exit__(self, *exc):
        return False


_NO_SWITCH = _NoSwitch()


def _on(device: torch.device):
    """Context in which `device` is current: nothing at all when it already is (the usual case)."""
    idx = device.index
    if idx is None or idx == torch._C._cuda_getDevice():
        return _NO_SWITCH
    return torch.cuda.device(idx)


def status_word(device: torch.device) -> torch.Tensor:
    """Per-device int32 the kernels set when a bounded wait runs out."""
    idx = device.index if device.index is not None else torch.cuda.current_device()
    word = _status_words.get(idx)      # dict reads are atomic; the lock only guards creation
    if word is None:
        with _status_lock:
            word = _status_words.get(idx)
            if word is None:
                word = torch.zeros(1, dtype=torch.int32, device=torch.device("cuda", idx))
                _status_words[idx] = word
    return word


def check_device_status(device: Optional[torch.device] = None) -> None:
    """Synchronise and raise if any kernel on `device` reported a wait that ran out."""
    device = device or torch.device("cuda", torch.cuda.current_device())
    word = status_word(device)
    code = int(word.item())
    if code != 0:
        word.zero_()
        raise RuntimeError(f"rtx_b200 kernel reported: {N.DEVICE_STATUS_NAMES.get(code, code)}")


def _require(t: torch.Tensor, dtype: torch.dtype, name: str) -> None:
    if not isinstance(t, torch.Tensor):
        raise TypeError(f"{name} must be a torch.Tensor")
    if t.device.type != "cuda":
        raise ValueError(f"{name} must be a CUDA tensor")
    if t.dtype != dtype:
        raise TypeError(f"{name} must have dtype {dtype}, got {t.dtype}")
    if t.dim() != 2 or not t.is_contiguous():
        raise ValueError(f"{name} must be a contiguous 2-D tensor")


def mx_storage_k(k: int) -> int:
    return (k + 31) // 32 * 32


def mxfp8_scale_numel(rows: int, k: int, layout: int) -> int:
    return N.query("rtxb_mxfp8_scale_bytes", rows, k, layout)


def nvfp4_scale_numel(rows: int, k: int, layout: int) -> int:
    return N.query("rtxb_nvfp4_scale_bytes", rows, k, layout)


# ---------------------------------------------------------------------------
# MXFP8
# ---------------------------------------------------------------------------

def mxfp8_quantize(src: torch.Tensor, *, layout: int = N.SCALE_MMA128, rounding: int = N.ROUND_INFINITY,
                   q: Optional[torch.Tensor] = None, scales: Optional[torch.Tensor] = None
                   ) -> Tuple[torch.Tensor, torch.Tensor]:
    """(src bf16 [R,K]) -> (q u8 [R,Kp] E4M3 codes, scales u8 E8M0 codes in `layout`)."""
    _require(src, torch.bfloat16, "src")
    rows, k = src.shape
    kp = mx_storage_k(k)
    if q is None:
        q = torch.empty(rows, kp, dtype=torch.uint8, device=src.device)
    if scales is None:
        scales = torch.empty(mxfp8_scale_numel(rows, k, layout), dtype=torch.uint8, device=src.device)
    with _on(src.device):
        N.call("rtxb_mxfp8_quantize", src.data_ptr(), rows, k, k, q.data_ptr(), scales.data_ptr(), layout, rounding,
               _stream_ptr())
    return q, scales


def mxfp8_quantize_transposed(src: torch.Tensor, *, layout: int = N.SCALE_MMA128,
                              rounding: int = N.ROUND_INFINITY) -> Tuple[torch.Tensor, torch.Tensor]:
    """src bf16 stored [K,R] -> quantisation of src.T: q u8 [R,Kp] with 32-blocks along K."""
    _require(src, torch.bfloat16, "src")
    k, rows = src.shape
    kp = mx_storage_k(k)
    q = torch.empty(rows, kp, dtype=torch.uint8, device=src.device)
    scales = torch.empty(mxfp8_scale_numel(rows, k, layout), dtype=torch.uint8, device=src.device)
    with _on(src.device):
        N.call("rtxb_mxfp8_quantize_transposed", src.data_ptr(), rows, k, rows, q.data_ptr(), scales.data_ptr(),
               layout, rounding, _stream_ptr())
    return q, scales


def mxfp8_quantize_dual(src: torch.Tensor, *, layout: int = N.SCALE_MMA128, rounding: int = N.ROUND_INFINITY):
    """src bf16 [M, N] -> (q_rows [M, Np], s_rows, q_t [N, Mp], s_t): the row quantization and the
    quantization of the transpose from one read of src (the backward's gradient operand)."""
    _require(src, torch.bfloat16, "src")
    m, n = src.shape
    np_, mp = mx_storage_k(n), mx_storage_k(m)
    q_rows = torch.empty(m, np_, dtype=torch.uint8, device=src.device)
    s_rows = torch.empty(mxfp8_scale_numel(m, n, layout), dtype=torch.uint8, device=src.device)
    q_t = torch.empty(n, mp, dtype=torch.uint8, device=src.device)
    s_t = torch.empty(mxfp8_scale_numel(n, m, layout), dtype=torch.uint8, device=src.device)
    with _on(src.device):
        N.call("rtxb_mxfp8_quantize_dual", src.data_ptr(), m, n, n, q_rows.data_ptr(), s_rows.data_ptr(), q_t.data_ptr(),
               s_t.data_ptr(), layout, rounding, _stream_ptr())
    return q_rows, s_rows, q_t, s_t


def mxfp8_gemm(qa, sa, qb, sb, m: int, n: int, k: int, *, out_dtype: torch.dtype = torch.bfloat16,
               out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """(qx, qw, sx, sw) -> out[m,n]; scales in the mma128 layout."""
    if out is None:
        out = torch.empty(m, n, dtype=out_dtype, device=qa.device)
    code = N.OUT_BF16 if out.dtype == torch.bfloat16 else N.OUT_F32
    with _on(qa.device):
        N.call("rtxb_mxfp8_gemm", qa.data_ptr(), sa.data_ptr(), qb.data_ptr(), sb.data_ptr(), out.data_ptr(), m, n, k,
               out.stride(0), code, _stream_ptr(), status_word(qa.device).data_ptr())
    return out


def mxfp8_gemm_row_blocks(qa, sa, qb, sb, m: int, n: int, k: int, blocks, *, first_block: int = 0) -> None:
    """The packed GEMM with its [m, n] output split into row blocks: block j (rows j*R .. j*R+R-1, R = the rows of
    blocks[0], a multiple of 256) goes to the tensor blocks[j], which may be a peer-mapped buffer of another GPU."""
    import ctypes

    rows = int(blocks[0].shape[0])
    dtype = blocks[0].dtype
    for b in blocks:
        if b.dtype is not dtype or b.dim() != 2 or b.shape[1] != n or b.stride(1) != 1 or b.stride(0) != blocks[0].stride(0):
            raise ValueError("output blocks must be row-major [rows, n] tensors of one dtype and pitch")
    ptrs = (ctypes.c_void_p * len(blocks))(*[b.data_ptr() for b in blocks])
    with _on(qa.device):
        N.call("rtxb_mxfp8_gemm_row_blocks", qa.data_ptr(), sa.data_ptr(), qb.data_ptr(), sb.data_ptr(), ptrs, len(blocks),
               rows, m, n, k, blocks[0].stride(0), N.OUT_BF16 if dtype == torch.bfloat16 else N.OUT_F32, first_block,
               _stream_ptr(), status_word(qa.device).data_ptr())


def mxfp8_gemm_glu(qa, sa, qb, sb, m: int, inter: int, k: int, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    if out is None:
        out = torch.empty(m, inter, dtype=torch.bfloat16, device=qa.device)
    with _on(qa.device):
        N.call("rtxb_mxfp8_gemm_glu", qa.data_ptr(), sa.data_ptr(), qb.data_ptr(), sb.data_ptr(), out.data_ptr(), m,
               inter, k, out.stride(0), _stream_ptr(), status_word(qa.device).data_ptr())
    return out


def mxfp8_linear_fwd_fused_x(x: torch.Tensor, qw: torch.Tensor, sw: torch.Tensor, n: int,
                             out: Optional[torch.Tensor] = None, rounding: int = N.ROUND_INFINITY) -> torch.Tensor:
    """(x bf16 [M,K], packed weight [N,Kp] + mma128 scales) -> out bf16 [M,N] in ONE launch: the GEMM's
    quantizer warps encode X tile by tile (no packed copy of X)."""
    _require(x, torch.bfloat16, "x")
    m, k = x.shape
    if out is None:
        out = torch.empty(m, n, dtype=torch.bfloat16, device=x.device)
    with _on(x.device):
        N.call("rtxb_mxfp8_linear_fwd_fused_x", x.data_ptr(), x.stride(0), qw.data_ptr(), sw.data_ptr(), out.data_ptr(),
               m, n, k, out.stride(0), rounding, _stream_ptr(), status_word(x.device).data_ptr())
    return out


class Workspace:
    """Caller-owned scratch for the composite entry points; grows on demand and is
    reused by every call made on the stream it was created for."""

    def __init__(self, device: torch.device):
        self.device = device
        self.buf: Optional[torch.Tensor] = None

    def get(self, nbytes: int) -> torch.Tensor:
        if self.buf is None or self.buf.numel() < nbytes:
            self.buf = torch.empty(nbytes, dtype=torch.uint8, device=self.device)
        return self.buf


def mxfp8_linear_fwd(x: torch.Tensor, w: torch.Tensor, ws: Workspace, out: Optional[torch.Tensor] = None,
                     rounding: int = N.ROUND_INFINITY) -> torch.Tensor:
    """(x bf16 [M,K], w bf16 [N,K]) -> out bf16 [M,N]: quantize both, block-scaled GEMM."""
    _require(x, torch.bfloat16, "x")
    _require(w, torch.bfloat16, "weight")
    m, k = x.shape
    n = w.shape[0]
    if w.shape[1] != k:
        raise ValueError("x and weight disagree on K")
    if out is None:
        out = torch.empty(m, n, dtype=torch.bfloat16, device=x.device)
    nbytes = N.query("rtxb_mxfp8_linear_workspace_bytes", m, n, k)
    buf = ws.get(nbytes)
    with _on(x.device):
        N.call("rtxb_mxfp8_linear_fwd", x.data_ptr(), w.data_ptr(), out.data_ptr(), m, n, k, rounding, buf.data_ptr(),
               buf.numel(), _stream_ptr(), status_word(x.device).data_ptr())
    return out


def mxfp8_gemm_glu_mx(qa, sa, qb, sb, m: int, inter: int, k: int, *, want_bf16: bool = False):
    """GLU GEMM whose epilogue emits H as MXFP8: returns (q_h u8 [m, inter], s_h u8 tiles, h bf16 | None)."""
    q = torch.empty(m, inter, dtype=torch.uint8, device=qa.device)
    s = torch.empty(mxfp8_scale_numel(m, inter, N.SCALE_MMA128), dtype=torch.uint8, device=qa.device)
    h = torch.empty(m, inter, dtype=torch.bfloat16, device=qa.device) if want_bf16 else None
    with _on(qa.device):
        N.call("rtxb_mxfp8_gemm_glu_mx", qa.data_ptr(), sa.data_ptr(), qb.data_ptr(), sb.data_ptr(),
               h.data_ptr() if want_bf16 else None, q.data_ptr(), s.data_ptr(), m, inter, k, inter, _stream_ptr(),
               status_word(qa.device).data_ptr())
    return q, s, h


def mxfp8_gemm_glu_mx_fused_x(x: torch.Tensor, qb, sb, inter: int, *, want_bf16: bool = False):
    """mxfp8_gemm_glu_mx with X given in BF16 and quantized by the GEMM's own quantizer warps."""
    _require(x, torch.bfloat16, "x")
    m, k = x.shape
    q = torch.empty(m, inter, dtype=torch.uint8, device=x.device)
    s = torch.empty(mxfp8_scale_numel(m, inter, N.SCALE_MMA128), dtype=torch.uint8, device=x.device)
    h = torch.empty(m, inter, dtype=torch.bfloat16, device=x.device) if want_bf16 else None
    with _on(x.device):
        N.call("rtxb_mxfp8_gemm_glu_mx_fused_x", x.data_ptr(), x.stride(0), qb.data_ptr(), sb.data_ptr(),
               h.data_ptr() if want_bf16 else None, q.data_ptr(), s.data_ptr(), m, inter, k, inter, _stream_ptr(),
               status_word(x.device).data_ptr())
    return q, s, h


def mxfp8_glu_mlp_fwd(x, w_gate_up, w_down, ws: Workspace, h: Optional[torch.Tensor] = None,
                      y: Optional[torch.Tensor] = None, want_hidden: bool = True):
    """want_hidden=False: H is never materialized in BF16 (returned as None)."""
    _require(x, torch.bfloat16, "x")
    _require(w_gate_up, torch.bfloat16, "w_gate_up")
    _require(w_down, torch.bfloat16, "w_down")
    m, k = x.shape
    inter = w_gate_up.shape[0] // 2
    n_out = w_down.shape[0]
    if w_gate_up.shape[1] != k or w_down.shape[1] != inter:
        raise ValueError("weight shapes do not chain")
    if h is None and want_hidden:
        h = torch.empty(m, inter, dtype=torch.bfloat16, device=x.device)
    if y is None:
        y = torch.empty(m, n_out, dtype=torch.bfloat16, device=x.device)
    nbytes = N.query("rtxb_mxfp8_glu_mlp_workspace_bytes", m, k, inter, n_out)
    buf = ws.get(nbytes)
    with _on(x.device):
        N.call("rtxb_mxfp8_glu_mlp_fwd", x.data_ptr(), w_gate_up.data_ptr(), w_down.data_ptr(),
               h.data_ptr() if h is not None else None, y.data_ptr(), m, k, inter, n_out, buf.data_ptr(), buf.numel(), _stream_ptr(),
               status_word(x.device).data_ptr())
    return h, y


def mxfp8_linear_bwd(dy, x, w, ws: Workspace, *, need_dx: bool = True, need_dw: bool = True,
                     dw_dtype: torch.dtype = torch.bfloat16, dx_out: Optional[torch.Tensor] = None,
                     dw_out: Optional[torch.Tensor] = None):
    """(dY [M,N], X [M,K], W [N,K]) -> (dX bf16 [M,K] | None, dW [N,K] | None); results go into
    `dx_out` / `dw_out` (contiguous, right shape and dtype) when given."""
    _require(dy, torch.bfloat16, "grad_output")
    m, n = dy.shape
    k = w.shape[1] if w is not None else x.shape[1]
    dx = dw = None
    if need_dx:
        dx = dx_out if dx_out is not None else torch.empty(m, k, dtype=torch.bfloat16, device=dy.device)
        if tuple(dx.shape) != (m, k) or dx.dtype is not torch.bfloat16 or not dx.is_contiguous():
            raise ValueError("dx_out must be a contiguous BF16 [M, K] tensor")
    if need_dw:
        dw_dtype = dw_out.dtype if dw_out is not None else dw_dtype
        dw = dw_out if dw_out is not None else torch.empty(n, k, dtype=dw_dtype, device=dy.device)
        if tuple(dw.shape) != (n, k) or dw.dtype not in (torch.bfloat16, torch.float32) or not dw.is_contiguous():
            raise ValueError("dw_out must be a contiguous BF16 or FP32 [N, K] tensor")
    if need_dx:
        _require(w, torch.bfloat16, "weight")
    if need_dw:
        _require(x, torch.bfloat16, "x")
    nbytes = N.query("rtxb_mxfp8_backward_workspace_bytes", m, n, k)
    buf = ws.get(nbytes)
    with _on(dy.device):
        N.call("rtxb_mxfp8_linear_bwd", dy.data_ptr(), x.data_ptr() if x is not None else None,
               w.data_ptr() if w is not None else None, dx.data_ptr() if need_dx else None,
               dw.data_ptr() if need_dw else None, N.OUT_BF16 if dw_dtype == torch.bfloat16 else N.OUT_F32, m, n, k,
               buf.data_ptr(), buf.numel(), _stream_ptr(), status_word(dy.device).data_ptr())
    return dx, dw


def peer_barrier(flag_ptrs, rank: int, epoch_counter: torch.Tensor, limit_ns: int = 2_000_000_000) -> None:
    """Node barrier through flag words in peer-mapped memory on the current stream: `flag_ptrs[t]` is the address
    of rank t's array of eight int32 words as mapped into this process; `epoch_counter` is one int32 of this
    rank's device memory that the kernel advances (zero before the first barrier)."""
    import ctypes

    if epoch_counter.dtype is not torch.int32 or epoch_counter.numel() != 1 or epoch_counter.device.type != "cuda":
        raise ValueError("epoch_counter must be one int32 on the device")
    ptrs = (ctypes.c_void_p * len(flag_ptrs))(*flag_ptrs)
    device = epoch_counter.device
    with _on(device):
        N.call("rtxb_peer_barrier", ptrs, len(flag_ptrs), rank, epoch_counter.data_ptr(), limit_ns, _stream_ptr(),
               status_word(device).data_ptr())


def sum_parts_f32_to_bf16(parts: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """parts f32 [S, ...] contiguous -> bf16 [...]: the S partial sums added in index order, one rounding."""
    if parts.dtype is not torch.float32 or not parts.is_contiguous() or parts.dim() < 2:
        raise ValueError("parts must be a contiguous FP32 tensor [S, ...]")
    count = parts[0].numel()
    if out is None:
        out = torch.empty(parts.shape[1:], dtype=torch.bfloat16, device=parts.device)
    if out.numel() != count or out.dtype is not torch.bfloat16 or not out.is_contiguous():
        raise ValueError("out must be a contiguous BF16 tensor with one part's element count")
    with _on(parts.device):
        N.call("rtxb_sum_parts_f32_to_bf16", parts.data_ptr(), int(parts.shape[0]), count, count, out.data_ptr(),
               _stream_ptr())
    return out


# ---------------------------------------------------------------------------
# Launch controls: GEMM schedule of the calling thread, SM margin of the process
# ---------------------------------------------------------------------------

GEMM_SCHEDULES = {"auto": 0, "single": 1, "pair": 2, "stream": 3, "fused_x": 4}


class gemm_schedule:
    """Context manager: GEMMs launched by this thread inside use the named schedule ("auto", "single",
    "pair", "stream"); restored on exit.  All schedules give the same bits."""

    def __init__(self, name: str):
        if name not in GEMM_SCHEDULES:
            raise ValueError(f"unknown GEMM schedule {name!r}; built: {', '.join(GEMM_SCHEDULES)}")
        self.code, self.prev = GEMM_SCHEDULES[name], 0

    def __enter__(self):
        self.prev = N.query("rtxb_get_gemm_schedule")
        N.call("rtxb_set_gemm_schedule", self.code)
        return self

    def __exit__(self, *exc):
        N.call("rtxb_set_gemm_schedule", self.prev)
        return False


class _NoSchedule:
    def __enter__(self):
        return self

    def __exit__(self, *exc):
        return False


_NO_SCHEDULE = _NoSchedule()


def schedule_of(gemm_config):
    """The context manager for a GEMM config's schedule ("auto" costs nothing)."""
    name = getattr(gemm_config, "schedule", "auto")
    return _NO_SCHEDULE if name == "auto" else gemm_schedule(name)


class sm_margin:
    """Context manager: the library's persistent kernels launched inside leave `sms` SMs unused, so
    that a collective running beside them (NCCL all-reduce of dW during the dX GEMM) gets to run.
    Process-wide setting (one process per GPU); restored on exit."""

    def __init__(self, sms: int):
        self.sms, self.prev = int(sms), 0

    def __enter__(self):
        self.prev = N.query("rtxb_get_sm_margin")
        N.call("rtxb_set_sm_margin", self.sms)
        return self

    def __exit__(self, *exc):
        N.call("rtxb_set_sm_margin", self.prev)
        return False


# ---------------------------------------------------------------------------
# NVFP4
# ---------------------------------------------------------------------------

def nvfp4_tensor_scale(src: torch.Tensor, mode: int = N.TENSOR_SCALE_POWER2,
                       other_scale: Optional[torch.Tensor] = None):
    """Device-side |max| reduction + outer-scale rule.  Returns scale f32[1], and
    also scale*other_scale f32[1] when `other_scale` is given."""
    _require(src, torch.bfloat16, "src")
    rows, k = src.shape
    scratch = torch.empty(1, dtype=torch.int32, device=src.device)
    scale = torch.empty(1, dtype=torch.float32, device=src.device)
    prod = torch.empty(1, dtype=torch.float32, device=src.device) if other_scale is not None else None
    with _on(src.device):
        N.call("rtxb_nvfp4_tensor_scale", src.data_ptr(), rows, k, k, mode, scratch.data_ptr(), scale.data_ptr(),
               other_scale.data_ptr() if other_scale is not None else None,
               prod.data_ptr() if prod is not None else None, _stream_ptr())
    return (scale, prod) if other_scale is not None else scale


def nvfp4_quantize(src: torch.Tensor, tensor_scale: Optional[torch.Tensor], *, layout: int = N.SCALE_MMA128):
    """(src bf16 [R,K], tensor_scale f32[1] | None) -> (q u8 [R,Kp/2], scales u8 E4M3 codes)."""
    _require(src, torch.bfloat16, "src")
    rows, k = src.shape
    kp = mx_storage_k(k)
    q = torch.empty(rows, kp // 2, dtype=torch.uint8, device=src.device)
    scales = torch.empty(nvfp4_scale_numel(rows, k, layout), dtype=torch.uint8, device=src.device)
    with _on(src.device):
        N.call("rtxb_nvfp4_quantize", src.data_ptr(), rows, k, k, q.data_ptr(), scales.data_ptr(), layout,
               tensor_scale.data_ptr() if tensor_scale is not None else None, _stream_ptr())
    return q, scales


def nvfp4_quantize_dynamic(src: torch.Tensor, mode: int = N.TENSOR_SCALE_POWER2,
                           other_scale: Optional[torch.Tensor] = None, *, layout: int = N.SCALE_MMA128):
    """Outer scale from the tensor's own |max| and quantization in one call (two chained launches
    for decode-sized tensors).  Returns (q, scales, tensor_scale f32[1], scale*other_scale f32[1] | None)."""
    _require(src, torch.bfloat16, "src")
    rows, k = src.shape
    kp = mx_storage_k(k)
    q = torch.empty(rows, kp // 2, dtype=torch.uint8, device=src.device)
    scales = torch.empty(nvfp4_scale_numel(rows, k, layout), dtype=torch.uint8, device=src.device)
    scratch = torch.empty(64, dtype=torch.int32, device=src.device)
    scale = torch.empty(1, dtype=torch.float32, device=src.device)
    prod = torch.empty(1, dtype=torch.float32, device=src.device) if other_scale is not None else None
    with _on(src.device):
        N.call("rtxb_nvfp4_quantize_dynamic", src.data_ptr(), rows, k, k, mode, q.data_ptr(), scales.data_ptr(), layout,
               scale.data_ptr(), other_scale.data_ptr() if other_scale is not None else None,
               prod.data_ptr() if prod is not None else None, scratch.data_ptr(), _stream_ptr())
    return q, scales, scale, prod


_PREQUANT_W_BYTES: dict = {}


def nvfp4_linear_fwd_prequant_w(x, qw, sw, w_scale, n: int, ws: Workspace, out: Optional[torch.Tensor] = None,
                                scale_mode: int = N.TENSOR_SCALE_POWER2) -> torch.Tensor:
    """Packed weight (payload, mma128 block scales, outer scale), BF16 activations quantized on the
    fly with their current outer scale; the GEMM overlaps the activation quantizer."""
    _require(x, torch.bfloat16, "x")
    m, k = x.shape
    if out is None:
        out = torch.empty(m, n, dtype=torch.bfloat16, device=x.device)
    nbytes = _PREQUANT_W_BYTES.get((m, k))
    if nbytes is None:
        nbytes = _PREQUANT_W_BYTES[(m, k)] = N.query("rtxb_nvfp4_linear_prequant_w_workspace_bytes", m, k)
    buf = ws.get(nbytes)
    with _on(x.device):
        N.call("rtxb_nvfp4_linear_fwd_prequant_w", x.data_ptr(), qw.data_ptr(), sw.data_ptr(), w_scale.data_ptr(),
               out.data_ptr(), m, n, k, scale_mode, buf.data_ptr(), buf.numel(), _stream_ptr(),
               status_word(x.device).data_ptr())
    return out


def nvfp4_quantize_delayed(src: torch.Tensor, history: torch.Tensor, next_history: torch.Tensor, *,
                           window_max: bool = True, mode: int = N.TENSOR_SCALE_POWER2,
                           other_scale: Optional[torch.Tensor] = None, layout: int = N.SCALE_MMA128):
    """Delayed policy for one operand: quantize with the scale of the |max| history, observe the current
    |max| in the same pass, write the successor history.  Returns (q, scales, scale f32[1], product | None)."""
    _require(src, torch.bfloat16, "src")
    rows, k = src.shape
    kp = mx_storage_k(k)
    q = torch.empty(rows, kp // 2, dtype=torch.uint8, device=src.device)
    scales = torch.empty(nvfp4_scale_numel(rows, k, layout), dtype=torch.uint8, device=src.device)
    scale = torch.empty(1, dtype=torch.float32, device=src.device)
    prod = torch.empty(1, dtype=torch.float32, device=src.device) if other_scale is not None else None
    with _on(src.device):
        N.call("rtxb_nvfp4_quantize_delayed", src.data_ptr(), rows, k, k, q.data_ptr(), scales.data_ptr(), layout,
               history.data_ptr(), next_history.data_ptr(), history.numel(), int(window_max), mode, scale.data_ptr(),
               other_scale.data_ptr() if other_scale is not None else None,
               prod.data_ptr() if prod is not None else None, _stream_ptr())
    return q, scales, scale, prod


def nvfp4_linear_fwd_delayed(x, w, ws: Workspace, x_history, w_history, next_x_history, next_w_history, *,
                             window_max: bool = True, scale_mode: int = N.TENSOR_SCALE_POWER2,
                             out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """NVFP4 forward under the delayed policy: two quantizer launches (each also observes its operand's
    |max| for the next step) and the GEMM; no reduction over the current tensors before the quantization."""
    _require(x, torch.bfloat16, "x")
    _require(w, torch.bfloat16, "weight")
    m, k = x.shape
    n = w.shape[0]
    if w.shape[1] != k:
        raise ValueError("x and weight disagree on K")
    for t in (x_history, w_history, next_x_history, next_w_history):
        if t.dtype is not torch.float32 or not t.is_contiguous() or t.numel() != x_history.numel():
            raise ValueError("amax histories must be contiguous FP32 vectors of one length")
    if out is None:
        out = torch.empty(m, n, dtype=torch.bfloat16, device=x.device)
    nbytes = N.query("rtxb_nvfp4_linear_workspace_bytes", m, n, k)
    buf = ws.get(nbytes)
    with _on(x.device):
        N.call("rtxb_nvfp4_linear_fwd_delayed", x.data_ptr(), w.data_ptr(), out.data_ptr(), m, n, k,
               x_history.data_ptr(), w_history.data_ptr(), next_x_history.data_ptr(), next_w_history.data_ptr(),
               x_history.numel(), int(window_max), scale_mode, buf.data_ptr(), buf.numel(), _stream_ptr(),
               status_word(x.device).data_ptr())
    return out


def nvfp4_effective_region_rows(rows: int, requested: int) -> int:
    """The reference's `_effective_scale_region_rows` (rtx/fp4.py:89-94) with "one region" spelled as
    `rows`: a request that does not split the rows evenly into more than one region covers the tensor."""
    if requested <= 0 or rows <= requested or rows % requested:
        return rows
    return requested


def nvfp4_region_scales(src: torch.Tensor, region_rows: int, mode: int = N.TENSOR_SCALE_POWER2) -> torch.Tensor:
    """FP32 outer scale of every region of `region_rows` consecutive rows (must divide the rows)."""
    _require(src, torch.bfloat16, "src")
    rows, k = src.shape
    scales = torch.empty(rows // max(region_rows, 1), dtype=torch.float32, device=src.device)
    scratch = torch.empty(1, dtype=torch.int32, device=src.device)
    with _on(src.device):
        N.call("rtxb_nvfp4_region_scales", src.data_ptr(), rows, k, k, region_rows, mode, scratch.data_ptr(),
               scales.data_ptr(), _stream_ptr())
    return scales


def nvfp4_quantize_regions(src: torch.Tensor, region_scales: torch.Tensor, region_rows: int, *,
                           layout: int = N.SCALE_MMA128):
    """Every region of rows quantized with its own outer scale -> (q, block scales)."""
    _require(src, torch.bfloat16, "src")
    rows, k = src.shape
    kp = mx_storage_k(k)
    q = torch.empty(rows, kp // 2, dtype=torch.uint8, device=src.device)
    scales = torch.empty(nvfp4_scale_numel(rows, k, layout), dtype=torch.uint8, device=src.device)
    with _on(src.device):
        N.call("rtxb_nvfp4_quantize_regions", src.data_ptr(), rows, k, k, q.data_ptr(), scales.data_ptr(), layout,
               region_scales.data_ptr(), region_rows, _stream_ptr())
    return q, scales


def nvfp4_gemm_regions(qa, sa, qb, sb, m: int, n: int, k: int, x_region_scales, x_region_rows: int,
                       w_region_scales, w_region_rows: int, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out[m, n] = bf16(acc * (xs[m / Rx] * ws[n / Rw]))."""
    if out is None:
        out = torch.empty(m, n, dtype=torch.bfloat16, device=qa.device)
    with _on(qa.device):
        N.call("rtxb_nvfp4_gemm_regions", qa.data_ptr(), sa.data_ptr(), qb.data_ptr(), sb.data_ptr(), out.data_ptr(),
               m, n, k, out.stride(0), x_region_scales.data_ptr(), x_region_rows, w_region_scales.data_ptr(),
               w_region_rows, _stream_ptr(), status_word(qa.device).data_ptr())
    return out


def nvfp4_linear_fwd_regions(x, w, ws: Workspace, x_region_rows: int, w_region_rows: int,
                             out: Optional[torch.Tensor] = None,
                             scale_mode: int = N.TENSOR_SCALE_POWER2) -> torch.Tensor:
    """NVFP4 forward with the row-region outer scales (region sizes are requests, see
    nvfp4_effective_region_rows): two region-|max| launches, two quantizers, the GEMM — or, where both operands'
    regions are small, one region-|max| launch, one quantizer launch and the GEMM as its programmatic dependent."""
    _require(x, torch.bfloat16, "x")
    _require(w, torch.bfloat16, "weight")
    m, k = x.shape
    n = w.shape[0]
    if w.shape[1] != k:
        raise ValueError("x and weight disagree on K")
    if out is None:
        out = torch.empty(m, n, dtype=torch.bfloat16, device=x.device)
    nbytes = N.query("rtxb_nvfp4_linear_regions_workspace_bytes", m, n, k, x_region_rows, w_region_rows)
    buf = ws.get(nbytes)
    with _on(x.device):
        N.call("rtxb_nvfp4_linear_fwd_regions", x.data_ptr(), w.data_ptr(), out.data_ptr(), m, n, k, x_region_rows,
               w_region_rows, scale_mode, buf.data_ptr(), buf.numel(), _stream_ptr(),
               status_word(x.device).data_ptr())
    return out


def nvfp4_gemm(qa, sa, qb, sb, m: int, n: int, k: int, output_scale: Optional[torch.Tensor], *,
               out_dtype: torch.dtype = torch.bfloat16, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    if out is None:
        out = torch.empty(m, n, dtype=out_dtype, device=qa.device)
    code = N.OUT_BF16 if out.dtype == torch.bfloat16 else N.OUT_F32
    with _on(qa.device):
        N.call("rtxb_nvfp4_gemm", qa.data_ptr(), sa.data_ptr(), qb.data_ptr(), sb.data_ptr(), out.data_ptr(), m, n, k,
               out.stride(0), code, output_scale.data_ptr() if output_scale is not None else None, _stream_ptr(),
               status_word(qa.device).data_ptr())
    return out


def nvfp4_linear_fwd(x, w, ws: Workspace, out: Optional[torch.Tensor] = None,
                     scale_mode: int = N.TENSOR_SCALE_POWER2) -> torch.Tensor:
    _require(x, torch.bfloat16, "x")
    _require(w, torch.bfloat16, "weight")
    m, k = x.shape
    n = w.shape[0]
    if w.shape[1] != k:
        raise ValueError("x and weight disagree on K")
    if out is None:
        out = torch.empty(m, n, dtype=torch.bfloat16, device=x.device)
    nbytes = N.query("rtxb_nvfp4_linear_workspace_bytes", m, n, k)
    buf = ws.get(nbytes)
    with _on(x.device):
        N.call("rtxb_nvfp4_linear_fwd", x.data_ptr(), w.data_ptr(), out.data_ptr(), m, n, k, scale_mode,
               buf.data_ptr(), buf.numel(), _stream_ptr(), status_word(x.device).data_ptr())
    return out
