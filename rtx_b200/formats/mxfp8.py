"""MXFP8 packed-tensor type and scale-layout views (rtx/formats/mxfp8.py:8-213).

The reference aliases TorchAO's `MXTensor`.  TorchAO is used here too when it
imports; otherwise a small container with the same attribute surface stands in
(`qdata`, `scale`, `block_size`, `orig_dtype`, `elem_dtype`,
`is_swizzled_scales`, `_rtx_scale_layout`, `_rtx_logical_shape`,
`dequantize()`).  The native scale layout of the sm_100a kernels is `mma128`,
the 128-row tiling tcgen05.cp consumes; `mma64` was an SM120 schedule and is
rejected.
"""

from __future__ import annotations

from math import ceil

import torch

from .common import (ScaleLayout, flattened_matrix_shape, scales_mma128_to_row_major, scales_row_major_to_mma128)

try:  # pragma: no cover - depends on the environment
    from torchao.prototype.mx_formats.mx_tensor import MXTensor as _AOMXTensor
    HAVE_TORCHAO = True
except Exception:  # ModuleNotFoundError or an incompatible build
    _AOMXTensor = None
    HAVE_TORCHAO = False


class _PackedMXTensor:
    """Attribute-compatible stand-in for TorchAO's MXTensor (E4M3 payload, E8M0 scales)."""

    def __init__(self, qdata, scale, shape, scale_layout):
        self.qdata = qdata
        self.scale = scale
        self.block_size = 32
        self.orig_dtype = torch.bfloat16
        self.elem_dtype = torch.float8_e4m3fn
        self.is_swizzled_scales = scale_layout != "row_major"
        self._rtx_scale_layout = scale_layout
        self._rtx_logical_shape = tuple(int(d) for d in shape)

    @property
    def shape(self):
        return torch.Size(self._rtx_logical_shape)

    @property
    def device(self):
        return self.qdata.device

    @property
    def dtype(self):
        return self.orig_dtype

    def to(self, device):
        return _PackedMXTensor(self.qdata.to(device), self.scale.to(device), self._rtx_logical_shape,
                               self._rtx_scale_layout)

    def dequantize(self, dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
        rows, k = flattened_matrix_shape(self._rtx_logical_shape)
        storage_k = int(self.qdata.shape[-1])
        nb = storage_k // 32
        codes = self.scale
        if self._rtx_scale_layout != "row_major":
            codes = scales_mma128_to_row_major(codes, rows, nb, ceil(nb / 4))
        codes = codes.reshape(rows, nb).view(torch.uint8).to(torch.int32)
        scale = (codes.clamp(min=1) << 23).view(torch.float32)
        vals = self.qdata.reshape(rows, storage_k).float() * scale.repeat_interleave(32, dim=1)
        return vals[:, :k].reshape(self._rtx_logical_shape).to(dtype)


MXTensor = _AOMXTensor if HAVE_TORCHAO else _PackedMXTensor
MXFP8Tensor = MXTensor


def mxfp8_matrix_shape(value) -> tuple[int, int]:
    shape = getattr(value, "_rtx_logical_shape", None) or tuple(value.shape)
    return flattened_matrix_shape(tuple(int(d) for d in shape))


def make_mxfp8_tensor(qdata: torch.Tensor, scales: torch.Tensor, shape: tuple[int, ...],
                      scale_layout: ScaleLayout = "row_major"):
    """Wrap kernel-produced storage without copying (rtx/formats/mxfp8.py:85-111)."""
    if qdata.device != scales.device:
        raise ValueError("MXFP8 qdata and scales must share one device")
    if scale_layout == "mma64":
        raise ValueError("the mma64 scale layout is an SM120 schedule; sm_100a kernels use row_major or mma128")
    rows, k = flattened_matrix_shape(tuple(shape))
    storage_k = (k + 31) // 32 * 32
    if qdata.numel() != rows * storage_k:
        raise ValueError(f"MXFP8 qdata has {qdata.numel()} values, expected {rows * storage_k}")
    if qdata.dtype == torch.uint8:
        qdata = qdata.view(torch.float8_e4m3fn)
    if scales.dtype == torch.uint8:
        scales = scales.view(torch.float8_e8m0fnu)
    qdata = qdata.view(*shape[:-1], storage_k)
    nb = storage_k // 32
    expected = rows * nb if scale_layout == "row_major" else ceil(rows / 128) * ceil(nb / 4) * 512
    if scales.numel() != expected:
        raise ValueError(f"{scale_layout} MXFP8 scales have {scales.numel()} values, expected {expected}")
    if HAVE_TORCHAO:  # pragma: no cover
        from torchao.quantization.quantize_.common import KernelPreference

        value = MXTensor.from_qdata_and_scales(qdata, scales, torch.bfloat16, block_size=32,
                                               kernel_preference=KernelPreference.AUTO,
                                               is_swizzled_scales=scale_layout != "row_major")
        value._rtx_scale_layout = scale_layout
        value._rtx_logical_shape = tuple(int(d) for d in shape)
        return value
    return _PackedMXTensor(qdata, scales, shape, scale_layout)


def validate_mxfp8_tensor(value) -> None:
    if not isinstance(value, MXTensor):
        raise TypeError(f"expected an MXFP8Tensor, got {type(value).__name__}")
    if value.block_size != 32 or value.elem_dtype is not torch.float8_e4m3fn:
        raise TypeError("MXFP8 operands use E4M3 payloads with 32-value E8M0 blocks")
    if value.qdata.device.type != "cuda":
        raise ValueError("packed MXFP8 operands must live on a CUDA device")


def mxfp8_scale_layout(value) -> ScaleLayout:
    rows, k = mxfp8_matrix_shape(value)
    nb = int(value.qdata.shape[-1]) // 32
    marker = getattr(value, "_rtx_scale_layout", None)
    if not value.is_swizzled_scales:
        if value.scale.numel() != rows * nb:
            raise ValueError(f"row-major MXFP8 scales have {value.scale.numel()} values, expected {rows * nb}")
        return "row_major"
    if marker == "mma64":
        raise ValueError("mma64 scales cannot feed the sm_100a kernels; requantize from the BF16 weight")
    if value.scale.numel() != ceil(rows / 128) * ceil(nb / 4) * 512:
        raise ValueError("blocked MXFP8 scale storage is not the 128-row tiling")
    return "mma128"


def mxfp8_qdata_2d(value) -> torch.Tensor:
    validate_mxfp8_tensor(value)
    rows, _ = mxfp8_matrix_shape(value)
    return value.qdata.reshape(rows, int(value.qdata.shape[-1]))


def mxfp8_scales_for_kernel(value) -> torch.Tensor:
    """Scale codes in the layout the GEMM consumes (mma128); row-major storage is re-tiled."""
    validate_mxfp8_tensor(value)
    rows, _ = mxfp8_matrix_shape(value)
    nb = int(value.qdata.shape[-1]) // 32
    if mxfp8_scale_layout(value) == "mma128":
        return value.scale.reshape(-1).view(torch.uint8)
    return scales_row_major_to_mma128(value.scale, rows, nb, ceil(nb / 4))


def convert_mxfp8_scale_layout(value, scale_layout: ScaleLayout):
    """Return `value` with its scales stored in `scale_layout` (payload shared)."""
    rows, _ = mxfp8_matrix_shape(value)
    nb = int(value.qdata.shape[-1]) // 32
    have = mxfp8_scale_layout(value)
    if have == scale_layout:
        return value
    if scale_layout == "mma128":
        scales = scales_row_major_to_mma128(value.scale, rows, nb, ceil(nb / 4))
    elif scale_layout == "row_major":
        scales = scales_mma128_to_row_major(value.scale, rows, nb, ceil(nb / 4))
    else:
        raise ValueError("sm_100a kernels use row_major or mma128 scales")
    return make_mxfp8_tensor(value.qdata, scales, tuple(value._rtx_logical_shape), scale_layout)
