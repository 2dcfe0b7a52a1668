"""NVFP4 packed-tensor type (rtx/formats/nvfp4.py:8-148): E2M1 payload two per
byte (even element in the low nibble), E4M3 block scale per 16 values, FP32
per-tensor scale.  TorchAO's NVFP4Tensor is aliased when it imports; otherwise
an attribute-compatible container stands in."""

from __future__ import annotations

from math import ceil

import torch

from .common import ScaleLayout, flattened_matrix_shape, scales_mma128_to_row_major, scales_row_major_to_mma128

try:  # pragma: no cover
    from torchao.prototype.mx_formats.nvfp4_tensor import NVFP4Tensor as _AONVFP4Tensor
    HAVE_TORCHAO = True
except Exception:
    _AONVFP4Tensor = None
    HAVE_TORCHAO = False

_E2M1 = (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0)


def nvfp4_storage_k(k: int) -> int:
    """Packed rows keep 16-byte alignment: K padded to 32 (rtx/configs/nvfp4.py:15-28)."""
    return (k + 31) // 32 * 32


def nvfp4_scale_chunks(storage_k: int) -> int:
    """512-byte scale tiles per 128 rows; whole 256-value GEMM K tiles (4 tiles of 64 values)."""
    return (ceil(storage_k / 64) + 3) // 4 * 4


class _PackedNVFP4Tensor:
    def __init__(self, qdata, scale, per_tensor_scale, shape, scale_layout):
        self.qdata = qdata
        self.scale = scale
        self.block_size = 16
        self.orig_dtype = torch.bfloat16
        self.per_tensor_scale = per_tensor_scale
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
        return _PackedNVFP4Tensor(self.qdata.to(device), self.scale.to(device), self.per_tensor_scale.to(device),
                                  self._rtx_logical_shape, self._rtx_scale_layout)

    def dequantize(self, dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
        rows, k = flattened_matrix_shape(self._rtx_logical_shape)
        storage_k = nvfp4_storage_k(k)
        nb = storage_k // 16
        codes = self.scale
        if self._rtx_scale_layout != "row_major":
            codes = scales_mma128_to_row_major(codes, rows, nb, nvfp4_scale_chunks(storage_k))
        sb = codes.reshape(rows, nb).view(torch.float8_e4m3fn).float()
        packed = self.qdata.reshape(rows, storage_k // 2).view(torch.uint8)
        table = torch.tensor(_E2M1, dtype=torch.float32, device=packed.device)
        lo, hi = packed & 0xF, packed >> 4
        dec = lambda c: torch.where((c & 8) != 0, -table[(c & 7).long()], table[(c & 7).long()])
        vals = torch.stack((dec(lo), dec(hi)), dim=-1).reshape(rows, storage_k)
        vals = vals * sb.repeat_interleave(16, dim=1) * self.per_tensor_scale.float().reshape(())
        return vals[:, :k].reshape(self._rtx_logical_shape).to(dtype)


NVFP4Tensor = _AONVFP4Tensor if HAVE_TORCHAO else _PackedNVFP4Tensor


def make_nvfp4_tensor(qdata, scales, tensor_scale, shape, scale_layout: ScaleLayout = "row_major"):
    """rtx/formats/nvfp4.py:14-70 with the sm_100a tiling for `mma128`."""
    rows, k = flattened_matrix_shape(tuple(shape))
    fp4_dtype = getattr(torch, "float4_e2m1fn_x2", None)
    if qdata.dtype not in (torch.uint8, fp4_dtype):
        raise TypeError("NVFP4 qdata must use a uint8 container or torch.float4_e2m1fn_x2")
    if (qdata.numel() * 2) % rows:
        raise ValueError("NVFP4 qdata rows do not divide its packed storage")
    storage_k = qdata.numel() * 2 // rows
    if storage_k != nvfp4_storage_k(k):
        raise ValueError(f"NVFP4 qdata storage K={storage_k} cannot represent logical K={k}; "
                         f"expected native 16-byte-row-aligned K={nvfp4_storage_k(k)}")
    if scales.dtype == torch.uint8:
        scales = scales.view(torch.float8_e4m3fn)
    if scales.dtype is not torch.float8_e4m3fn:
        raise TypeError("NVFP4 block scales must use float8_e4m3fn")
    if tensor_scale.dtype is not torch.float32 or tensor_scale.numel() != 1:
        raise TypeError("NVFP4 per-tensor scale must be one FP32 value")
    if not (qdata.device == scales.device == tensor_scale.device):
        raise ValueError("NVFP4 qdata and both scale levels must share one device")
    if scale_layout == "row_major":
        expected = rows * (storage_k // 16)
    elif scale_layout == "mma128":
        expected = ceil(rows / 128) * nvfp4_scale_chunks(storage_k) * 512
    else:
        raise ValueError("NVFP4 supports row-major or 128-row blocked scales")
    if scales.numel() != expected:
        raise ValueError(f"NVFP4 {scale_layout} scales have {scales.numel()} values, expected {expected}")
    return _PackedNVFP4Tensor(qdata.view(*shape[:-1], storage_k // 2), scales, tensor_scale.reshape(()), shape,
                              scale_layout) if not HAVE_TORCHAO else _wrap_torchao(qdata, scales, tensor_scale, shape,
                                                                                  scale_layout, storage_k)


def _wrap_torchao(qdata, scales, tensor_scale, shape, scale_layout, storage_k):  # pragma: no cover
    value = NVFP4Tensor(qdata.view(*shape[:-1], storage_k // 2), scales, 16, torch.bfloat16, tensor_scale.reshape(()),
                        is_swizzled_scales=scale_layout != "row_major")
    value._rtx_scale_layout = scale_layout
    value._rtx_logical_shape = tuple(int(d) for d in shape)
    return value


def nvfp4_matrix_shape(value) -> tuple[int, int]:
    shape = getattr(value, "_rtx_logical_shape", None) or tuple(value.shape)
    return flattened_matrix_shape(tuple(int(d) for d in shape))


def validate_nvfp4_tensor(value) -> None:
    if not isinstance(value, NVFP4Tensor):
        raise TypeError(f"expected an NVFP4Tensor, got {type(value).__name__}")
    if value.block_size != 16:
        raise TypeError("NVFP4 operands use 16-value E4M3 blocks")
    if value.qdata.device.type != "cuda":
        raise ValueError("packed NVFP4 operands must live on a CUDA device")


def nvfp4_scale_layout(value) -> ScaleLayout:
    return "mma128" if value.is_swizzled_scales else "row_major"


def nvfp4_qdata_2d(value) -> torch.Tensor:
    validate_nvfp4_tensor(value)
    rows, k = nvfp4_matrix_shape(value)
    return value.qdata.reshape(rows, nvfp4_storage_k(k) // 2).view(torch.uint8)


def nvfp4_scales_for_kernel(value) -> torch.Tensor:
    validate_nvfp4_tensor(value)
    rows, k = nvfp4_matrix_shape(value)
    storage_k = nvfp4_storage_k(k)
    if nvfp4_scale_layout(value) == "mma128":
        return value.scale.reshape(-1).view(torch.uint8)
    return scales_row_major_to_mma128(value.scale, rows, storage_k // 16, nvfp4_scale_chunks(storage_k))
