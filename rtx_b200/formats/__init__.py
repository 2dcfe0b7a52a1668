"""Packed operand types and scale-layout conversion (rtx/formats/__init__.py)."""

from .common import (PACKED_OPERAND_SCHEMA_VERSION, SCALE_LAYOUT_CODES, SCALE_LAYOUT_NAMES, LinearOperandState,
                     Orientation, ScaleLayout, flattened_matrix_shape, reject_packed_dtype_conversion,
                     scales_mma128_to_row_major, scales_row_major_to_mma128)
from .mxfp8 import (MXFP8Tensor, MXTensor, convert_mxfp8_scale_layout, make_mxfp8_tensor, mxfp8_matrix_shape,
                    mxfp8_qdata_2d, mxfp8_scale_layout, mxfp8_scales_for_kernel, validate_mxfp8_tensor)
from .nvfp4 import (NVFP4Tensor, make_nvfp4_tensor, nvfp4_matrix_shape, nvfp4_qdata_2d, nvfp4_scale_layout,
                    nvfp4_scales_for_kernel, nvfp4_storage_k, validate_nvfp4_tensor)

__all__ = [n for n in dir() if not n.startswith("_")]
