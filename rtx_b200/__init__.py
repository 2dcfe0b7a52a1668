"""rtx_b200 — the block-scaled quantize+GEMM path of `rtx` for NVIDIA B200 (sm_100a).

Same public names as the reference package (rtx/__init__.py:6-91), restricted to the
hot path; attributes are resolved lazily so that importing the package touches
neither CUDA nor the native library.
"""

from ._version import __version__

_LAZY_EXPORTS = {
    "MXTensor": ("formats", "MXTensor"),
    "MXFP8Tensor": ("formats", "MXFP8Tensor"),
    "NVFP4Tensor": ("formats", "NVFP4Tensor"),
    "LinearOperandState": ("formats", "LinearOperandState"),
    "AutotuneMode": ("types", "AutotuneMode"),
    "LinearBackend": ("types", "LinearBackend"),
    "MXFP8Backend": ("types", "MXFP8Backend"),
    "NVFP4Backend": ("types", "NVFP4Backend"),
    "NVFP4ScalingMode": ("types", "NVFP4ScalingMode"),
    "MXFP8Linear": ("fp8", "MXFP8Linear"),
    "NVFP4Linear": ("fp4", "NVFP4Linear"),
    "DEFAULT_NVFP4_X_SCALE_REGION_ROWS": ("fp4", "DEFAULT_NVFP4_X_SCALE_REGION_ROWS"),
    "DEFAULT_NVFP4_WEIGHT_SCALE_REGION_ROWS": ("fp4", "DEFAULT_NVFP4_WEIGHT_SCALE_REGION_ROWS"),
    "mxfp8_linear": ("fp8", "mxfp8_linear"),
    "nvfp4_linear": ("fp4", "nvfp4_linear"),
    "quantize_mxfp8": ("fp8", "quantize_mxfp8"),
    "quantize_nvfp4": ("fp4", "quantize_nvfp4"),
    "DEFAULT_MXFP8_INFERENCE_CONFIG": ("configs", "DEFAULT_MXFP8_INFERENCE_CONFIG"),
    "DEFAULT_MXFP8_PREQUANT_CONFIG": ("configs", "DEFAULT_MXFP8_PREQUANT_CONFIG"),
    "MXFP8PrequantConfig": ("configs", "MXFP8PrequantConfig"),
    "MXFP8QuantConfig": ("configs", "MXFP8QuantConfig"),
    "MXFP8GemmConfig": ("configs", "MXFP8GemmConfig"),
    "MXFP8WeightPrequantConfig": ("configs", "MXFP8WeightPrequantConfig"),
    "MXFP8FullyPrequantConfig": ("configs", "MXFP8FullyPrequantConfig"),
    "MXFP8FwdConfig": ("configs", "MXFP8FwdConfig"),
    "MXFP8Problem": ("configs", "MXFP8Problem"),
    "NVFP4ScaleConfig": ("configs", "NVFP4ScaleConfig"),
    "NVFP4DynamicConfig": ("configs", "NVFP4DynamicConfig"),
    "NVFP4GemmConfig": ("configs", "NVFP4GemmConfig"),
    "NVFP4FullyPrequantConfig": ("configs", "NVFP4FullyPrequantConfig"),
    "NVFP4QuantConfig": ("configs", "NVFP4QuantConfig"),
    "NVFP4WeightPrequantConfig": ("configs", "NVFP4WeightPrequantConfig"),
    "NVFP4Problem": ("configs", "NVFP4Problem"),
    "DEFAULT_MXFP8_BWD_CONFIG": ("configs", "DEFAULT_MXFP8_BWD_CONFIG"),
    "DEFAULT_FUSED_MXFP8_BWD_CONFIG": ("configs", "DEFAULT_FUSED_MXFP8_BWD_CONFIG"),
    "MXFP8BwdConfig": ("configs", "MXFP8BwdConfig"),
    "MXFP8BwdMatmulConfig": ("configs", "MXFP8BwdMatmulConfig"),
    "mxfp8_linear_backward": ("fp8_bwd", "mxfp8_linear_backward"),
    "clear_runtime_caches": ("runtime", "clear_runtime_caches"),
    "validate_runtime_environment": ("runtime", "validate_runtime_environment"),
    "MXFP8TrainingConfig": ("ptq", "MXFP8TrainingConfig"),
    "NVFP4TrainingConfig": ("ptq", "NVFP4TrainingConfig"),
    "MXFP8WeightOnlyConfig": ("ptq", "MXFP8WeightOnlyConfig"),
    "NVFP4WeightOnlyConfig": ("ptq", "NVFP4WeightOnlyConfig"),
    "convert_to_mxfp8_training": ("ptq", "convert_to_mxfp8_training"),
    "convert_to_nvfp4_training": ("ptq", "convert_to_nvfp4_training"),
    "quantize_": ("ptq", "quantize_"),
    # sm_100a additions
    "mxfp8_glu_mlp": ("glu", "mxfp8_glu_mlp"),
    "SwiGLU": ("glu", "SwiGLU"),
    "quantized_weight_cache": ("weight_cache", "quantized_weight_cache"),
    "KernelAdapter": ("autotune", "KernelAdapter"),
    "data_parallel_linear_backward": ("parallel", "data_parallel_linear_backward"),
}

__all__ = ["__version__", *_LAZY_EXPORTS]


def __getattr__(name: str):
    try:
        module_name, attr = _LAZY_EXPORTS[name]
    except KeyError:
        raise AttributeError(f"module {__name__!r} has no attribute {name!r}") from None
    from importlib import import_module

    value = getattr(import_module(f".{module_name}", __name__), attr)
    globals()[name] = value
    return value


def __dir__():
    return sorted(__all__)


def install_as_rtx() -> None:
    """Make `import rtx` (and `rtx.fp8`, `rtx.fp4`, `rtx.fp8_bwd`, `rtx.formats`, `rtx.configs`, `rtx.runtime`,
    `rtx.ptq`, `rtx.types`) resolve to this package, for code written against the reference's package
    name, and publish the Inductor launcher registries under the reference's attribute names
    (`torch._rtx_mxfp8_launchers` and friends, rtx/fp8.py:207-230) next to `torch._rtx_b200_launchers`.
    Refuses when a different `rtx` package is already imported: the two cannot both own the `rtx::` ops."""
    import sys
    from importlib import import_module

    this = sys.modules[__name__]
    other = sys.modules.get("rtx")
    if other is not None and other is not this:
        raise RuntimeError("another package named 'rtx' is already imported; rtx_b200 cannot take its name")
    sys.modules["rtx"] = this
    for sub in ("fp8", "fp4", "fp8_bwd", "formats", "configs", "runtime", "ptq", "types", "autotune"):
        sys.modules[f"rtx.{sub}"] = import_module(f".{sub}", __name__)
    import torch

    from . import inductor

    torch._rtx_mxfp8_launchers = inductor.REGISTRIES["mxfp8_fwd"]
    torch._rtx_mxfp8_bwd_launchers = inductor.REGISTRIES["mxfp8_bwd"]
    torch._rtx_nvfp4_launchers = inductor.REGISTRIES["nvfp4_jit_row_region_fwd"]
