"""Literal types of the public API (same names and values as rtx/types.py:6-23)."""

from typing import Literal

AutotuneMode = Literal["off", "cache", "balanced", "online", "coordinate"]
LinearBackend = Literal["auto", "fused", "materialized"]
MXFP8Backend = LinearBackend
NVFP4Backend = LinearBackend
NVFP4ScalingMode = Literal["current", "block", "jit_row_region", "delayed"]
WeightMode = Literal["dynamic", "prequantized"]
