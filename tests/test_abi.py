"""The C-ABI library builds without a GPU, loads, and exports every symbol that
include/rtxb.h declares.  No kernel is launched here."""
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "rtxb.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(rtxb_[a-z0-9_]+)\s*\(", text)))


def test_header_symbols_are_exported(native_lib):
    from rtx_b200 import _native

    declared = _declared_symbols()
    assert len(declared) >= 20
    for name in declared:
        assert hasattr(native_lib, name), f"librtxb.so does not export {name}"
        assert name in _native.SIGNATURES, f"{name} has no ctypes signature"
    assert sorted(_native.SIGNATURES) == declared


def test_queries_and_argument_checks(native_lib):
    from rtx_b200 import _native as N

    assert native_lib.rtxb_version() >= 100
    assert native_lib.rtxb_error_string(0) == b"ok"
    assert N.query("rtxb_mxfp8_storage_k", 17) == 32
    assert N.query("rtxb_nvfp4_storage_k", 129) == 160
    assert N.query("rtxb_mxfp8_scale_bytes", 256, 1024, N.SCALE_ROW_MAJOR) == 256 * 32
    assert N.query("rtxb_mxfp8_scale_bytes", 200, 1000, N.SCALE_MMA128) == 2 * 8 * 512
    assert N.query("rtxb_nvfp4_scale_bytes", 128, 256, N.SCALE_MMA128) == 4 * 512
    assert N.query("rtxb_mxfp8_linear_workspace_bytes", 256, 1024, 1024) >= (256 + 1024) * 1024
    # rejected before any CUDA call: null operands, bad layouts, short workspace
    assert native_lib.rtxb_mxfp8_quantize(None, 1, 32, 32, None, None, 0, 1, None) == -1
    assert native_lib.rtxb_mxfp8_quantize(None, 1, 32, 32, None, None, N.SCALE_MMA64, 1, None) == -2
    assert native_lib.rtxb_mxfp8_gemm(None, None, None, None, None, 1, 1, 1, 1, 0, None, None) == -1
    assert native_lib.rtxb_mxfp8_linear_fwd(None, None, None, 8, 8, 32, 1, None, 0, None, None) == -4
    with pytest.raises(N.NativeError, match="workspace"):
        N.call("rtxb_mxfp8_linear_fwd", None, None, None, 8, 8, 32, 1, None, 0, None, None)


def test_missing_library_is_loud(monkeypatch, tmp_path):
    from rtx_b200 import _native as N

    monkeypatch.setattr(N, "_lib", None)
    monkeypatch.setattr(N, "LIB_PATH", str(tmp_path / "absent.so"))
    with pytest.raises(ImportError, match="no CPU or PyTorch fallback"):
        N.load()
