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


def test_newer_entry_points_reject_bad_arguments_before_any_launch(native_lib):
    """Decode, row-region, delayed, dual-quantize and SM-margin entry points: every rejection below happens
    in host code, so it can be checked without a GPU."""
    import ctypes

    from rtx_b200 import _native as N

    L = native_lib
    buf = (ctypes.c_uint8 * 4096)()
    p = ctypes.addressof(buf) + (16 - ctypes.addressof(buf) % 16) % 16      # any 16-byte aligned non-null address
    assert L.rtxb_nvfp4_quantize_dynamic(None, 1, 32, 32, 1, None, None, 2, None, None, None, None, None) == -1
    assert L.rtxb_nvfp4_quantize_dynamic(p, 1, 32, 16, 1, p, p, 2, p, None, None, p, None) == -1      # ld < k
    assert L.rtxb_nvfp4_quantize_dynamic(p, 1, 32, 32, 7, p, p, 2, p, None, None, p, None) == -1      # scale mode
    assert L.rtxb_nvfp4_quantize_dynamic(p, 1, 32, 32, 1, p, p, 2, p, p, None, p, None) == -1         # scales go together
    assert L.rtxb_nvfp4_linear_fwd_prequant_w(p, p, p, None, p, 1, 64, 256, 0, p, 1 << 20, None, None) == -1
    assert L.rtxb_nvfp4_linear_fwd_prequant_w(p, p, p, p, p, 1, 64, 256, 0, None, 0, None, None) == -4
    assert N.query("rtxb_nvfp4_linear_prequant_w_workspace_bytes", 8, 8192) >= 8 * 4096
    # regions must divide the rows; a single region needs the scratch word
    assert L.rtxb_nvfp4_region_scales(p, 10, 32, 32, 4, 1, p, p, None) == -1
    assert L.rtxb_nvfp4_region_scales(p, 10, 32, 32, 10, 1, None, p, None) == -1
    assert L.rtxb_nvfp4_quantize_regions(p, 10, 32, 32, p, p, 2, None, 5, None) == -1
    assert L.rtxb_nvfp4_quantize_regions(p, 10, 32, 32, p, p, N.SCALE_MMA64, p, 5, None) == -2
    assert L.rtxb_nvfp4_gemm_regions(p, p, p, p, p, 10, 8, 32, 8, p, 3, p, 4, None, None) == -1      # 3 does not divide 10
    ws = N.query("rtxb_nvfp4_linear_regions_workspace_bytes", 256, 512, 256, 5, 4)
    assert ws >= 256 * 128 + 512 * 128
    assert L.rtxb_nvfp4_linear_fwd_regions(p, p, p, 256, 512, 256, 5, 4, 1, p, ws - 1, None, None) == -4
    # delayed: history length 1/4/16/64, two distinct generations
    assert L.rtxb_nvfp4_quantize_delayed(p, 1, 32, 32, p, p, 2, p, p + 256, 5, 1, 1, p, None, None, None) == -1
    assert L.rtxb_nvfp4_quantize_delayed(p, 1, 32, 32, p, p, 2, p, p, 4, 1, 1, p, None, None, None) == -1
    assert L.rtxb_nvfp4_linear_fwd_delayed(p, p, p, 8, 8, 32, p, p, p, p, 4, 1, 1, None, 0, None, None) == -4
    # dual quantizer
    assert L.rtxb_mxfp8_quantize_dual(p, 4, 32, 32, p, p, None, p, 2, 1, None) == -1
    assert L.rtxb_mxfp8_quantize_dual(p, 4, 32, 16, p, p, p, p, 2, 1, None) == -1
    assert L.rtxb_mxfp8_quantize_dual(p, 4, 32, 32, p, p, p, p, N.SCALE_MMA64, 1, None) == -2
    # SM margin: process-wide setting with a sane range
    assert L.rtxb_get_sm_margin() == 0
    assert L.rtxb_set_sm_margin(32) == 0 and L.rtxb_get_sm_margin() == 32
    assert L.rtxb_set_sm_margin(-1) == -1 and L.rtxb_set_sm_margin(1000) == -1 and L.rtxb_get_sm_margin() == 32
    assert L.rtxb_set_sm_margin(0) == 0
    # the GEMM schedule switch is per thread and refuses unknown schedules
    assert L.rtxb_get_gemm_schedule() == 0
    for code in (1, 2, 3):
        assert L.rtxb_set_gemm_schedule(code) == 0 and L.rtxb_get_gemm_schedule() == code
    assert L.rtxb_set_gemm_schedule(5) == -1 and L.rtxb_set_gemm_schedule(-1) == -1
    assert L.rtxb_get_gemm_schedule() == 3
    import threading
    seen = []
    worker = threading.Thread(target=lambda: seen.append(L.rtxb_get_gemm_schedule()))
    worker.start()
    worker.join()
    assert seen == [0]
    assert L.rtxb_set_gemm_schedule(0) == 0
    # the multi-GPU helpers refuse bad arguments before anything is launched
    import ctypes

    one = (ctypes.c_void_p * 1)(ctypes.c_void_p(0x1000))
    word = ctypes.c_void_p(0x2000)
    assert L.rtxb_peer_barrier(None, 1, 0, word, 2_000_000, None, None) == -1          # no flag arrays
    assert L.rtxb_peer_barrier(one, 9, 0, word, 2_000_000, None, None) == -1           # more than eight ranks
    assert L.rtxb_peer_barrier(one, 1, 1, word, 2_000_000, None, None) == -1           # rank outside the group
    assert L.rtxb_peer_barrier(one, 1, 0, None, 2_000_000, None, None) == -1           # no epoch counter
    assert L.rtxb_peer_barrier(one, 1, 0, word, 10, None, None) == -1                  # limit below 1 ms
    assert L.rtxb_selftest_wait_timeout(10, None, word, None) == -1
    assert L.rtxb_selftest_wait_timeout(20_000_000, None, None, None) == -1            # reports through the status word


def test_missing_library_is_loud(monkeypatch, tmp_path):
    from rtx_b200 import _native as N

    monkeypatch.setattr(N, "_lib", None)
    monkeypatch.setattr(N, "LIB_PATH", str(tmp_path / "absent.so"))
    with pytest.raises(ImportError, match="no CPU or PyTorch fallback"):
        N.load()


def test_device_status_codes_agree_between_header_kernels_and_python():
    """RTXB_DEV_* in the header, the DeviceStatus enum the kernels store, and the names Python reports."""
    from rtx_b200 import _native

    header = open(os.path.join(ROOT, "include", "rtxb.h")).read()
    macros = {name: int(v) for name, v in re.findall(r"#define (RTXB_DEV_[A-Z_]+) (\d+)", header)}
    device = open(os.path.join(ROOT, "rtx_b200", "csrc", "common.cuh")).read()
    enum = {name: int(v) for name, v in re.findall(r"(kStatus[A-Za-z]+) = (\d+)", device)}
    assert sorted(macros.values()) == sorted(enum.values()) == sorted(_native.DEVICE_STATUS_NAMES)
    assert macros["RTXB_DEV_WAIT_SELFTEST"] == enum["kStatusWaitSelfTest"] == 5
    assert macros["RTXB_DEV_WAIT_QUANT"] == enum["kStatusWaitQuant"]
