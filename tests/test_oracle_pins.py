"""Pins the CPU oracle to the reference: every array in tests/golden/ was
produced by executing the reference's own functions (see make_golden.py)."""
import hashlib

import numpy as np
import pytest
import torch

from oracle import mx_oracle as O


def _bf16_from_bits(a: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(a.view(np.int16).copy()).view(torch.bfloat16)


def _bits(t: torch.Tensor) -> np.ndarray:
    return t.contiguous().view(torch.int16).numpy().view(np.uint16)


def _canon_nan(q: np.ndarray) -> np.ndarray:
    """E4M3 has two NaN codes (0x7F, 0xFF); the sign of a NaN is not part of the contract
    (x86 arithmetic yields the negative one, the PTX converter the positive one)."""
    q = q.copy()
    q[(q & 0x7F) == 0x7F] = 0x7F
    return q


def _sha(t: torch.Tensor) -> str:
    return hashlib.sha256(_bits(t).tobytes()).hexdigest()


def test_known_answer_480(golden):
    """tests/test_mxfp8_quant.py:186-220: 480 -> |q| 448 / code 127 (floor), 240 / code 128 (infinity)."""
    arrays, _ = golden
    src = torch.zeros(1, 32)
    src[0, 0] = 480
    for rounding, want_max, want_code in (("floor", 448.0, 127), ("infinity", 240.0, 128)):
        q, s = O.mxfp8_quantize(src.bfloat16(), rounding)
        assert O.e4m3_decode(q).abs().max().item() == want_max
        assert int(s[0, 0]) == want_code
        assert np.array_equal(q.numpy(), arrays[f"ka480_{rounding}_q"])
        assert np.array_equal(s.numpy(), arrays[f"ka480_{rounding}_s"])


@pytest.mark.parametrize("name", ["q1701", "q1703", "qrag", "qtiny", "q33", "special"])
@pytest.mark.parametrize("rounding", ["infinity", "floor"])
def test_quantizer_matches_reference_bytes(golden, name, rounding):
    arrays, _ = golden
    x = _bf16_from_bits(arrays[f"{name}_x"])
    q, s = O.mxfp8_quantize(x, rounding)
    assert np.array_equal(_canon_nan(q.numpy()), _canon_nan(arrays[f"{name}_{rounding}_q"]))
    assert np.array_equal(s.numpy(), arrays[f"{name}_{rounding}_s"])


def test_golden_inputs_regenerate_from_seeds(golden):
    arrays, manifest = golden
    for name in ("q1701", "q1703", "qrag"):
        torch.manual_seed(manifest[name]["seed"])
        x = torch.randn(*manifest[name]["shape"]).bfloat16()
        assert np.array_equal(_bits(x), arrays[f"{name}_x"])


@pytest.mark.parametrize("mnk", [(128, 128, 128), (37, 70, 128), (5, 129, 256), (3, 5, 1), (7, 11, 17), (9, 131, 127)])
def test_forward_matches_reference_bits(golden, mnk):
    """tests/test_mxfp8_fwd.py:359-380 shapes, rtol=0 atol=0 against the reference's `_reference_linear`."""
    arrays, _ = golden
    m, n, k = mnk
    torch.manual_seed(123)
    x = (torch.randn(m, k) * 0.5).bfloat16()
    w = (torch.randn(n, k) * 0.5).bfloat16()
    assert np.array_equal(_bits(O.mxfp8_linear(x, w)), arrays[f"fwd_{m}_{n}_{k}_y"])


def test_forward_digests(golden):
    arrays, manifest = golden
    torch.manual_seed(321)
    x = (torch.randn(257, 256) * 0.5).bfloat16()
    w = (torch.randn(385, 256) * 0.5).bfloat16()
    assert _sha(O.mxfp8_linear(x, w)) == manifest["fwd_257_385_256"]["sha256_y"]
    inp = O.make_inputs(1)
    y = O.mxfp8_linear(inp["x"], inp["w"])
    assert np.array_equal(_bits(y[:16, :16].contiguous()), arrays["config1_y_corner"])
    assert _sha(y) == manifest["config1"]["sha256_y"]


def test_e4m3_codec_against_torch_cast():
    codes = torch.arange(256, dtype=torch.uint8)
    want = codes.view(torch.float8_e4m3fn).float()
    got = O.e4m3_decode(codes)
    assert torch.equal(torch.nan_to_num(got, nan=-1.0), torch.nan_to_num(want, nan=-1.0))
    finite = want[~want.isnan()].sort().values
    mids = (finite[1:] + finite[:-1]) / 2
    g = torch.Generator().manual_seed(3)
    v = torch.cat([mids, finite, torch.randn(100000, generator=g) * 30, torch.randn(100000, generator=g) * 0.01])
    v = v.clamp(-448, 448)
    assert torch.equal(O.e4m3_encode(v), v.to(torch.float8_e4m3fn).view(torch.uint8))
    assert int(O.e4m3_encode(torch.tensor([1e9]))[0]) == 0x7E
    assert int(O.e4m3_encode(torch.tensor([float("nan")]))[0]) == 0x7F


def test_e2m1_codec_round_trip_and_ties():
    codes = torch.arange(16, dtype=torch.uint8)
    assert torch.equal(O.e2m1_encode(O.e2m1_decode(codes)) & 0x7, codes & 0x7)
    ties = torch.tensor([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 7.0, -0.25, -5.0])
    assert O.e2m1_encode(ties).tolist() == [0, 2, 2, 4, 4, 6, 6, 7, 8, 14]


def test_scale_layout_formula():
    """tests/test_mxfp8_quant.py:108-120: physical = (row%32)*16 + ((row//32)%4)*4 + block%4."""
    s = (torch.arange(256 * 8) % 251).to(torch.uint8).reshape(256, 8)
    tiles = O.scales_to_mma128(s)
    assert tiles.shape == (2, 2, 512)
    for row, blk in [(0, 0), (33, 5), (127, 3), (128, 4), (255, 7)]:
        phys = (row % 32) * 16 + ((row // 32) % 4) * 4 + blk % 4
        assert tiles[row // 128, blk // 4, phys] == s[row, blk]
    assert torch.equal(O.scales_from_mma128(tiles, 256, 8), s)


def test_transposed_quant_is_quant_of_transpose():
    """tests/test_mxfp8_bwd.py:695-730."""
    torch.manual_seed(5)
    x = torch.randn(96, 40).bfloat16()
    q, s = O.mxfp8_quantize_transposed(x)
    q2, s2 = O.mxfp8_quantize(x.t().contiguous())
    assert torch.equal(q, q2) and torch.equal(s, s2)
    assert q.shape == (40, 96)


def test_nvfp4_internal_consistency():
    """NVFP4 parity is unpinned (no TorchAO here); check the restatement's invariants:
    storage K (rtx tests/test_nvfp4.py:222-229), scale rules, dequantisation error."""
    assert [O.nvfp4_storage_k(k) for k in (17, 129, 144, 145)] == [32, 160, 160, 160]
    torch.manual_seed(1907)
    x = torch.randn(128, 128).bfloat16()
    st = O.nvfp4_tensor_scale(x, "exact")
    assert torch.equal(st, (x.float().abs().amax() / 2688.0).reshape(1))
    p2 = O.nvfp4_tensor_scale(x, "power2")
    assert float(torch.log2(p2)) == round(float(torch.log2(p2))) and p2 >= st and p2 < 2 * st
    assert float(O.nvfp4_tensor_scale(torch.zeros(4, 32), "power2")) == 1.0
    assert float(O.nvfp4_tensor_scale(x, "block")) == 1.0
    q, sb = O.nvfp4_quantize(x, st)
    assert q.shape == (128, 64) and sb.shape == (128, 8) and q.dtype == torch.uint8
    deq = O.nvfp4_dequantize(q, sb, st)
    rel = ((deq - x.float()).norm() / x.float().norm()).item()
    assert rel < 0.12
    # the block holding the tensor amax uses the top of both ranges: scale 448, payload +-6
    r, c = divmod(int(x.float().abs().argmax()), 128)
    assert int(sb[r, c // 16]) == 0x7E
    nib = (int(q[r, c // 2]) >> (4 * (c % 2))) & 0x7
    assert nib == 7


def test_glu_and_backward_shapes():
    torch.manual_seed(0)
    x = torch.randn(64, 96).bfloat16()
    wgu = (torch.randn(256, 96) / 10).bfloat16()
    wd = (torch.randn(80, 128) / 11).bfloat16()
    h, y = O.mxfp8_glu_mlp(x, wgu, wd)
    h2, _ = O.mxfp8_glu_mlp(x, wgu, wd, fused_rounding=False)
    assert h.shape == (64, 128) and y.shape == (64, 80)
    assert (O.bf16_ulp_distance(h, h2) <= 2).float().mean() > 0.95
    dy = (torch.randn(64, 256) * 0.1).bfloat16()
    dx, dw = O.mxfp8_backward(x, wgu, dy)
    assert dx.shape == (64, 96) and dw.shape == (256, 96)
    ref_dx = dy.float() @ wgu.float()
    assert ((dx.float() - ref_dx).norm() / ref_dx.norm()) < 0.07


def test_cpu_baseline_path_equals_oracle():
    """The timed CPU baseline (oracle/cpu_path.py) computes the same bits as the pinned oracle."""
    from oracle import cpu_path as C

    torch.manual_seed(11)
    x = torch.randn(96, 200).bfloat16()
    wgu = (torch.randn(256, 200) / 14).bfloat16()
    wd = (torch.randn(72, 128) / 11).bfloat16()
    q, s = C.mx_quantize(x)
    qo, so = O.mxfp8_quantize(x)
    assert torch.equal(q.view(torch.uint8), qo) and torch.equal(s, so)
    h, y = C.mx_glu_mlp(x, wgu, wd)
    ho, yo = O.mxfp8_glu_mlp(x, wgu, wd)
    assert torch.equal(h, ho) and torch.equal(y, yo)


def test_nvfp4_row_region_oracle_is_consistent():
    """Row-region policy restated from the reference (unpinned like the rest of NVFP4): a single region
    over the tensor is the `current` policy, regions are quantized independently, and the region-size
    fallback follows rtx/fp4.py:89-94."""
    torch.manual_seed(11)
    x = (torch.randn(40, 128) * torch.logspace(-2, 2, 40).unsqueeze(1)).bfloat16()
    w = torch.randn(32, 128).bfloat16()
    assert O.nvfp4_effective_region_rows(40, 5) == 5 and O.nvfp4_effective_region_rows(16384, 5) == 16384
    assert O.nvfp4_effective_region_rows(4, 4) == 4 and O.nvfp4_effective_region_rows(28672, 4) == 4
    assert torch.equal(O.nvfp4_linear_regions(x, w, 40, 32), O.nvfp4_linear(x, w))
    scales = O.nvfp4_region_scales(x, 5)
    assert scales.shape == (8,) and scales[0] < scales[-1]
    assert torch.equal(scales[3:4], O.nvfp4_tensor_scale(x[15:20]))
    q, s = O.nvfp4_quantize_regions(x, scales, 5)
    q3, s3 = O.nvfp4_quantize(x[15:20], scales[3:4])
    assert torch.equal(q[15:20], q3) and torch.equal(s[15:20], s3)
    # regional scales track the local range: closer to the FP32 product than one scale for the tensor
    ref = x.float() @ w.float().t()
    err_region = (O.nvfp4_linear_regions(x, w, 5, 4).float() - ref).norm()
    err_tensor = (O.nvfp4_linear(x, w).float() - ref).norm()
    assert err_region <= err_tensor


# ----------------------------------------------------------------------------- NVFP4 outer scale

def _outer_scale_fixture():
    import json
    import os

    here = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
    arrays = np.load(os.path.join(here, "nvfp4_outer_scale.npz"))
    with open(os.path.join(here, "nvfp4_outer_scale.json")) as f:
        return arrays, json.load(f)


@pytest.mark.parametrize("mode", ["exact", "power2"])
def test_nvfp4_outer_scale_matches_reference_on_every_bf16_magnitude(mode):
    """rtx/fp4.py:343-365 executed on every non-negative BF16 bit pattern (zero, subnormals, +inf)
    and NaN; the oracle's rule (division form) must give the same FP32 bits on all of them."""
    arrays, meta = _outer_scale_fixture()
    assert meta["bf16_inputs_where_integer_rule_differs"] == []
    bf16_bits = arrays["bf16_bits"].astype(np.int64)
    amax = torch.from_numpy((bf16_bits << 16).astype(np.uint32).view(np.float32).copy())
    want = arrays[f"{mode}_scale_bits"]
    assert len(want) == 0x7F81 + 1
    got = np.array([O.nvfp4_scale_rule(a, mode).view(torch.int32).item() & 0xFFFFFFFF for a in amax], dtype=np.uint32)
    bad = np.nonzero(got != want)[0]
    assert bad.size == 0, [(hex(int(bf16_bits[i])), hex(int(got[i])), hex(int(want[i]))) for i in bad[:8]]
    # zero and NaN decode to 1.0
    one = np.float32(1.0).view(np.uint32)
    assert want[0] == one and want[-1] == one


def test_nvfp4_outer_scale_fp32_probes_list_the_known_deviation():
    """On FP32 |max| values one ulp above 2688 * 2^e (never produced by a BF16 tensor) the kernels'
    exponent-bump rule doubles the scale where exp2(ceil(log2(t))) rounds the logarithm down to an
    integer.  The fixture lists those inputs; the oracle reproduces the integer rule on them and
    the reference's bits everywhere else."""
    arrays, meta = _outer_scale_fixture()
    probes = torch.from_numpy(arrays["fp32_probe_bits"].view(np.float32).copy())
    ref = arrays["fp32_probe_power2_scale_bits"]
    listed = {e["amax_bits"]: e for e in meta["fp32_probes_where_integer_rule_differs"]}
    assert 0 < len(listed) < len(probes)
    for a, r in zip(probes, ref):
        got = O.nvfp4_scale_rule(a, "power2").view(torch.int32).item() & 0xFFFFFFFF
        key = int(a.view(torch.int32).item()) & 0xFFFFFFFF
        if key in listed:
            assert got == listed[key]["integer_rule_scale_bits"] == listed[key]["reference_scale_bits"] + (1 << 23)
        else:
            assert got == int(r)


def test_nvfp4_kernel_form_quotient_differs_only_in_exact_mode():
    """amax * Float32(1/2688) (quantizer kernels) against amax / 2688 (PyTorch functions): the power
    of two is the same on every BF16 magnitude, the exact scale is not."""
    arrays, _ = _outer_scale_fixture()
    bits = arrays["bf16_bits"].astype(np.int64)[1:0x7F80]
    amax = torch.from_numpy((bits << 16).astype(np.uint32).view(np.float32).copy())
    step = 7   # a thinned sweep keeps the CPU suite short; the exhaustive division-form sweep is above
    p2_t = [O.nvfp4_scale_rule(a, "power2", "torch").item() for a in amax[::step]]
    p2_k = [O.nvfp4_scale_rule(a, "power2", "kernel").item() for a in amax[::step]]
    assert p2_t == p2_k
    ex_t = torch.cat([O.nvfp4_scale_rule(a, "exact", "torch") for a in amax[::step]])
    ex_k = torch.cat([O.nvfp4_scale_rule(a, "exact", "kernel") for a in amax[::step]])
    normal = ex_t >= 2.0 ** -126
    assert (ex_t != ex_k).any() and ((ex_t - ex_k).abs()[normal] <= ex_t[normal] * 2.0 ** -22).all()
