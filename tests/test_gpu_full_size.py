"""Parity at the benchmark configurations' real sizes (3: NVFP4 forward 16384 x 28672 x 8192;
4: MXFP8 backward 16384 x 4096 x 4096; 5: NVFP4 decode, N in {8192, 28672}, K = 8192), the NVFP4
outer scale against the bits of the reference's own PyTorch functions, and the TorchAO byte
comparison the reference's test suite holds (skipped where TorchAO is not installed).

The CPU oracle cannot finish these sizes in seconds, so the checks are the size-independent
ones: sampled rows of every quantized payload against the oracle (bit exact), output tiles
from the first / middle / last tile rows and columns against an FP32 matmul of the operands
dequantised on the device with plain torch ops (the output bar: rel-Frobenius <= 1e-3 and
<= 1 BF16 ulp on >= 99.9 %), and column sums over the whole output (linearity)."""
import json
import os

import numpy as np
import pytest
import torch

from oracle import mx_oracle as O

pytestmark = pytest.mark.gpu

REL_FRO_MAX = 1e-3
FRAC_1ULP_MIN = 0.999
GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


@pytest.fixture(scope="module")
def gpu(native_lib):
    if not torch.cuda.is_available():
        pytest.fail("these tests need a CUDA device")
    from rtx_b200 import _native as N
    from rtx_b200 import ops

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    torch.backends.cuda.matmul.allow_tf32 = False   # the checker's matmuls are true FP32
    return ops, N, dev, ops.Workspace(dev)


def _ok(ops, dev):
    torch.cuda.synchronize()
    ops.check_device_status(dev)


def _assert_output(got, want):
    rep = O.parity_report(got.cpu(), want.cpu())
    assert rep["rel_fro"] <= REL_FRO_MAX and rep["frac_le_1ulp"] >= FRAC_1ULP_MIN, rep


def _tile_index(rows, nb, chunks, dev):
    r = torch.arange(rows, device=dev).unsqueeze(1)
    b = torch.arange(nb, device=dev).unsqueeze(0)
    return (((r // 128) * chunks + b // 4) * 512 + (r % 32) * 16 + ((r // 32) % 4) * 4 + b % 4).reshape(-1)


def _deq_mx(q, s_tiles, rows, k):
    """MXFP8 payload + mma128 E8M0 tiles -> FP32 [rows, Kp] on the device (checker only)."""
    nb = (k + 31) // 32
    codes = s_tiles[_tile_index(rows, nb, (nb + 3) // 4, q.device)].reshape(rows, nb).to(torch.int32)
    scale = (codes.clamp(min=1) << 23).view(torch.float32)
    return q.view(torch.float8_e4m3fn).float() * scale.repeat_interleave(32, dim=1)


_E2M1 = [0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0, -0.0, -0.5, -1.0, -1.5, -2.0, -3.0, -4.0, -6.0]


def _deq_nv(q, s_tiles, rows, k, row_slice=None):
    """NVFP4 payload + mma128 E4M3 tiles -> FP32 [rows, Kp] WITHOUT the outer scale (checker only)."""
    kp = (k + 31) // 32 * 32
    nb = kp // 16
    chunks = ((nb + 3) // 4 + 3) // 4 * 4
    idx = _tile_index(rows, nb, chunks, q.device).reshape(rows, nb)
    if row_slice is not None:
        idx, q = idx[row_slice], q[row_slice]
    sb = s_tiles[idx.reshape(-1)].reshape(-1, nb).view(torch.float8_e4m3fn).float()
    lut = torch.tensor(_E2M1, device=q.device)
    vals = torch.stack([lut[(q & 0xF).long()], lut[(q >> 4).long()]], dim=-1).reshape(q.shape[0], kp)
    return vals * sb.repeat_interleave(16, dim=1)


# ----------------------------------------------------------------------------- NVFP4 outer scale

def _outer_scale_fixture():
    arrays = np.load(os.path.join(GOLDEN, "nvfp4_outer_scale.npz"))
    with open(os.path.join(GOLDEN, "nvfp4_outer_scale.json")) as f:
        return arrays, json.load(f)


@pytest.mark.parametrize("mode", ["exact", "power2"])
def test_nvfp4_tensor_scale_matches_reference_bits(gpu, mode):
    """rtxb_nvfp4_tensor_scale against the output of rtx/fp4.py:343-365 (executed to make the
    fixture): every BF16 magnitude whose quotient by 2688 is a power of two (mantissa 0x28) with
    its two neighbours, zero, the smallest and largest subnormals and normals, +inf, NaN, and a
    seeded sample of the rest."""
    ops, N, dev, _ = gpu
    arrays, _ = _outer_scale_fixture()
    bf16_bits = arrays["bf16_bits"].astype(np.int64)
    want = arrays[f"{mode}_scale_bits"]
    pick = {0, 1, 2, 0x7F, 0x80, 0x81, 0x7F7F, 0x7F80, len(bf16_bits) - 1}
    for i in range(len(bf16_bits) - 1):
        if (bf16_bits[i] & 0x7F) == 0x28:
            pick.update({i - 1, i, i + 1})
    rng = np.random.default_rng(5)
    pick.update(int(i) for i in rng.integers(0, len(bf16_bits) - 1, 150))
    code = N.TENSOR_SCALE_EXACT if mode == "exact" else N.TENSOR_SCALE_POWER2
    bad = []
    for i in sorted(pick):
        x = torch.zeros(4, 64, dtype=torch.int16)
        x[2, 17] = int(np.array(bf16_bits[i], dtype=np.uint16).view(np.int16))
        st = ops.nvfp4_tensor_scale(x.view(torch.bfloat16).to(dev), code)
        got = int(st.cpu().view(torch.int32).item()) & 0xFFFFFFFF
        if got != int(want[i]):
            bad.append((hex(int(bf16_bits[i])), hex(got), hex(int(want[i]))))
    _ok(ops, dev)
    assert not bad, bad[:8]


@pytest.mark.parametrize("mode", ["exact", "power2"])
def test_nvfp4_region_scales_on_every_bf16_magnitude(gpu, mode):
    """One launch, one region per BF16 magnitude.  The row-region kernels form amax * (1/2688) as the
    reference's quantizer kernels do (rtx/kernels/nvfp4_quant.py:117-143): bit-equal to the oracle's
    kernel form everywhere, and in power-of-two mode also to the reference's PyTorch bits."""
    ops, N, dev, _ = gpu
    arrays, _ = _outer_scale_fixture()
    bf16_bits = arrays["bf16_bits"][:-1]          # finite and +inf; NaN is checked below
    rows = len(bf16_bits)
    x = torch.zeros(rows, 32, dtype=torch.int16)
    x[:, 5] = torch.from_numpy(bf16_bits.view(np.int16).copy())
    code = N.TENSOR_SCALE_EXACT if mode == "exact" else N.TENSOR_SCALE_POWER2
    got = ops.nvfp4_region_scales(x.view(torch.bfloat16).to(dev), 1, code)
    _ok(ops, dev)
    got = got.cpu().view(torch.int32).numpy().view(np.uint32)
    amax = (bf16_bits.astype(np.uint32) << 16).view(np.float32)
    recip = np.float32(1.0 / 2688.0)
    with np.errstate(over="ignore"):
        quotient = (amax * recip).astype(np.float32)
    if mode == "exact":
        want = quotient.view(np.uint32).copy()
    else:
        b = np.maximum(quotient, np.float32(2.0 ** -126)).view(np.uint32)
        e = b & np.uint32(0x7F800000)
        want = np.where((b & np.uint32(0x7FFFFF)) != 0, e + np.uint32(1 << 23), e).astype(np.uint32)
        assert np.array_equal(want[1:], arrays["power2_scale_bits"][1:-1])
    want[0] = np.float32(1.0).view(np.uint32)
    assert np.array_equal(got, want)
    nan = torch.zeros(2, 32, dtype=torch.bfloat16)
    nan[1, 3] = float("nan")
    got = ops.nvfp4_region_scales(nan.to(dev), 1, code).cpu()
    assert got.tolist() == [1.0, 1.0]


def test_nvfp4_payload_matches_torchao_when_installed(gpu):
    """The reference's own pin (tests/test_nvfp4.py:724-755): 128 x 128 randn, seed 1907, exact outer
    scale amax / 2688; payload bytes and E4M3 block scales equal NVFP4Tensor.to_nvfp4 bit for bit.
    Runs only where TorchAO is installed (it is the reference's dependency, not this library's)."""
    pytest.importorskip("torchao")
    from torchao.prototype.mx_formats.nvfp4_tensor import NVFP4Tensor

    ops, N, dev, _ = gpu
    torch.manual_seed(1907)
    x = torch.randn(128, 128, device=dev, dtype=torch.bfloat16)
    scale = x.float().abs().amax() / 2688.0
    q, s = ops.nvfp4_quantize(x, scale.reshape(1), layout=N.SCALE_ROW_MAJOR)
    _ok(ops, dev)
    ao = NVFP4Tensor.to_nvfp4(x, block_size=16, per_tensor_scale=scale, use_triton_kernel=False)
    assert torch.equal(q.view(torch.uint8).reshape(128, 64), ao.qdata.view(torch.uint8).reshape(128, 64))
    assert torch.equal(s.reshape(128, 8).view(torch.float8_e4m3fn).float(), ao.scale.float().reshape(128, 8))


# ----------------------------------------------------------------------------- configuration 3

def test_full_size_config3_nvfp4_forward(gpu):
    ops, N, dev, ws = gpu
    inp = O.make_inputs(3)
    x, w = inp["x"], inp["w"]
    m, k = x.shape
    n = w.shape[0]
    xd, wd = x.to(dev), w.to(dev)
    sx_t, sw_t = (ops.nvfp4_tensor_scale(t, N.TENSOR_SCALE_POWER2) for t in (xd, wd))
    _ok(ops, dev)
    assert torch.equal(sx_t.cpu(), O.nvfp4_tensor_scale(x, "power2"))
    assert torch.equal(sw_t.cpu(), O.nvfp4_tensor_scale(w, "power2"))
    qx, sx = ops.nvfp4_quantize(xd, sx_t)
    qw, sw = ops.nvfp4_quantize(wd, sw_t)
    _ok(ops, dev)
    # sampled payload rows and their block scales against the oracle
    for t, q, s, st, rows in ((x, qx, sx, sx_t, m), (w, qw, sw, sw_t, n)):
        nb = k // 16
        idx = _tile_index(rows, nb, ((nb + 3) // 4 + 3) // 4 * 4, dev).reshape(rows, nb)
        for r0 in (0, rows // 2 - 32, rows - 64):
            qo, so = O.nvfp4_quantize(t[r0:r0 + 64], st.cpu())
            assert torch.equal(q[r0:r0 + 64].cpu(), qo)
            assert torch.equal(s[idx[r0:r0 + 64].reshape(-1)].reshape(64, nb).cpu(), so)
    y = ops.nvfp4_linear_fwd(xd, wd, ws, scale_mode=N.TENSOR_SCALE_POWER2)
    _ok(ops, dev)
    out_scale = (sx_t * sw_t).reshape(())
    for r0 in (0, m // 2 - 128, m - 256):
        dx = _deq_nv(qx, sx, m, k, slice(r0, r0 + 256))
        for c0 in (0, n // 2 - 128, n - 256):
            dwt = _deq_nv(qw, sw, n, k, slice(c0, c0 + 256))
            want = ((dx @ dwt.t()) * out_scale).bfloat16()
            _assert_output(y[r0:r0 + 256, c0:c0 + 256].contiguous(), want)
    # linearity over the whole output: column sums of the FP32-output GEMM
    one = torch.ones(1, device=dev)
    y32 = ops.nvfp4_gemm(qx, sx, qw, sw, m, n, k, one, out_dtype=torch.float32)
    _ok(ops, dev)
    got = y32.double().sum(dim=0)
    del y32
    col = torch.zeros(k, dtype=torch.float64, device=dev)
    for r0 in range(0, m, 2048):
        col += _deq_nv(qx, sx, m, k, slice(r0, r0 + 2048)).double().sum(dim=0)
    want = torch.cat([_deq_nv(qw, sw, n, k, slice(c0, c0 + 2048)).double() @ col for c0 in range(0, n, 2048)])
    assert ((got - want).norm() / want.norm()) < 1e-5
    # the default policy (row regions) and the delayed policy at the same size: same tiles, looser only in
    # that their outer scales differ per region / come from the history
    y_regions = ops.nvfp4_linear_fwd_regions(xd, wd, ws, 8, 4)
    _ok(ops, dev)
    xs = ops.nvfp4_region_scales(xd, 8)
    wsc = ops.nvfp4_region_scales(wd, 4)
    qxr, sxr = ops.nvfp4_quantize_regions(xd, xs, 8)
    qwr, swr = ops.nvfp4_quantize_regions(wd, wsc, 4)
    _ok(ops, dev)
    r0, c0 = m - 256, n // 2 - 128
    acc = _deq_nv(qxr, sxr, m, k, slice(r0, r0 + 256)) @ _deq_nv(qwr, swr, n, k, slice(c0, c0 + 256)).t()
    factor = xs[r0 // 8:(r0 + 256) // 8].repeat_interleave(8).unsqueeze(1) * \
        wsc[c0 // 4:(c0 + 256) // 4].repeat_interleave(4).unsqueeze(0)
    _assert_output(y_regions[r0:r0 + 256, c0:c0 + 256].contiguous(), (acc * factor).bfloat16())


# ----------------------------------------------------------------------------- configuration 4

@pytest.mark.parametrize("dw_dtype", [torch.float32, torch.bfloat16])
def test_full_size_config4_mxfp8_backward(gpu, dw_dtype):
    ops, N, dev, ws = gpu
    inp = O.make_inputs(4)
    x, w, dy = inp["x"], inp["w"], inp["dy"]
    m, k = x.shape
    n = w.shape[0]
    xd, wd, dyd = x.to(dev), w.to(dev), dy.to(dev)
    dx, dw = ops.mxfp8_linear_bwd(dyd, xd, wd, ws, dw_dtype=dw_dtype)
    _ok(ops, dev)
    # the four operands as the backward quantizes them
    qa, sa, qc, sc = ops.mxfp8_quantize_dual(dyd)            # dY rows (along N), dY^T (along M)
    qb, sb = ops.mxfp8_quantize_transposed(wd)               # W^T [K, N], blocks along N
    qd, sd = ops.mxfp8_quantize_transposed(xd)               # X^T [K, M], blocks along M
    _ok(ops, dev)
    for r0 in (0, m // 2, m - 64):
        qo, _ = O.mxfp8_quantize(dy[r0:r0 + 64])
        assert torch.equal(qa[r0:r0 + 64].cpu(), qo)
    for c0 in (0, n // 2, n - 64):
        qo, _ = O.mxfp8_quantize(dy[:, c0:c0 + 64].t().contiguous())
        assert torch.equal(qc[c0:c0 + 64].cpu(), qo)
    for c0 in (0, k - 64):
        qo, _ = O.mxfp8_quantize(x[:, c0:c0 + 64].t().contiguous())
        assert torch.equal(qd[c0:c0 + 64].cpu(), qo)
        qo, _ = O.mxfp8_quantize(w[:, c0:c0 + 64].t().contiguous())
        assert torch.equal(qb[c0:c0 + 64].cpu(), qo)
    # dX tiles: contraction over N
    da, db = _deq_mx(qa, sa, m, n), _deq_mx(qb, sb, k, n)
    for r0 in (0, m // 2 - 128, m - 256):
        want = (da[r0:r0 + 256] @ db.t()).bfloat16()
        _assert_output(dx[r0:r0 + 256].contiguous(), want)
    del da, db
    # dW whole: contraction over the 16384 token rows
    dc, dd = _deq_mx(qc, sc, n, m), _deq_mx(qd, sd, k, m)
    want = dc @ dd.t()
    if dw_dtype is torch.float32:
        assert ((dw - want).norm() / want.norm()) < 1e-5
    else:
        _assert_output(dw, want.bfloat16())
    # linearity of dX over all rows
    got = dx.double().sum(dim=0)
    ref = _deq_mx(qa, sa, m, n).double().sum(dim=0) @ _deq_mx(qb, sb, k, n).double().t()
    assert ((got - ref).norm() / ref.norm()) < 2e-3   # dX is BF16-rounded per element


# ----------------------------------------------------------------------------- configuration 5

@pytest.mark.parametrize("n", [8192, 28672])
def test_full_size_config5_nvfp4_decode(gpu, n):
    ops, N, dev, ws = gpu
    k = 8192
    inp = O.make_inputs(5, m=64, n=n, k=k)
    w = inp["w"]
    wd = w.to(dev)
    w_scale = ops.nvfp4_tensor_scale(wd, N.TENSOR_SCALE_EXACT)
    qw, sw = ops.nvfp4_quantize(wd, w_scale)
    _ok(ops, dev)
    assert torch.equal(w_scale.cpu(), O.nvfp4_tensor_scale(w, "exact"))
    for r0 in (0, n // 2, n - 64):
        qo, _ = O.nvfp4_quantize(w[r0:r0 + 64], w_scale.cpu())
        assert torch.equal(qw[r0:r0 + 64].cpu(), qo)
    dwt = _deq_nv(qw, sw, n, k)
    for m in (1, 8, 16, 64):
        x = inp["x"][:m].contiguous()
        xd = x.to(dev)
        for _ in range(2):
            y = ops.nvfp4_linear_fwd_prequant_w(xd, qw, sw, w_scale, n, ws, scale_mode=N.TENSOR_SCALE_POWER2)
        qx, sx, x_scale, o_scale = ops.nvfp4_quantize_dynamic(xd, N.TENSOR_SCALE_POWER2, w_scale)
        _ok(ops, dev)
        assert torch.equal(x_scale.cpu(), O.nvfp4_tensor_scale(x, "power2"))
        qo, _ = O.nvfp4_quantize(x, x_scale.cpu())
        assert torch.equal(qx.cpu(), qo)
        want = ((_deq_nv(qx, sx, m, k) @ dwt.t()) * o_scale).bfloat16()
        _assert_output(y, want)
        # the step-by-step route gives the same bits as the one-call decode entry
        y2 = ops.nvfp4_gemm(qx, sx, qw, sw, m, n, k, o_scale)
        _ok(ops, dev)
        assert torch.equal(y, y2)
