"""Parity of the CUDA path (through the C ABI) against the CPU oracle and the
committed golden fixtures.  Bars: quantized payloads and scales bit exact;
GEMM outputs rel-Frobenius <= 1e-3 and <= 1 BF16 ulp on >= 99.9 % of elements
versus the FP32-accumulated dequantized oracle (bit exact on the reference's
own small shapes)."""
import numpy as np
import pytest
import torch

from oracle import mx_oracle as O

pytestmark = pytest.mark.gpu

REL_FRO_MAX = 1e-3
FRAC_1ULP_MIN = 0.999


@pytest.fixture(scope="module")
def gpu(native_lib):
    if not torch.cuda.is_available():
        pytest.fail("these tests need a CUDA device")
    from rtx_b200 import _native as N
    from rtx_b200 import ops

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    return ops, N, dev, ops.Workspace(dev)


def _unpack_scales(t, rows, nb, chunks):
    return O.scales_from_mma128(t.cpu().reshape(-1, chunks, 512), rows, nb)


def _canon_nan(q):
    q = q.clone()
    q[(q & 0x7F) == 0x7F] = 0x7F
    return q


def _assert_output(got, want, bit_exact=False):
    rep = O.parity_report(got.cpu(), want)
    if bit_exact:
        assert rep["bit_equal"], rep
    assert rep["rel_fro"] <= REL_FRO_MAX and rep["frac_le_1ulp"] >= FRAC_1ULP_MIN, rep


def _ok(ops, dev):
    torch.cuda.synchronize()
    ops.check_device_status(dev)


# ----------------------------------------------------------------------------- quantizers

@pytest.mark.parametrize("shape", [(128, 256), (64, 256), (1, 32), (1, 1), (5, 33), (9, 127), (257, 385), (300, 1000)])
@pytest.mark.parametrize("rounding", ["infinity", "floor"])
def test_mxfp8_quantizer_bit_exact(gpu, shape, rounding):
    ops, N, dev, _ = gpu
    torch.manual_seed(1701)
    x = torch.randn(*shape).bfloat16()
    qo, so = O.mxfp8_quantize(x, rounding)
    nb = so.shape[1]
    for layout in (N.SCALE_ROW_MAJOR, N.SCALE_MMA128):
        q, s = ops.mxfp8_quantize(x.to(dev), layout=layout, rounding=N.ROUND_INFINITY if rounding == "infinity" else N.ROUND_FLOOR)
        _ok(ops, dev)
        s = s.cpu().reshape(shape[0], nb) if layout == N.SCALE_ROW_MAJOR else _unpack_scales(s, shape[0], nb, (nb + 3) // 4)
        assert torch.equal(q.cpu(), qo)
        assert torch.equal(s, so)


def test_mxfp8_quantizer_golden_fixtures(gpu, golden):
    """Bytes produced by executing the reference (tests/golden/make_golden.py)."""
    ops, N, dev, _ = gpu
    arrays, _ = golden
    for name in ("q1701", "q1703", "qrag", "qtiny", "q33", "special"):
        x = torch.from_numpy(arrays[f"{name}_x"].view(np.int16).copy()).view(torch.bfloat16)
        for rounding, code in (("infinity", N.ROUND_INFINITY), ("floor", N.ROUND_FLOOR)):
            q, s = ops.mxfp8_quantize(x.to(dev), layout=N.SCALE_ROW_MAJOR, rounding=code)
            _ok(ops, dev)
            want_q = torch.from_numpy(arrays[f"{name}_{rounding}_q"].copy())
            want_s = torch.from_numpy(arrays[f"{name}_{rounding}_s"].copy())
            assert torch.equal(_canon_nan(q.cpu()), _canon_nan(want_q)), (name, rounding)
            assert torch.equal(s.cpu().reshape(want_s.shape), want_s), (name, rounding)


def test_mxfp8_known_answer_480(gpu):
    ops, N, dev, _ = gpu
    src = torch.zeros(1, 32)
    src[0, 0] = 480
    for code, want_max, want_scale in ((N.ROUND_FLOOR, 448.0, 127), (N.ROUND_INFINITY, 240.0, 128)):
        q, s = ops.mxfp8_quantize(src.bfloat16().to(dev), layout=N.SCALE_ROW_MAJOR, rounding=code)
        _ok(ops, dev)
        assert O.e4m3_decode(q.cpu()).abs().max().item() == want_max
        assert int(s.cpu()[0]) == want_scale


@pytest.mark.parametrize("shape", [(128, 128), (256, 64), (33, 5), (127, 9), (385, 257), (1, 1), (2048, 96)])
def test_mxfp8_transposed_quantizer_equals_quant_of_transpose(gpu, shape):
    """rtx tests/test_mxfp8_bwd.py:695-730."""
    ops, N, dev, _ = gpu
    torch.manual_seed(1705)
    x = torch.randn(*shape).bfloat16()   # stored [K, R]
    qo, so = O.mxfp8_quantize(x.t().contiguous())
    k, r = shape
    nb = so.shape[1]
    for layout in (N.SCALE_ROW_MAJOR, N.SCALE_MMA128):
        q, s = ops.mxfp8_quantize_transposed(x.to(dev), layout=layout)
        _ok(ops, dev)
        s = s.cpu().reshape(r, nb) if layout == N.SCALE_ROW_MAJOR else _unpack_scales(s, r, nb, (nb + 3) // 4)
        assert torch.equal(q.cpu(), qo) and torch.equal(s, so)


@pytest.mark.parametrize("shape", [(128, 128), (5, 17), (9, 129), (257, 400), (1, 1)])
@pytest.mark.parametrize("mode", ["exact", "power2", "block"])
def test_nvfp4_quantizer_bit_exact(gpu, shape, mode):
    ops, N, dev, _ = gpu
    torch.manual_seed(1907)
    x = torch.randn(*shape).bfloat16()
    st_o = O.nvfp4_tensor_scale(x, mode)
    if mode == "block":
        st = None
    else:
        st = ops.nvfp4_tensor_scale(x.to(dev), N.TENSOR_SCALE_EXACT if mode == "exact" else N.TENSOR_SCALE_POWER2)
        _ok(ops, dev)
        assert torch.equal(st.cpu(), st_o)
    qo, so = O.nvfp4_quantize(x, st_o)
    nb = so.shape[1]
    for layout in (N.SCALE_ROW_MAJOR, N.SCALE_MMA128):
        q, s = ops.nvfp4_quantize(x.to(dev), st, layout=layout)
        _ok(ops, dev)
        chunks = ((nb + 3) // 4 + 3) // 4 * 4
        s = s.cpu().reshape(shape[0], nb) if layout == N.SCALE_ROW_MAJOR else _unpack_scales(s, shape[0], nb, chunks)
        assert torch.equal(q.cpu(), qo) and torch.equal(s, so)


def test_nvfp4_tensor_scale_zero_tensor(gpu):
    ops, N, dev, _ = gpu
    st = ops.nvfp4_tensor_scale(torch.zeros(16, 64, dtype=torch.bfloat16, device=dev))
    assert float(st.cpu()) == 1.0


def test_quantizers_reject_bad_arguments(gpu):
    ops, N, dev, _ = gpu
    x = torch.zeros(4, 32, dtype=torch.bfloat16, device=dev)
    with pytest.raises(N.NativeError, match="mma64"):
        ops.mxfp8_quantize(x, layout=N.SCALE_MMA64)
    with pytest.raises(TypeError):
        ops.mxfp8_quantize(x.float())
    with pytest.raises(ValueError):
        ops.mxfp8_quantize(x.cpu())


# ----------------------------------------------------------------------------- forward

@pytest.mark.parametrize("mnk", [(128, 128, 128), (37, 70, 128), (5, 129, 256), (3, 5, 1), (7, 11, 17), (9, 131, 127)])
def test_mxfp8_forward_reference_shapes_bit_exact(gpu, golden, mnk):
    """rtx tests/test_mxfp8_fwd.py:359-380: fused output rtol=0, atol=0; compared with the
    reference's own output bits and with the oracle."""
    ops, N, dev, ws = gpu
    arrays, _ = golden
    m, n, k = mnk
    torch.manual_seed(123)
    x = (torch.randn(m, k) * 0.5).bfloat16()
    w = (torch.randn(n, k) * 0.5).bfloat16()
    y = ops.mxfp8_linear_fwd(x.to(dev), w.to(dev), ws)
    _ok(ops, dev)
    want = torch.from_numpy(arrays[f"fwd_{m}_{n}_{k}_y"].view(np.int16).copy()).view(torch.bfloat16)
    assert torch.equal(y.cpu().view(torch.int16), want.view(torch.int16))
    _assert_output(y, O.mxfp8_linear(x, w), bit_exact=True)


@pytest.mark.parametrize("mnk", [(257, 385, 256), (256, 1024, 1024), (1000, 3000, 2048), (129, 257, 4096)])
def test_mxfp8_forward_larger_shapes(gpu, mnk):
    ops, N, dev, ws = gpu
    m, n, k = mnk
    if mnk == (256, 1024, 1024):
        inp = O.make_inputs(1)          # benchmark configuration 1, seed 0
        x, w = inp["x"], inp["w"]
    else:
        torch.manual_seed(321)
        x = (torch.randn(m, k) * 0.5).bfloat16()
        w = (torch.randn(n, k) * 0.5).bfloat16()
    y = ops.mxfp8_linear_fwd(x.to(dev), w.to(dev), ws)
    _ok(ops, dev)
    _assert_output(y, O.mxfp8_linear(x, w))


def test_mxfp8_forward_floor_rounding_ablation(gpu):
    ops, N, dev, ws = gpu
    torch.manual_seed(9)
    x = torch.randn(130, 200).bfloat16()
    w = torch.randn(90, 200).bfloat16()
    y = ops.mxfp8_linear_fwd(x.to(dev), w.to(dev), ws, rounding=N.ROUND_FLOOR)
    _ok(ops, dev)
    _assert_output(y, O.mxfp8_linear(x, w, "floor"))


def test_mxfp8_prequantized_gemm_f32_and_repeatability(gpu):
    """Packed-operand GEMM (rtx tests/test_mxfp8_quant.py:222-254), FP32 output, and eight
    repeats into NaN-poisoned outputs to catch stale-barrier races (rtx tests/test_mxfp8_fwd.py:664-672)."""
    ops, N, dev, _ = gpu
    torch.manual_seed(1702)
    m, n, k = 384, 640, 512
    x, w = torch.randn(m, k).bfloat16(), torch.randn(n, k).bfloat16()
    qa, sa = ops.mxfp8_quantize(x.to(dev))
    qb, sb = ops.mxfp8_quantize(w.to(dev))
    want = O.mxfp8_linear_f32(x, w)
    first = None
    for _ in range(8):
        out = torch.full((m, n), float("nan"), dtype=torch.float32, device=dev)
        ops.mxfp8_gemm(qa, sa, qb, sb, m, n, k, out=out)
        _ok(ops, dev)
        got = out.cpu()
        assert not torch.isnan(got).any()
        assert ((got - want).norm() / want.norm()) < 1e-5
        first = got if first is None else first
        assert torch.equal(got, first)


@pytest.mark.parametrize("schedule,operand", [("pair", "a"), ("pair", "b"), ("single", "a"), ("single", "b"),
                                              ("stream", "b")])
def test_odd_k_tiles_with_nan_in_the_next_row_block(gpu, schedule, operand):
    """K = 384 is three 128-byte K steps: kernels that hand over two K steps per barrier load a
    fourth step past the end of K.  Its scale bytes are those of the NEXT 128-row block; a NaN
    there (E8M0 0xFF) must not reach this block's outputs.  The reference keeps unrelated rows
    and columns finite, and so must the product: everything outside the poisoned row / column
    is bit-equal to the result without the NaN."""
    ops, N, dev, _ = gpu
    m, n, k = (64 if schedule == "stream" else 384), 512, 384   # the streaming kernel serves M <= 128
    torch.manual_seed(77)
    x, w = torch.randn(m, k).bfloat16(), torch.randn(n, k).bfloat16()
    qa0, sa0 = ops.mxfp8_quantize(x.to(dev))
    qb0, sb0 = ops.mxfp8_quantize(w.to(dev))
    want_clean = O.mxfp8_linear(x, w)
    bad_row = 128 + 5          # first K block of a row in row block 1
    if operand == "a":
        x[bad_row, 0] = float("nan")
    else:
        w[bad_row, 0] = float("nan")
    qa, sa = ops.mxfp8_quantize(x.to(dev))
    qb, sb = ops.mxfp8_quantize(w.to(dev))
    with ops.gemm_schedule(schedule):
        clean = ops.mxfp8_gemm(qa0, sa0, qb0, sb0, m, n, k)
        got = ops.mxfp8_gemm(qa, sa, qb, sb, m, n, k)
    _ok(ops, dev)
    clean, got = clean.cpu(), got.cpu()
    _assert_output(clean, want_clean)
    keep = torch.ones(m if operand == "a" else n, dtype=torch.bool)
    keep[bad_row] = False
    if operand == "a":
        assert torch.isnan(got[bad_row].float()).all()
        assert torch.equal(got[keep].view(torch.int16), clean[keep].view(torch.int16))
    else:
        assert torch.isnan(got[:, bad_row].float()).all()
        assert torch.equal(got[:, keep].view(torch.int16), clean[:, keep].view(torch.int16))


@pytest.mark.parametrize("dims", [(128, 128, 128, 128), (256, 512, 384, 512), (300, 256, 256, 200), (64, 96, 128, 80)])
def test_mxfp8_glu_mlp(gpu, dims):
    ops, N, dev, ws = gpu
    m, k, inter, n_out = dims
    inp = O.make_inputs(2, m=m, k=k, inter=inter)
    x, wgu = inp["x"], inp["w_gate_up"]
    torch.manual_seed(4)
    wd = (torch.randn(n_out, inter) / inter ** 0.5).bfloat16()
    h, y = ops.mxfp8_glu_mlp_fwd(x.to(dev), wgu.to(dev), wd.to(dev), ws)
    _ok(ops, dev)
    ho, yo = O.mxfp8_glu_mlp(x, wgu, wd)
    _assert_output(h, ho)
    # Y is compared on the device's own H so that one-ulp differences in H do not compound
    _assert_output(y, O.mxfp8_linear(h.cpu(), wd))
    rep = O.parity_report(y.cpu(), yo)
    assert rep["rel_fro"] <= 5e-3, rep


@pytest.mark.parametrize("dims", [(128, 128, 128), (300, 256, 384), (2048, 512, 1024)])
def test_glu_epilogue_emits_h_as_mxfp8(gpu, dims):
    """The quantizing GLU epilogue equals quantizing its own BF16 H with the row quantizer, bit for bit,
    whether or not the BF16 copy is also written; the MLP result does not depend on materializing H."""
    ops, N, dev, ws = gpu
    m, k, inter = dims
    inp = O.make_inputs(2, m=m, k=k, inter=inter)
    x, wgu, wd = inp["x"].to(dev), inp["w_gate_up"].to(dev), inp["w_down"].to(dev)
    qx, sx = ops.mxfp8_quantize(x)
    qg, sg = ops.mxfp8_quantize(wgu)
    q1, s1, h = ops.mxfp8_gemm_glu_mx(qx, sx, qg, sg, m, inter, k, want_bf16=True)
    q2, s2, none = ops.mxfp8_gemm_glu_mx(qx, sx, qg, sg, m, inter, k, want_bf16=False)
    h_ref = ops.mxfp8_gemm_glu(qx, sx, qg, sg, m, inter, k)
    qh, sh = ops.mxfp8_quantize(h)
    _ok(ops, dev)
    assert none is None
    assert torch.equal(h, h_ref)
    assert torch.equal(q1, qh) and torch.equal(q1, q2)
    nb = inter // 32
    want_s = _unpack_scales(sh, m, nb, (nb + 3) // 4)
    assert torch.equal(_unpack_scales(s1, m, nb, (nb + 3) // 4), want_s)
    assert torch.equal(_unpack_scales(s2, m, nb, (nb + 3) // 4), want_s)
    h1, y1 = ops.mxfp8_glu_mlp_fwd(x, wgu, wd, ws, want_hidden=True)
    h0, y0 = ops.mxfp8_glu_mlp_fwd(x, wgu, wd, ws, want_hidden=False)
    _ok(ops, dev)
    assert h0 is None and torch.equal(y0, y1) and torch.equal(h1, h)


def test_mxfp8_glu_rejects_ragged_inter(gpu):
    ops, N, dev, ws = gpu
    x = torch.zeros(8, 64, dtype=torch.bfloat16, device=dev)
    with pytest.raises(N.NativeError, match="inter"):
        ops.mxfp8_glu_mlp_fwd(x, torch.zeros(2 * 96, 64, dtype=torch.bfloat16, device=dev),
                              torch.zeros(32, 96, dtype=torch.bfloat16, device=dev), ws)


# ----------------------------------------------------------------------------- failure path

def test_a_wait_that_nothing_completes_runs_out_and_reports(gpu):
    """Every kernel role waits with a bound.  The self-test kernel waits on a barrier that nothing completes:
    after the limit it stores its code in the status word and returns normally; the host sees the code through
    the same check every call site uses, the context stays usable and the next GEMM gives the right bits.
    Nothing traps or hangs: the failure is a wait that is allowed to run out."""
    import ctypes

    ops, N, dev, _ = gpu
    status = ops.status_word(dev)
    waited = torch.zeros(1, dtype=torch.int64, device=dev)
    limit_ns = 20_000_000
    N.call("rtxb_selftest_wait_timeout", limit_ns, torch.cuda.current_stream().cuda_stream, status.data_ptr(),
           waited.data_ptr())
    torch.cuda.synchronize()
    assert int(status.item()) == 5
    assert limit_ns <= int(waited.item()) < 50 * limit_ns
    with pytest.raises(RuntimeError, match="self-test wait ran out"):
        ops.check_device_status(dev)
    assert int(status.item()) == 0                      # the check clears the word
    with pytest.raises(N.NativeError):
        N.call("rtxb_selftest_wait_timeout", 10, None, status.data_ptr(), None)    # limit below 1 ms: refused
    # the context is intact: a GEMM right after gives the oracle's bits
    x, w = torch.randn(128, 128).bfloat16(), torch.randn(128, 128).bfloat16()
    qa, sa = ops.mxfp8_quantize(x.to(dev))
    qb, sb = ops.mxfp8_quantize(w.to(dev))
    _assert_output(ops.mxfp8_gemm(qa, sa, qb, sb, 128, 128, 128), O.mxfp8_linear(x, w))
    _ok(ops, dev)


def test_node_barrier_alone_and_with_a_rank_that_never_arrives(gpu):
    """rtxb_peer_barrier on one GPU: a group of one passes at once, epoch after epoch; in a group of two whose other
    rank never signals, the bounded wait runs out after the limit, the status word says which wait it was, and the
    context stays usable.  (Ranks that do arrive are covered by the two-GPU tests: kernels that wait for one
    another are never run as separate launches on one GPU.)"""
    ops, N, dev, _ = gpu
    mine = torch.zeros(8, dtype=torch.int32, device=dev)
    absent = torch.zeros(8, dtype=torch.int32, device=dev)
    epoch = torch.zeros(1, dtype=torch.int32, device=dev)
    for _ in range(3):
        ops.peer_barrier([mine.data_ptr()], 0, epoch)
    _ok(ops, dev)
    assert mine.tolist()[0] == 3 and epoch.item() == 3                   # the kernel keeps the count itself
    # the same launch replayed from a captured graph keeps counting (no per-call number in the launch)
    graph, side = torch.cuda.CUDAGraph(), torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        ops.peer_barrier([mine.data_ptr()], 0, epoch)
    torch.cuda.current_stream().wait_stream(side)
    with torch.cuda.graph(graph):
        ops.peer_barrier([mine.data_ptr()], 0, epoch)
    for _ in range(3):
        graph.replay()
    _ok(ops, dev)
    assert epoch.item() == 7 and mine.tolist()[0] == 7
    ops.peer_barrier([mine.data_ptr(), absent.data_ptr()], 0, epoch, limit_ns=20_000_000)
    torch.cuda.synchronize()
    assert absent.tolist()[0] == 8 and mine.tolist()[:2] == [8, 0]      # we signalled both; rank 1 never did
    with pytest.raises(RuntimeError, match="another rank's flag never arrived"):
        ops.check_device_status(dev)
    with pytest.raises(N.NativeError):
        ops.peer_barrier([mine.data_ptr()], 1, epoch)                    # rank outside the group
    ops.peer_barrier([mine.data_ptr()], 0, epoch)
    _ok(ops, dev)


# ----------------------------------------------------------------------------- backward

@pytest.mark.parametrize("mnk", [(128, 128, 128), (256, 384, 512), (100, 70, 50), (512, 256, 1024), (33, 1, 7)])
@pytest.mark.parametrize("dw_dtype", [torch.bfloat16, torch.float32])
def test_mxfp8_backward(gpu, mnk, dw_dtype):
    ops, N, dev, ws = gpu
    m, n, k = mnk
    inp = O.make_inputs(4, m=m, n=n, k=k)
    x, w, dy = inp["x"], inp["w"], inp["dy"]
    dx, dw = ops.mxfp8_linear_bwd(dy.to(dev), x.to(dev), w.to(dev), ws, dw_dtype=dw_dtype)
    _ok(ops, dev)
    dxo, dwo = O.mxfp8_backward(x, w, dy, dw_dtype=torch.float32)
    _assert_output(dx, dxo)
    if dw_dtype == torch.bfloat16:
        _assert_output(dw, dwo.bfloat16())
    else:
        assert ((dw.cpu() - dwo).norm() / dwo.norm().clamp(min=1e-30)) < 1e-5
    # sanity against the unquantized FP32 product (rtx tests/test_mxfp8_bwd.py:634-653: < 7 %)
    if min(m, n, k) >= 32:
        ref = dy.float() @ w.float()
        assert ((dx.float().cpu() - ref).norm() / ref.norm()) < 0.07


def test_mxfp8_backward_single_outputs(gpu):
    ops, N, dev, ws = gpu
    inp = O.make_inputs(4, m=128, n=128, k=128)
    x, w, dy = (inp[k].to(dev) for k in ("x", "w", "dy"))
    dx, dw = ops.mxfp8_linear_bwd(dy, x, w, ws)
    dx2, none = ops.mxfp8_linear_bwd(dy, None, w, ws, need_dw=False)
    none2, dw2 = ops.mxfp8_linear_bwd(dy, x, None, ws, need_dx=False)
    _ok(ops, dev)
    assert none is None and none2 is None
    assert torch.equal(dx, dx2) and torch.equal(dw, dw2)


# ----------------------------------------------------------------------------- NVFP4

@pytest.mark.parametrize("mnk", [(128, 256, 256), (128, 128, 128), (37, 70, 128), (5, 129, 272), (257, 385, 512), (9, 131, 127), (512, 1024, 2048)])
@pytest.mark.parametrize("mode", ["power2", "exact"])
def test_nvfp4_forward(gpu, mnk, mode):
    ops, N, dev, ws = gpu
    m, n, k = mnk
    inp = O.make_inputs(3, m=m, n=n, k=k)
    x, w = inp["x"], inp["w"]
    y = ops.nvfp4_linear_fwd(x.to(dev), w.to(dev), ws,
                             scale_mode=N.TENSOR_SCALE_POWER2 if mode == "power2" else N.TENSOR_SCALE_EXACT)
    _ok(ops, dev)
    _assert_output(y, O.nvfp4_linear(x, w, mode=mode))
    ref = x.float() @ w.float().t()
    if k >= 128:   # rtx benchmarks/validate_production.py:75-76: NVFP4 forward rel-L2 < 18 %
        assert ((y.float().cpu() - ref).norm() / ref.norm()) < 0.18


@pytest.mark.parametrize("m", [1, 8, 16, 64, 128])
def test_nvfp4_decode_with_prequantized_weight(gpu, m):
    """Benchmark configuration 5 in small: packed weights (exact outer scale), activations quantized on the
    fly; M <= 128 takes the 128 x 64 streaming kernel."""
    ops, N, dev, _ = gpu
    n, k = 1536, 2048
    inp = O.make_inputs(5, m=m, n=n, k=k)
    x, w = inp["x"], inp["w"]
    ws_o, xs_o = O.nvfp4_tensor_scale(w, "exact"), O.nvfp4_tensor_scale(x, "exact")
    w_scale = ops.nvfp4_tensor_scale(w.to(dev), N.TENSOR_SCALE_EXACT)
    qw, sw = ops.nvfp4_quantize(w.to(dev), w_scale)
    xd = x.to(dev)
    x_scale, o_scale = ops.nvfp4_tensor_scale(xd, N.TENSOR_SCALE_EXACT, other_scale=w_scale)
    qx, sx = ops.nvfp4_quantize(xd, x_scale)
    y = ops.nvfp4_gemm(qx, sx, qw, sw, m, n, k, o_scale)
    y32 = ops.nvfp4_gemm(qx, sx, qw, sw, m, n, k, o_scale, out_dtype=torch.float32)
    _ok(ops, dev)
    want = O.nvfp4_linear(x, w, x_scale=xs_o, w_scale=ws_o)
    _assert_output(y, want)
    _assert_output(y32.bfloat16(), want)


@pytest.mark.parametrize("shape", [(1, 8192), (8, 8192), (8, 8256), (64, 2048), (64, 8192), (100, 1000), (128, 4128),
                                   (300, 8192)])
@pytest.mark.parametrize("mode", ["exact", "power2"])
def test_nvfp4_quantize_dynamic_equals_two_pass(gpu, shape, mode):
    """The small-tensor route of the dynamic quantizer (two chained launches: per-CTA |max| partials,
    then scale rule + quantize) gives the bytes of the separate |max| / finalize / quantize launches
    (whole buffers, padding included) and of the oracle; (300, 8192) is above its size limit and takes
    the three-launch route behind the same entry point."""
    ops, N, dev, _ = gpu
    rows, k = shape
    torch.manual_seed(rows * 131 + k)
    x = (torch.randn(rows, k) * 3).bfloat16()
    x[0, 0] = 97.0
    code = N.TENSOR_SCALE_EXACT if mode == "exact" else N.TENSOR_SCALE_POWER2
    xd = x.to(dev)
    other = torch.tensor([0.375], dtype=torch.float32, device=dev)
    q, s, scale, prod = ops.nvfp4_quantize_dynamic(xd, code, other_scale=other)
    scale2, prod2 = ops.nvfp4_tensor_scale(xd, code, other_scale=other)
    q2, s2 = ops.nvfp4_quantize(xd, scale2)
    _ok(ops, dev)
    assert torch.equal(scale, scale2) and torch.equal(prod, prod2)
    assert torch.equal(q, q2) and torch.equal(s, s2)
    st = O.nvfp4_tensor_scale(x, mode)
    assert float(scale.cpu()) == float(st)
    qo, so = O.nvfp4_quantize(x, st)
    assert torch.equal(q.cpu(), qo)
    q_rm, s_rm, _, _ = ops.nvfp4_quantize_dynamic(xd, code, layout=N.SCALE_ROW_MAJOR)
    assert torch.equal(q_rm, q2)
    assert torch.equal(s_rm.cpu().view(rows, -1)[:, :so.shape[1]], so)


@pytest.mark.parametrize("shape_r", [((40, 256), 5), ((128, 1024), 4), ((300, 1000), 5), ((512, 4096), 8),
                                     ((48, 2052), 8), ((37, 64), 37), ((6, 33), 1)])
@pytest.mark.parametrize("mode", ["power2", "exact"])
def test_nvfp4_row_region_scales_and_payload(gpu, shape_r, mode):
    """Row-region policy: one outer scale per region of rows from the region's |max| (bit equal to the
    oracle), and payload / block scales of every row quantized with its region's scale."""
    ops, N, dev, _ = gpu
    (rows, k), r = shape_r
    torch.manual_seed(rows * 7 + k)
    x = (torch.randn(rows, k) * torch.logspace(-2, 2, rows).unsqueeze(1)).bfloat16()   # regions differ in range
    code = N.TENSOR_SCALE_EXACT if mode == "exact" else N.TENSOR_SCALE_POWER2
    xd = x.to(dev)
    scales = ops.nvfp4_region_scales(xd, r, code)
    want_scales = O.nvfp4_region_scales(x, r, mode)
    _ok(ops, dev)
    assert torch.equal(scales.cpu(), want_scales)
    q, s = ops.nvfp4_quantize_regions(xd, scales, r, layout=N.SCALE_ROW_MAJOR)
    q2, s2 = ops.nvfp4_quantize_regions(xd, scales, r)
    _ok(ops, dev)
    qo, so = O.nvfp4_quantize_regions(x, want_scales, r)
    assert torch.equal(q.cpu(), qo) and torch.equal(q2.cpu(), qo)
    assert torch.equal(s.cpu().view(rows, -1)[:, :so.shape[1]], so)
    nb = so.shape[1]
    chunks = (nb + 3) // 4
    chunks = (chunks + 3) // 4 * 4
    assert torch.equal(O.scales_from_mma128(s2.cpu().view(-1, chunks, 512), rows, nb), so)


@pytest.mark.parametrize("mnk_r", [((40, 64, 128), 5, 4), ((260, 384, 512), 5, 4), ((257, 385, 256), 5, 4),
                                   ((1000, 3000, 2048), 5, 4), ((128, 8192, 1024), 8, 8), ((64, 512, 256), 1, 1)])
def test_nvfp4_row_region_linear(gpu, mnk_r):
    """Forward with row-region outer scales against the oracle: out = bf16(acc * (xs[m / Rx] * ws[n / Rw])).
    (257, 385) does not split into regions of 5 / 4 rows: both operands fall back to one region, which
    must equal the `current` policy bit for bit."""
    ops, N, dev, ws = gpu
    (m, n, k), rx, rw = mnk_r
    torch.manual_seed(m + n + k)
    x = (torch.randn(m, k) * torch.logspace(-1, 1, m).unsqueeze(1)).bfloat16()
    w = (torch.randn(n, k) / k ** 0.5 * torch.logspace(-1, 1, n).unsqueeze(1)).bfloat16()
    y = ops.nvfp4_linear_fwd_regions(x.to(dev), w.to(dev), ws, rx, rw)
    _ok(ops, dev)
    _assert_output(y, O.nvfp4_linear_regions(x, w, rx, rw))
    if (m, n) == (257, 385):
        y_cur = ops.nvfp4_linear_fwd(x.to(dev), w.to(dev), ws)
        _ok(ops, dev)
        assert torch.equal(y, y_cur)


@pytest.mark.parametrize("hist", [(1, True), (4, True), (16, False), (64, True)])
@pytest.mark.parametrize("mode", ["power2", "exact"])
def test_nvfp4_delayed_operand(gpu, hist, mode):
    """Delayed policy, one operand: quantized with the scale of the |max| history (window maximum or most
    recent entry), current |max| observed in the same pass and published as next_history[0], history
    rotated by one."""
    ops, N, dev, _ = gpu
    length, window = hist
    torch.manual_seed(length * 3 + int(window))
    x = (torch.randn(300, 1000) * 2).bfloat16()
    history = (torch.rand(length) * 6 + 0.5).float()
    nxt = torch.full((length,), -1.0)
    code = N.TENSOR_SCALE_EXACT if mode == "exact" else N.TENSOR_SCALE_POWER2
    other = torch.tensor([0.25], device=dev)
    hd, nd = history.to(dev), nxt.to(dev)
    q, s, scale, prod = ops.nvfp4_quantize_delayed(x.to(dev), hd, nd, window_max=window, mode=code, other_scale=other,
                                                   layout=N.SCALE_ROW_MAJOR)
    _ok(ops, dev)
    qo, so, scale_o, next_o = O.nvfp4_delayed_operand(x, history, "window_max" if window else "most_recent", mode)
    assert torch.equal(scale.cpu(), scale_o) and float(prod.cpu()) == float(scale_o) * 0.25
    assert torch.equal(q.cpu(), qo)
    assert torch.equal(s.cpu().view(300, -1)[:, :so.shape[1]], so)
    assert torch.equal(nd.cpu(), next_o)
    assert torch.equal(hd.cpu(), history)          # the prior generation is read only


def test_nvfp4_delayed_linear_steps(gpu):
    """Three steps of the delayed forward with drifting activations: every step equals the oracle fed with
    the same histories, and the histories evolve as the oracle's do."""
    ops, N, dev, ws = gpu
    m, n, k = 260, 384, 512
    torch.manual_seed(5)
    w = (torch.randn(n, k) / k ** 0.5).bfloat16()
    xh = torch.full((4,), 3.0)
    wh = w.float().abs().amax().reshape(1).expand(4).clone()
    xd_h, wd_h = xh.to(dev), wh.to(dev)
    xd_n, wd_n = torch.empty_like(xd_h), torch.empty_like(wd_h)
    for step in range(3):
        x = (torch.randn(m, k) * (1.0 + 2.0 * step)).bfloat16()     # the range drifts: the scale lags one step
        y = ops.nvfp4_linear_fwd_delayed(x.to(dev), w.to(dev), ws, xd_h, wd_h, xd_n, wd_n)
        _ok(ops, dev)
        want, xh, wh = O.nvfp4_linear_delayed(x, w, xh, wh)
        _assert_output(y, want)
        assert torch.equal(xd_n.cpu(), xh) and torch.equal(wd_n.cpu(), wh)
        xd_h, xd_n = xd_n, xd_h
        wd_h, wd_n = wd_n, wd_h


@pytest.mark.parametrize("m", [1, 8, 16, 64, 128])
@pytest.mark.parametrize("n", [1536, 19456])
def test_nvfp4_linear_fwd_prequant_w(gpu, m, n):
    """Decode entry point: packed weight + activations quantized on the fly, the GEMM launched as a
    programmatic dependent of the quantizer.  Equal to the step-by-step route bit for bit and to the
    oracle within the output tolerance; N = 19456 takes the 128 x 256 kernel, 1536 the streaming one."""
    ops, N, dev, ws = gpu
    k = 2048
    inp = O.make_inputs(5, m=m, n=n, k=k)
    x, w = inp["x"], inp["w"]
    wd, xd = w.to(dev), x.to(dev)
    w_scale = ops.nvfp4_tensor_scale(wd, N.TENSOR_SCALE_EXACT)
    qw, sw = ops.nvfp4_quantize(wd, w_scale)
    for _ in range(2):
        y = ops.nvfp4_linear_fwd_prequant_w(xd, qw, sw, w_scale, n, ws, scale_mode=N.TENSOR_SCALE_EXACT)
    x_scale, o_scale = ops.nvfp4_tensor_scale(xd, N.TENSOR_SCALE_EXACT, other_scale=w_scale)
    qx, sx = ops.nvfp4_quantize(xd, x_scale)
    y2 = ops.nvfp4_gemm(qx, sx, qw, sw, m, n, k, o_scale)
    _ok(ops, dev)
    assert torch.equal(y, y2)
    want = O.nvfp4_linear(x, w, x_scale=O.nvfp4_tensor_scale(x, "exact"), w_scale=O.nvfp4_tensor_scale(w, "exact"))
    _assert_output(y, want)


@pytest.mark.parametrize("shape", [(128, 128), (256, 384), (300, 1000), (33, 65), (1, 32), (1000, 72)])
@pytest.mark.parametrize("layout", ["mma128", "row_major"])
def test_mxfp8_quantize_dual_equals_separate_passes(gpu, shape, layout):
    """The dual quantizer (gradient read once for the dX and the dW operand) gives the bytes of the row
    quantizer and of the transposed quantizer, scale buffers included."""
    ops, N, dev, _ = gpu
    m, n = shape
    torch.manual_seed(m * 3 + n)
    g = (torch.randn(m, n) * 0.1).bfloat16().to(dev)
    code = N.SCALE_MMA128 if layout == "mma128" else N.SCALE_ROW_MAJOR
    q_rows, s_rows, q_t, s_t = ops.mxfp8_quantize_dual(g, layout=code)
    q1, s1 = ops.mxfp8_quantize(g, layout=code)
    q2, s2 = ops.mxfp8_quantize_transposed(g, layout=code)
    _ok(ops, dev)
    assert torch.equal(q_rows, q1) and torch.equal(s_rows, s1)
    assert torch.equal(q_t, q2) and torch.equal(s_t, s2)


@pytest.mark.parametrize("mnk", [(1, 64, 512), (3, 1000, 768), (4, 130, 2048), (4, 8192, 8192), (2, 4096, 4096)])
@pytest.mark.parametrize("mode", ["power2", "exact"])
def test_nvfp4_decode_one_kernel_equals_the_chain(gpu, mnk, mode):
    """M <= 4 and K a multiple of 256: the activations are quantized inside the GEMM kernel (every CTA
    reduces |max| of X, applies the scale rule and writes the swizzled A tiles itself).  Bit equal to the
    separate |max| / quantize / GEMM launches, and within tolerance of the oracle."""
    ops, N, dev, ws = gpu
    m, n, k = mnk
    torch.manual_seed(m * 5 + n + k)
    x = (torch.randn(m, k) * 1.7).bfloat16()
    w = (torch.randn(n, k) / k ** 0.5).bfloat16()
    code = N.TENSOR_SCALE_EXACT if mode == "exact" else N.TENSOR_SCALE_POWER2
    wd, xd = w.to(dev), x.to(dev)
    w_scale = ops.nvfp4_tensor_scale(wd, N.TENSOR_SCALE_EXACT)
    qw, sw = ops.nvfp4_quantize(wd, w_scale)
    for _ in range(2):
        y = ops.nvfp4_linear_fwd_prequant_w(xd, qw, sw, w_scale, n, ws, scale_mode=code)
    x_scale, o_scale = ops.nvfp4_tensor_scale(xd, code, other_scale=w_scale)
    qx, sx = ops.nvfp4_quantize(xd, x_scale)
    y2 = ops.nvfp4_gemm(qx, sx, qw, sw, m, n, k, o_scale)
    _ok(ops, dev)
    assert torch.equal(y, y2)
    want = O.nvfp4_linear(x, w, x_scale=O.nvfp4_tensor_scale(x, mode), w_scale=O.nvfp4_tensor_scale(w, "exact"))
    _assert_output(y, want)


@pytest.mark.parametrize("mnk", [(1, 64, 32), (128, 8192, 512), (100, 4100, 1000), (17, 63, 4096), (16, 19456, 256)])
def test_mxfp8_skinny_shapes(gpu, mnk):
    ops, N, dev, ws = gpu
    m, n, k = mnk
    torch.manual_seed(77)
    x = torch.randn(m, k).bfloat16()
    w = (torch.randn(n, k) / k ** 0.5).bfloat16()
    y = ops.mxfp8_linear_fwd(x.to(dev), w.to(dev), ws)
    _ok(ops, dev)
    _assert_output(y, O.mxfp8_linear(x, w))


@pytest.mark.parametrize("mnk", [(64, 512, 1024), (128, 8192, 512), (100, 4100, 1000), (300, 640, 512), (1, 64, 32)])
def test_gemm_schedules_give_the_same_bits(gpu, mnk):
    """Every built GEMM kernel, forced for the call with the per-thread schedule switch, returns the bits the
    library's own choice returns (K is accumulated in the same order by all of them); the switch is restored
    on exit and refuses unknown names."""
    ops, N, dev, ws = gpu
    m, n, k = mnk
    torch.manual_seed(4242)
    x = torch.randn(m, k).bfloat16().to(dev)
    w = (torch.randn(n, k) / k ** 0.5).bfloat16().to(dev)
    auto = ops.mxfp8_linear_fwd(x, w, ws).clone()
    xs, wsc = ops.nvfp4_tensor_scale(x, N.TENSOR_SCALE_POWER2), ops.nvfp4_tensor_scale(w, N.TENSOR_SCALE_POWER2)
    qx, sx = ops.nvfp4_quantize(x, xs)
    qw, sw = ops.nvfp4_quantize(w, wsc)
    out_scale = xs * wsc
    auto4 = ops.nvfp4_gemm(qx, sx, qw, sw, m, n, k, out_scale).clone()
    _ok(ops, dev)
    for name in ("single", "pair", "stream"):
        with ops.gemm_schedule(name):
            assert N.query("rtxb_get_gemm_schedule") == ops.GEMM_SCHEDULES[name]
            got = ops.mxfp8_linear_fwd(x, w, ws).clone()
            got4 = ops.nvfp4_gemm(qx, sx, qw, sw, m, n, k, out_scale).clone()
        _ok(ops, dev)
        assert N.query("rtxb_get_gemm_schedule") == 0
        assert torch.equal(got.view(torch.int16), auto.view(torch.int16)), name
        assert torch.equal(got4.view(torch.int16), auto4.view(torch.int16)), name
    with pytest.raises(ValueError):
        ops.gemm_schedule("wide")


def test_decode_entry_honours_the_schedule(gpu):
    """M <= 4 with a packed weight takes one kernel by default; a forced large-tile schedule takes the
    three-launch chain with that GEMM instead and returns the same bits."""
    ops, N, dev, ws = gpu
    m, n, k = 2, 1024, 2048
    torch.manual_seed(99)
    x = torch.randn(m, k).bfloat16().to(dev)
    w = (torch.randn(n, k) / k ** 0.5).bfloat16().to(dev)
    w_scale = ops.nvfp4_tensor_scale(w, N.TENSOR_SCALE_POWER2)
    qw, sw = ops.nvfp4_quantize(w, w_scale)
    auto = ops.nvfp4_linear_fwd_prequant_w(x, qw, sw, w_scale, n, ws).clone()
    _ok(ops, dev)
    for name in ("single", "pair", "stream"):
        with ops.gemm_schedule(name):
            got = ops.nvfp4_linear_fwd_prequant_w(x, qw, sw, w_scale, n, ws).clone()
        _ok(ops, dev)
        assert torch.equal(got.view(torch.int16), auto.view(torch.int16)), name


# ----------------------------------------------------------------------------- full-size properties

def _deq_mx_gpu(q, s_tiles, rows, k):
    """Dequantise on the device with plain torch ops (checker only)."""
    nb = (k + 31) // 32
    chunks = (nb + 3) // 4
    r = torch.arange(rows, device=q.device).unsqueeze(1)
    b = torch.arange(nb, device=q.device).unsqueeze(0)
    idx = ((r // 128) * chunks + b // 4) * 512 + (r % 32) * 16 + ((r // 32) % 4) * 4 + b % 4
    codes = s_tiles[idx.reshape(-1)].reshape(rows, nb).to(torch.int32)
    scale = (codes.clamp(min=1) << 23).view(torch.float32)
    return q.view(torch.float8_e4m3fn).float() * scale.repeat_interleave(32, dim=1)


def test_full_size_config2_properties(gpu):
    """Benchmark configuration 2 at full size: sampled rows of every payload against the oracle,
    GEMM tiles from the first/middle/last tile rows and columns against an FP32 matmul of the
    device-dequantised operands, and a column checksum (linearity) over the whole output."""
    ops, N, dev, ws = gpu
    inp = O.make_inputs(2)
    x, wgu, wd = inp["x"], inp["w_gate_up"], inp["w_down"]
    m, k = x.shape
    inter = wgu.shape[0] // 2
    xd, wgud, wdd = x.to(dev), wgu.to(dev), wd.to(dev)
    qx, sx = ops.mxfp8_quantize(xd)
    qg, sg = ops.mxfp8_quantize(wgud)
    _ok(ops, dev)
    for rows in (slice(0, 64), slice(4000, 4064), slice(m - 64, m)):
        qo, _ = O.mxfp8_quantize(x[rows])
        assert torch.equal(qx[rows].cpu(), qo)
    qo, so = O.mxfp8_quantize(wgu[-128:])
    assert torch.equal(qg[-128:].cpu(), qo)
    h, y = ops.mxfp8_glu_mlp_fwd(xd, wgud, wdd, ws)
    _ok(ops, dev)
    dx = _deq_mx_gpu(qx, sx, m, k)
    dg = _deq_mx_gpu(qg, sg, 2 * inter, k)
    for r0 in (0, 4096 - 64, m - 128):
        for c0 in (0, 7168 - 64, inter - 128):
            acc_g = dx[r0:r0 + 128] @ dg[c0:c0 + 128].t()
            acc_u = dx[r0:r0 + 128] @ dg[inter + c0:inter + c0 + 128].t()
            want = (torch.nn.functional.silu(acc_g) * acc_u).bfloat16()
            _assert_output(h[r0:r0 + 128, c0:c0 + 128].contiguous(), want.cpu())
    # linearity: column sums of the plain GEMM equal (sum of rows of deq X) @ deq W^T
    yg = ops.mxfp8_gemm(qx, sx, qg, sg, m, 2 * inter, k, out_dtype=torch.float32)
    _ok(ops, dev)
    want = dx.double().sum(dim=0) @ dg.double().t()
    got = yg.double().sum(dim=0)
    assert ((got - want).norm() / want.norm()) < 1e-5
    # down projection on the device's own H
    qh, sh = ops.mxfp8_quantize(h)
    qd, sd = ops.mxfp8_quantize(wdd)
    dh, dd = _deq_mx_gpu(qh, sh, m, inter), _deq_mx_gpu(qd, sd, wd.shape[0], inter)
    for r0 in (0, m - 128):
        want = (dh[r0:r0 + 128] @ dd.t()).bfloat16()
        _assert_output(y[r0:r0 + 128].contiguous(), want.cpu())


# ----------------------------------------------------------------------------- in-kernel quantization of X

@pytest.mark.parametrize("mnk", [(256, 256, 256), (384, 512, 384), (300, 700, 1000), (129, 257, 96), (1000, 3000, 2048),
                                 (130, 64, 40), (8192, 512, 4096)])
@pytest.mark.parametrize("rounding", ["infinity", "floor"])
def test_fused_x_gemm_equals_quantize_then_gemm(gpu, mnk, rounding):
    """The pair GEMM whose quantizer warps encode X in the kernel (the reference's fused forward,
    rtx/kernels/mxfp8_fwd.py:936-2934) gives the bits of the row quantizer followed by the packed GEMM,
    ragged M / N / K and an odd number of K steps included; the composite forward routes to it under the
    "fused_x" schedule."""
    ops, N, dev, ws = gpu
    m, n, k = mnk
    code = N.ROUND_INFINITY if rounding == "infinity" else N.ROUND_FLOOR
    torch.manual_seed(31)
    x = (torch.randn(m, k) * 0.5).bfloat16().to(dev)
    w = (torch.randn(n, k) * 0.5).bfloat16().to(dev)
    x[m // 2, k // 3] = 300.0            # an outlier block
    qx, sx = ops.mxfp8_quantize(x, rounding=code)
    qw, sw = ops.mxfp8_quantize(w, rounding=code)
    with ops.gemm_schedule("pair"):
        want = ops.mxfp8_gemm(qx, sx, qw, sw, m, n, k)
    for _ in range(2):
        got = ops.mxfp8_linear_fwd_fused_x(x, qw, sw, n, rounding=code)
    _ok(ops, dev)
    assert torch.equal(got.view(torch.int16), want.view(torch.int16))
    with ops.gemm_schedule("fused_x"):
        routed = ops.mxfp8_linear_fwd(x, w, ws, rounding=code)
    _ok(ops, dev)
    assert torch.equal(routed.view(torch.int16), want.view(torch.int16))
    if rounding == "infinity" and m * n * k <= 1000 * 3000 * 2048:
        _assert_output(got, O.mxfp8_linear(x.cpu(), w.cpu()))


def test_fused_x_glu_mlp_equals_the_chain(gpu):
    ops, N, dev, ws = gpu
    inp = O.make_inputs(2, m=600, k=512, inter=768)
    x, wgu, wd = (inp[key].to(dev) for key in ("x", "w_gate_up", "w_down"))
    h0, y0 = ops.mxfp8_glu_mlp_fwd(x, wgu, wd, ws)
    with ops.gemm_schedule("fused_x"):
        h1, y1 = ops.mxfp8_glu_mlp_fwd(x, wgu, wd, ws)
        _, y2 = ops.mxfp8_glu_mlp_fwd(x, wgu, wd, ws, want_hidden=False)
    _ok(ops, dev)
    assert torch.equal(h0, h1) and torch.equal(y0, y1) and torch.equal(y0, y2)


def test_fused_x_nan_row_stays_in_its_row(gpu):
    ops, N, dev, _ = gpu
    m, n, k = 384, 256, 384
    torch.manual_seed(5)
    x, w = torch.randn(m, k).bfloat16().to(dev), torch.randn(n, k).bfloat16().to(dev)
    qw, sw = ops.mxfp8_quantize(w)
    clean = ops.mxfp8_linear_fwd_fused_x(x, qw, sw, n)
    x[133, 0] = float("nan")
    got = ops.mxfp8_linear_fwd_fused_x(x, qw, sw, n)
    _ok(ops, dev)
    keep = torch.ones(m, dtype=torch.bool, device=dev)
    keep[133] = False
    assert torch.isnan(got[133].float()).all()
    assert torch.equal(got[keep].view(torch.int16), clean[keep].view(torch.int16))


@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("mnk_blocks", [((1024, 512, 1024), 4, 0), ((1024, 512, 1024), 4, 3), ((2048, 384, 96), 8, 5),
                                        ((768, 300, 256), 2, 1)])
def test_gemm_with_row_block_outputs_equals_the_plain_gemm(gpu, mnk_blocks, out_dtype):
    """The GEMM whose output rows are split over several buffers (on a multi-GPU node: the staging slots of the
    ranks that own the blocks) writes, block by block, the bits of the plain GEMM, whatever block the tile order
    starts at; a last block shorter than the others is clipped."""
    ops, N, dev, _ = gpu
    (m, n, k), n_blocks, first = mnk_blocks
    torch.manual_seed(13)
    a, b = torch.randn(m, k).bfloat16().to(dev), torch.randn(n, k).bfloat16().to(dev)
    qa, sa = ops.mxfp8_quantize(a)
    qb, sb = ops.mxfp8_quantize(b)
    want = ops.mxfp8_gemm(qa, sa, qb, sb, m, n, k, out_dtype=out_dtype)
    rows = 256 * max(1, -(-m // (256 * n_blocks)))      # rows per block: whole 256-row tiles
    ldo = (n + 7) // 8 * 8
    blocks = [torch.full((rows, ldo), float("nan"), dtype=out_dtype, device=dev)[:, :n] for _ in range(-(-m // rows))]
    ops.mxfp8_gemm_row_blocks(qa, sa, qb, sb, m, n, k, blocks, first_block=first)
    _ok(ops, dev)
    got = torch.cat([blk for blk in blocks], dim=0)[:m]
    assert torch.equal(got, want)
    if m % rows:
        assert torch.isnan(blocks[-1][m % rows:].float()).all()      # rows past m are never written
