"""The reference-facing Python API on a B200: modules, functionals, custom ops, autograd,
packed weights — compared with the CPU oracle (same bars as test_gpu_parity.py)."""
import pytest
import torch

from oracle import mx_oracle as O

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def dev(native_lib):
    if not torch.cuda.is_available():
        pytest.fail("these tests need a CUDA device")
    d = torch.device("cuda", 0)
    torch.cuda.set_device(d)
    return d


def _close(got, want, bit_exact=False):
    rep = O.parity_report(got.detach().cpu(), want)
    if bit_exact:
        assert rep["bit_equal"], rep
    assert rep["rel_fro"] <= 1e-3 and rep["frac_le_1ulp"] >= 0.999, rep


def _done(dev):
    from rtx_b200 import ops

    torch.cuda.synchronize()
    ops.check_device_status(dev)


def test_mxfp8_linear_module_forward_backward(dev):
    import rtx_b200 as rtx

    torch.manual_seed(0)
    layer = rtx.MXFP8Linear(160, 96, device=dev)
    x = torch.randn(2, 3, 64, 160).bfloat16().to(dev).requires_grad_(True)   # leading dims are flattened
    y = layer(x)
    assert y.shape == (2, 3, 64, 96) and y.dtype is torch.bfloat16
    w_cpu, x_cpu = layer.weight.detach().cpu(), x.detach().cpu()
    _close(y, O.mxfp8_linear(x_cpu, w_cpu))
    g = (torch.randn(2, 3, 64, 96) * 0.1).bfloat16().to(dev)
    y.backward(g)
    _done(dev)
    dx, dw = O.mxfp8_backward(x_cpu.reshape(-1, 160), w_cpu, g.cpu().reshape(-1, 96), dw_dtype=torch.float32)
    _close(x.grad.reshape(-1, 160), dx)
    _close(layer.weight.grad, dw.bfloat16())
    assert x.grad.dtype is torch.bfloat16 and layer.weight.grad.dtype is torch.bfloat16
    # no_grad path takes the inference op and gives the same bits
    with torch.no_grad():
        assert torch.equal(layer(x), y)


def test_only_one_gradient_requested(dev):
    import rtx_b200 as rtx

    torch.manual_seed(1)
    w = (torch.randn(64, 128) / 11).bfloat16().to(dev)
    x = torch.randn(96, 128).bfloat16().to(dev).requires_grad_(True)
    rtx.mxfp8_linear(x, w).sum().backward()
    _done(dev)
    g = torch.ones(96, 64).bfloat16()
    dx, _ = O.mxfp8_backward(x.detach().cpu(), w.cpu(), g)
    _close(x.grad, dx)


def test_mxfp8_packed_weight_states_are_bit_identical(dev):
    """rtx tests/test_mxfp8_quant.py:467-546: dynamic, weight-prequantized and fully-prequantized
    operands give the same bits, including a ragged shape with storage K = 64."""
    import rtx_b200 as rtx

    for (m, n, k) in ((128, 128, 256), (17, 29, 33)):
        torch.manual_seed(1702)
        x = torch.randn(m, k).bfloat16().to(dev)
        layer = rtx.MXFP8Linear(k, n, device=dev)
        y_dyn = layer(x)
        packed_layer = layer.to_quantized_weight()
        assert sorted(packed_layer.state_dict()) == ["weight_data", "weight_packing_meta", "weight_scales"]
        meta = packed_layer.weight_packing_meta.tolist()
        assert meta == [3, 2, k, (k + 31) // 32 * 32]
        y_wq = packed_layer(x)
        y_full = rtx.mxfp8_linear(rtx.quantize_mxfp8(x), packed_layer.packed_weight())
        _done(dev)
        assert torch.equal(y_dyn, y_wq) and torch.equal(y_dyn, y_full)
        # row-major scales from an interchange checkpoint are re-tiled on the fly
        from rtx_b200.configs import MXFP8QuantConfig

        rm = rtx.quantize_mxfp8(layer.weight.detach(), config=MXFP8QuantConfig(scale_layout="row_major"))
        assert torch.equal(rtx.mxfp8_linear(x, rm), y_dyn)
        with pytest.raises(TypeError, match="cannot be cast"):
            packed_layer.to(torch.float16)
        with pytest.raises(RuntimeError, match="inference-only"):
            packed_layer(x.clone().requires_grad_(True))


def test_quantize_mxfp8_tensor_matches_oracle(dev):
    import rtx_b200 as rtx
    from rtx_b200.configs import MXFP8QuantConfig

    torch.manual_seed(3)
    x = torch.randn(4, 40, 100).bfloat16()
    t = rtx.quantize_mxfp8(x.to(dev), config=MXFP8QuantConfig(scale_layout="row_major"))
    _done(dev)
    qo, so = O.mxfp8_quantize(x.reshape(-1, 100))
    assert tuple(t.shape) == (4, 40, 100)
    assert torch.equal(t.qdata.reshape(-1, 128).view(torch.uint8).cpu(), qo)
    assert torch.equal(t.scale.reshape(-1, 4).view(torch.uint8).cpu(), so)
    want = O.mxfp8_dequantize(qo, so)[:, :100].reshape(4, 40, 100)
    assert torch.equal(t.dequantize(torch.float32).cpu(), want)


def test_mxfp8_linear_backward_functional_and_packed_op(dev):
    import rtx_b200 as rtx
    from rtx_b200.fp8_bwd import unpack_bwd

    inp = O.make_inputs(4, m=256, n=128, k=192)
    x, w, dy = (inp[k].to(dev) for k in ("x", "w", "dy"))
    dx, dw = rtx.mxfp8_linear_backward(dy.reshape(2, 128, 128), x.reshape(2, 128, 192), w)
    flat = torch.ops.rtx.mxfp8_linear_bwd_packed(dy, x, w, rtx.MXFP8BwdConfig().to_key())
    _done(dev)
    dxo, dwo = O.mxfp8_backward(inp["x"], inp["w"], inp["dy"], dw_dtype=torch.float32)
    assert dx.shape == (2, 128, 192)
    _close(dx.reshape(-1, 192), dxo)
    _close(dw, dwo.bfloat16())
    dx2, dw2 = unpack_bwd(flat, (256, 192), (128, 192))
    assert torch.equal(dx2, dx.reshape(-1, 192)) and torch.equal(dw2, dw)


def test_nvfp4_linear_module_and_packed_weight(dev):
    import rtx_b200 as rtx

    torch.manual_seed(1905)
    layer = rtx.NVFP4Linear(256, 192, device=dev)
    assert layer.scaling == "jit_row_region"          # the reference's default for dynamic operands
    x = torch.randn(3, 50, 256).bfloat16().to(dev).requires_grad_(True)
    y = layer(x)
    w_cpu, x_cpu = layer.weight.detach().cpu(), x.detach().cpu()
    _close(y, O.nvfp4_linear_regions(x_cpu, w_cpu))    # 150 rows / 5, 192 rows / 4
    cur = rtx.NVFP4Linear(256, 192, device=dev, scaling="current")
    with torch.no_grad():
        cur.weight.copy_(layer.weight)
        _close(cur(x.detach()), O.nvfp4_linear(x_cpu, w_cpu, mode="power2"))
        _close(rtx.nvfp4_linear(x.detach(), layer.weight.detach(), scale_region_rows=6),
               O.nvfp4_linear_regions(x_cpu, w_cpu, 6, 6))
    g = (torch.randn(3, 50, 192) * 0.1).bfloat16().to(dev)
    y.backward(g)
    _done(dev)
    dx, dw = O.mxfp8_backward(x_cpu.reshape(-1, 256), w_cpu, g.cpu().reshape(-1, 192), dw_dtype=torch.float32)
    _close(x.grad.reshape(-1, 256), dx)          # NVFP4 forward, MXFP8 backward
    _close(layer.weight.grad, dw.bfloat16())
    # delayed policy: the first call bootstraps the histories from its own operands (= current scaling, power
    # of two); the second call still uses the first call's |max| although its activations are 4x larger
    dly = rtx.NVFP4Linear(256, 192, device=dev, scaling="delayed")
    with torch.no_grad():
        dly.weight.copy_(layer.weight)
    xg = x.detach().clone().requires_grad_(True)
    y1 = dly(xg)
    _close(y1, O.nvfp4_linear(x_cpu, w_cpu, mode="power2"))
    y1.backward(g)
    _close(xg.grad.reshape(-1, 256), dx)
    x4 = (x_cpu * 4).bfloat16()
    with torch.no_grad():
        y2 = dly(x4.to(dev))
    _done(dev)
    h_x = x_cpu.float().abs().amax().reshape(1).expand(16).clone()
    h_w = w_cpu.float().abs().amax().reshape(1).expand(16).clone()
    _, h_x, h_w = O.nvfp4_linear_delayed(x_cpu.reshape(-1, 256), w_cpu, h_x, h_w)
    want2, h_x, h_w = O.nvfp4_linear_delayed(x4.reshape(-1, 256), w_cpu, h_x, h_w)
    _close(y2.reshape(-1, 192), want2)
    assert torch.equal(dly._x_amax_state.cpu(), h_x) and float(h_x[0]) == float(x4.float().abs().amax())
    # block policy: outer scales are 1
    blk = rtx.NVFP4Linear(256, 192, device=dev, scaling="block")
    with torch.no_grad():
        blk.weight.copy_(layer.weight)
        yb = blk(x.detach())
    one = torch.ones(1)
    _close(yb, O.nvfp4_linear(x_cpu, w_cpu, x_scale=one, w_scale=one))
    # packed weight: exact outer scales for both operands (rtx/fp4.py:3421-3446)
    packed = layer.to_quantized_weight()
    assert sorted(packed.state_dict()) == ["weight_block_scales", "weight_data", "weight_packing_meta",
                                           "weight_tensor_scale"]
    with torch.no_grad():
        yp = packed(x.detach())
    _done(dev)
    x2 = x_cpu.reshape(-1, 256)
    want = O.nvfp4_linear(x2, w_cpu, x_scale=O.nvfp4_tensor_scale(x2, "exact"), w_scale=O.nvfp4_tensor_scale(w_cpu, "exact"))
    _close(yp.reshape(-1, 192), want)
    # decode-sized call through the packed module: one kernel quantizes the two rows and runs the GEMM
    base = rtx.NVFP4Linear(512, 192, device=dev, scaling="current")
    dec = base.to_quantized_weight()
    xs, wb = torch.randn(2, 512).bfloat16(), base.weight.detach().cpu()
    with torch.no_grad():
        yd = dec(xs.to(dev))
    _done(dev)
    _close(yd, O.nvfp4_linear(xs, wb, x_scale=O.nvfp4_tensor_scale(xs, "exact"),
                              w_scale=O.nvfp4_tensor_scale(wb, "exact")))
    t = rtx.quantize_nvfp4(layer.weight.detach())
    qo, so = O.nvfp4_quantize(w_cpu, O.nvfp4_tensor_scale(w_cpu, "exact"))
    assert torch.equal(t.qdata.view(torch.uint8).cpu().reshape(192, 128), qo)


def test_glu_mlp_functional(dev):
    import rtx_b200 as rtx

    inp = O.make_inputs(2, m=192, k=256, inter=384)
    x, wgu, wd = inp["x"], inp["w_gate_up"], inp["w_down"]
    y, h = rtx.mxfp8_glu_mlp(x.to(dev).reshape(3, 64, 256), wgu.to(dev), wd.to(dev), return_hidden=True)
    _done(dev)
    ho, _ = O.mxfp8_glu_mlp(x, wgu, wd)
    _close(h.reshape(-1, 384), ho)
    _close(y.reshape(-1, 256), O.mxfp8_linear(h.reshape(-1, 384).cpu(), wd))
    # a width the fused epilogue cannot pair takes the unfused composition
    inp = O.make_inputs(2, m=64, k=128, inter=96)
    y2 = rtx.mxfp8_glu_mlp(inp["x"].to(dev), inp["w_gate_up"].to(dev), inp["w_down"].to(dev))
    _done(dev)
    _, yo = O.mxfp8_glu_mlp(inp["x"], inp["w_gate_up"], inp["w_down"], fused_rounding=False)
    rep = O.parity_report(y2.cpu(), yo)
    assert rep["rel_fro"] < 2e-2, rep


def test_data_parallel_backward_single_rank(dev):
    import rtx_b200 as rtx

    inp = O.make_inputs(4, m=256, n=128, k=128)
    x, w, dy = (inp[k].to(dev) for k in ("x", "w", "dy"))
    dx, dw = rtx.data_parallel_linear_backward(dy, x, w)
    dx1, dw1 = rtx.mxfp8_linear_backward(dy, x, w)
    _done(dev)
    assert torch.equal(dx, dx1) and torch.equal(dw, dw1)   # FP32 -> BF16 once either way


def test_torch_compile_fullgraph_matches_eager(dev):
    """rtx tests/test_mxfp8_bwd.py:520-589: a compiled stack equals eager bit for bit."""
    import rtx_b200 as rtx

    torch.manual_seed(7)
    model = torch.nn.Sequential(rtx.MXFP8Linear(128, 256, device=dev), torch.nn.GELU(),
                                rtx.NVFP4Linear(256, 128, device=dev))
    x = torch.randn(64, 128).bfloat16().to(dev)
    from rtx_b200 import inductor

    before = dict(inductor.CALLS)
    with torch.no_grad():
        eager = model(x)
        compiled = torch.compile(model, fullgraph=True, dynamic=False)(x)
    _done(dev)
    assert torch.equal(eager, compiled)
    # the compiled graph reaches the kernels through the Inductor lowerings (extern kernels writing into
    # Inductor's buffers), not through the custom-op dispatcher
    if all(inductor._DONE.get(g) for g in ("mxfp8", "nvfp4")):
        assert inductor.CALLS.get("mxfp8_fwd", 0) > before.get("mxfp8_fwd", 0)
        assert inductor.CALLS.get("nvfp4_jit_row_region_fwd", 0) > before.get("nvfp4_jit_row_region_fwd", 0)
    # training step through the compiled module: same gradients as eager
    def grads(mod):
        for p in model.parameters():
            p.grad = None
        xx = x.clone().requires_grad_(True)
        mod(xx).float().square().mean().backward()
        return [xx.grad.clone()] + [p.grad.clone() for p in model.parameters()]

    want = grads(model)
    before = dict(inductor.CALLS)
    got = grads(torch.compile(model, fullgraph=True, dynamic=False))
    _done(dev)
    for a, b in zip(want, got):
        assert torch.equal(a, b)
    # the backward of both layers is MXFP8 and reaches its kernels through the backward lowerings too
    if inductor._DONE.get("mxfp8_bwd"):
        assert inductor.CALLS.get("mxfp8_bwd", 0) >= before.get("mxfp8_bwd", 0) + 2


def test_runtime_caches_clear(dev):
    import rtx_b200 as rtx

    rtx.mxfp8_linear(torch.zeros(32, 32, dtype=torch.bfloat16, device=dev), torch.zeros(32, 32, dtype=torch.bfloat16, device=dev))
    released = rtx.clear_runtime_caches()
    assert released["fp8"]["workspaces"]["entries"] >= 1
    assert rtx.validate_runtime_environment(require_device=True)["capability"][0] == 10


def test_quantize_model_in_place(dev):
    """`quantize_` (rtx/ptq.py:292-384): packed inference modules replace the BF16 linears, the packed
    forward equals the oracle with exact outer scales, and the BF16 masters are gone."""
    import rtx_b200 as rtx
    from torch import nn

    torch.manual_seed(3)
    model = nn.Sequential(nn.Linear(256, 192, bias=False, dtype=torch.bfloat16),
                          nn.Linear(192, 128, bias=False, dtype=torch.bfloat16)).to(dev)
    w0 = model[0].weight.detach().cpu()
    x = torch.randn(40, 256).bfloat16()
    fp4 = rtx.quantize_(nn.Sequential(*[nn.Linear(l.in_features, l.out_features, bias=False, dtype=torch.bfloat16,
                                                   device=dev) for l in model]), rtx.NVFP4WeightOnlyConfig())
    assert all(isinstance(l, rtx.NVFP4Linear) and l.weight is None for l in fp4)
    mx = rtx.quantize_(model, rtx.MXFP8WeightOnlyConfig(), filter_fn=lambda m, fqn: fqn == "0")
    assert isinstance(mx[0], rtx.MXFP8Linear) and mx[0].weight_mode == "prequantized" and type(mx[1]) is nn.Linear
    assert "0.weight" not in mx.state_dict() and "0.weight_data" in mx.state_dict()
    with torch.no_grad():
        y = mx[0](x.to(dev))
    _done(dev)
    _close(y, O.mxfp8_linear(x, w0))


def test_out_overloads_write_into_given_tensors(dev):
    """Launch-only variants (rtx/fp8.py:648-680, rtx/fp8_bwd.py:1145-1248): same bits as the functional ops,
    written into tensors the caller owns."""
    import rtx_b200 as rtx  # noqa: F401  (registers the ops)
    from rtx_b200 import fp8_bwd  # noqa: F401
    from rtx_b200.configs import MXFP8BwdConfig, MXFP8PrequantConfig

    torch.manual_seed(21)
    fk, bk = MXFP8PrequantConfig().to_key(), MXFP8BwdConfig().to_key()
    x = torch.randn(96, 160).bfloat16().to(dev)
    w = (torch.randn(128, 160) / 12).bfloat16().to(dev)
    g = (torch.randn(96, 128) * 0.1).bfloat16().to(dev)
    y = torch.ops.rtx.mxfp8_linear_fwd(x, w, fk)
    y_buf = torch.zeros_like(y)
    torch.ops.rtx.mxfp8_linear_fwd_out(x, w, fk, y_buf)
    dx, dw = torch.ops.rtx.mxfp8_linear_bwd(g, x, w, bk)
    dx_buf, dw_buf = torch.zeros_like(x), torch.zeros_like(w)
    torch.ops.rtx.mxfp8_linear_bwd.out(g, x, w, bk, grad_x=dx_buf, grad_weight=dw_buf)
    dx2, dw2 = torch.zeros_like(x), torch.zeros_like(w)
    torch.ops.rtx.mxfp8_linear_dx.out(g, x, w, bk, grad_x=dx2)
    torch.ops.rtx.mxfp8_linear_dw.out(g, x, w, bk, grad_weight=dw2)
    _done(dev)
    assert torch.equal(y, y_buf)
    assert torch.equal(dx, dx_buf) and torch.equal(dw, dw_buf)
    assert torch.equal(dx, dx2) and torch.equal(dw, dw2)
    assert torch.equal(dx, torch.ops.rtx.mxfp8_linear_dx(g, x, w, bk))
    assert torch.equal(dw, torch.ops.rtx.mxfp8_linear_dw(g, x, w, bk))


def test_swiglu_block_fused_inference_and_training(dev):
    """The decoder's feed-forward block (rtx/models/decoder.py:349-384): inference takes the fused pipeline
    (also under torch.compile), training the two modules with SiLU * up between them; same parameters."""
    import rtx_b200 as rtx

    torch.manual_seed(31)
    blk = rtx.SwiGLU(256, 384, device=dev)
    assert list(blk.state_dict()) == ["gate_up_proj.weight", "down_proj.weight"]
    assert blk.gate_up_proj.weight.shape == (768, 256) and blk.down_proj.weight.shape == (256, 384)
    x = torch.randn(2, 70, 256).bfloat16().to(dev)
    with torch.no_grad():
        y = blk(x)
        y_c = torch.compile(blk, fullgraph=True, dynamic=False)(x)
    _done(dev)
    want = O.mxfp8_glu_mlp(x.cpu().reshape(-1, 256), blk.gate_up_proj.weight.detach().cpu(),
                           blk.down_proj.weight.detach().cpu())
    want = want[1] if isinstance(want, tuple) else want
    _close(y.reshape(-1, 256), want)
    assert torch.equal(y, y_c)
    # training: unfused composition, gradients reach both projections
    xg = x.clone().requires_grad_(True)
    blk(xg).float().square().mean().backward()
    _done(dev)
    assert xg.grad is not None and blk.gate_up_proj.weight.grad is not None and blk.down_proj.weight.grad is not None
    assert torch.isfinite(blk.down_proj.weight.grad.float()).all()
    # the other projection kinds share the parameter layout
    nv = rtx.SwiGLU(256, 384, linear="nvfp4", device=dev)
    nv.load_state_dict(blk.state_dict())
    with torch.no_grad():
        yn = nv(x)
    _done(dev)
    assert yn.shape == y.shape and torch.isfinite(yn.float()).all()


def test_autotune_picks_among_the_built_kernels(dev, tmp_path):
    """The schedule in a config selects the kernel that runs: every candidate of the adapter, passed through
    the functional API, returns the same bits; `pick` times them on the device, stores the winner under the
    reference's key scheme and a later `cache` lookup returns it (rtx/autotune/core.py:167-293,
    rtx/autotune/winners.py:26-45)."""
    import rtx_b200 as rtx
    from rtx_b200 import autotune as A

    m, n, k = 96, 2048, 1024
    torch.manual_seed(5)
    x = torch.randn(m, k).bfloat16().to(dev)
    w = (torch.randn(n, k) / k ** 0.5).bfloat16().to(dev)
    adapter = A.make_mxfp8_prequant_fwd_adapter()
    ctx = A.KernelContext("mxfp8_prequant_fwd", m, n, k)
    cands = adapter.candidates(ctx)
    assert [c.gemm.schedule for c in cands] == ["auto", "single", "pair", "stream", "fused_x"]
    outs = {}

    def evaluate(cfg):
        with torch.no_grad():
            outs[cfg.gemm.schedule] = rtx.mxfp8_linear(x, w, dynamic_config=cfg).clone()
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            for _ in range(5):
                rtx.mxfp8_linear(x, w, dynamic_config=cfg)
            stop.record()
        stop.synchronize()
        return A.TrialOutcome("ok", median_ms=start.elapsed_time(stop) / 5)

    best = A.pick(ctx, adapter, evaluate, mode="balanced", cache_dir=tmp_path)
    _done(dev)
    assert set(outs) == {"auto", "single", "pair", "stream", "fused_x"}
    for name, out in outs.items():
        assert torch.equal(out, outs["auto"]), name
    _close(outs["auto"], O.mxfp8_linear(x.cpu(), w.cpu()))
    assert A.pick(ctx, adapter, None, mode="cache", cache_dir=tmp_path) == best
    # NVFP4: the three policies accept a schedule through their forward config
    nv = A.make_nvfp4_dynamic_fwd_adapter()
    ref = None
    for cfg in nv.candidates(A.KernelContext("nvfp4_dynamic_fwd", m, n, k)):
        with torch.no_grad():
            y = rtx.nvfp4_linear(x, w, scaling="current", dynamic_config=cfg)
        _done(dev)
        ref = y if ref is None else ref
        assert torch.equal(y, ref), cfg.gemm.schedule


def test_module_tunes_on_first_use_and_reuses_the_stored_winner(dev, tmp_path):
    """`autotune="balanced"` on the module: the first call with a new M times the legal schedules on the
    call's own operands and stores the winner; a second module in `cache` mode picks it up; outputs are
    the bits of an untuned module whatever schedule won (rtx/fp8.py:804-886, 2302-2386)."""
    import rtx_b200 as rtx
    from rtx_b200 import autotune as A

    torch.manual_seed(11)
    k, n = 512, 768
    plain = rtx.MXFP8Linear(k, n, device=dev)
    tuned = rtx.MXFP8Linear(k, n, device=dev, autotune="balanced", autotune_cache_dir=tmp_path)
    cached = rtx.MXFP8Linear(k, n, device=dev, autotune="cache", autotune_cache_dir=tmp_path)
    packed = rtx.MXFP8Linear(k, n, device=dev, autotune="balanced", autotune_cache_dir=tmp_path,
                             packed_weight=rtx.quantize_mxfp8(plain.weight.detach()))
    with torch.no_grad():
        tuned.weight.copy_(plain.weight)
        cached.weight.copy_(plain.weight)
        x = torch.randn(320, k).bfloat16().to(dev)
        want = plain(x)
        got = tuned(x)
        again = tuned(x)
        _done(dev)
        path = A.runtime_winner_path(A.KernelContext("mxfp8_prequant_fwd", 320, n, k), tmp_path)
        assert path.exists()
        assert tuned.explain(m=320)["schedule_source"] == "tuned on first use"
        assert cached.explain(m=320)["schedule_source"] == "stored winner"
        assert cached.explain(m=320)["gemm_schedule"] == tuned.explain(m=320)["gemm_schedule"]
        assert torch.equal(got, want) and torch.equal(again, want) and torch.equal(cached(x), want)
        assert torch.equal(packed(x), want)          # the packed-weight state tunes its own family variant
        assert A.runtime_winner_path(A.KernelContext("mxfp8_prequant_fwd", 320, n, k, variant="weight_prequant"),
                                     tmp_path).exists()
    _done(dev)
    # training through a tuned module: the winner's key travels into the autograd op
    xg = torch.randn(320, k).bfloat16().to(dev).requires_grad_(True)
    tuned(xg).sum().backward()
    _done(dev)
    assert xg.grad is not None and tuned.weight.grad is not None


def test_nvfp4_module_tunes_on_first_use(dev, tmp_path):
    """`autotune="balanced"` on NVFP4Linear (row-region policy and packed weight): first call times the built
    schedules, stores a winner per (family, policy variant), later calls reuse it; same bits as an untuned module."""
    import rtx_b200 as rtx
    from rtx_b200 import autotune as A

    torch.manual_seed(12)
    k, n = 512, 1024
    plain = rtx.NVFP4Linear(k, n, device=dev)
    tuned = rtx.NVFP4Linear(k, n, device=dev, autotune="balanced", autotune_cache_dir=tmp_path)
    with torch.no_grad():
        tuned.weight.copy_(plain.weight)
        x = torch.randn(96, k).bfloat16().to(dev)
        want = plain(x)
        got, again = tuned(x), tuned(x)
        _done(dev)
        assert torch.equal(got, want) and torch.equal(again, want)
        assert A.runtime_winner_path(A.KernelContext("nvfp4_dynamic_fwd", 96, n, k, variant="jit_row_region"),
                                     tmp_path).exists()
        assert tuned.explain(m=96)["schedule_source"] == "tuned on first use"
        packed_plain = plain.to_quantized_weight()
        packed = rtx.NVFP4Linear(k, n, device=dev, autotune="balanced", autotune_cache_dir=tmp_path,
                                 packed_weight=packed_plain.packed_weight())
        assert torch.equal(packed(x), packed_plain(x))
        assert A.runtime_winner_path(A.KernelContext("nvfp4_weight_prequant_fwd", 96, n, k, variant="current"),
                                     tmp_path).exists()
    _done(dev)


def test_campaign_over_a_manifest_installs_winners_the_modules_find(dev, tmp_path):
    """A campaign in the reference's manifest format (autotune_manifests/*.json) over every tunable family:
    each target gets a winner whose output passed the bit-equality gate, stored where a module with
    autotune="cache" looks it up; the backward family is reported as skipped."""
    import json

    import rtx_b200 as rtx
    from rtx_b200 import campaign

    manifest = campaign.Manifest.from_dict({
        "schema_version": 2, "name": "gpu_unit", "seed": 5,
        "jobs": [{"family": f, "shapes": [{"m": 96, "n": 512, "k": 512, "name": "small"}], "regimes": regimes,
                  "promote": 2, "protocol": {"warmup_calls": 1, "samples": 3, "confirm_samples": 3}}
                 for f, regimes in (("mxfp8_prequant_fwd", ["hot", "rotate"]), ("mxfp8_weight_prequant_fwd", ["hot"]),
                                    ("nvfp4_dynamic_fwd", ["hot"]), ("nvfp4_jit_row_region_fwd", ["hot"]),
                                    ("nvfp4_delayed_fwd", ["hot"]), ("nvfp4_weight_prequant_fwd", ["hot"]),
                                    ("mxfp8_bwd", ["hot"]))]})
    summary = campaign.run_campaign(manifest, tmp_path / "out", cache_dir=tmp_path / "cache")
    _done(dev)
    assert [s["family"] for s in summary["skipped"]] == ["mxfp8_bwd"]
    assert len(summary["targets"]) == 7
    for t in summary["targets"]:
        assert t["decision"] == "winner" and "installed" in t, t
    trials = [json.loads(l) for l in open(tmp_path / "out" / "gpu_unit" / "trials.jsonl")]
    assert all(t["status"] == "ok" for t in trials), [t for t in trials if t["status"] != "ok"]
    # M = 96 admits every built schedule: 5 MXFP8 candidates (auto, single, pair, stream, fused_x), 4 NVFP4
    searched = [t for t in trials if t["phase"] == "search" and t["family"] == "mxfp8_prequant_fwd" and
                t["regime"] == "hot" and t["variant"] == "default"]
    assert len(searched) == 5
    for mod in (rtx.MXFP8Linear(512, 512, device=dev, autotune="cache", autotune_cache_dir=tmp_path / "cache"),
                rtx.NVFP4Linear(512, 512, device=dev, autotune="cache", autotune_cache_dir=tmp_path / "cache"),
                rtx.NVFP4Linear(512, 512, device=dev, scaling="delayed", autotune="cache",
                                autotune_cache_dir=tmp_path / "cache")):
        assert mod.explain(m=96)["schedule_source"] == "stored winner"
        assert mod.explain(m=128)["schedule_source"] == "configured (no stored winner)"


@pytest.mark.parametrize("chunk_rows", [None, 0, 256, 512])
def test_host_session_returns_the_bits_of_the_device_call(dev, chunk_rows):
    """`GluMlpHostSession` (host buffers in, host buffers out): whole-step and row-block pipelining give the
    bits of the device-resident MLP call, over several steps that re-use the buffer sets, ragged last block."""
    from rtx_b200 import ops
    from rtx_b200.host import GluMlpHostSession

    torch.manual_seed(21)
    m, k, inter, n_out = 1200, 512, 768, 384
    wgu = (torch.randn(2 * inter, k) / k ** 0.5).bfloat16().to(dev)
    wd = (torch.randn(n_out, inter) / inter ** 0.5).bfloat16().to(dev)
    session = GluMlpHostSession(wgu, wd, m, chunk_rows=chunk_rows)
    ws = ops.Workspace(dev)
    xs = [torch.randn(m if i != 2 else 700, k).bfloat16().pin_memory() for i in range(5)]
    ys = [torch.empty(x.shape[0], n_out, dtype=torch.bfloat16).pin_memory() for x in xs]
    for x, y in zip(xs, ys):
        session.submit(x, y)
    session.drain()
    assert session.launches_per_step == (2 + 3 * -(-1200 // chunk_rows) if chunk_rows else 5)   # the last step: 1200 rows
    for x, y in zip(xs, ys):
        _, want = ops.mxfp8_glu_mlp_fwd(x.to(dev), wgu, wd, ws, want_hidden=False)
        assert torch.equal(y, want.cpu())
    _done(dev)


def test_backend_fused_runs_the_in_kernel_quantizer_and_gives_the_same_bits(dev):
    """`backend="fused"` (module and function): the reference's one-kernel forward, here the CTA-pair GEMM whose own
    warps quantize the activations; bit-identical to the materialized pipeline, forward and through autograd."""
    import rtx_b200 as rtx

    torch.manual_seed(17)
    k, n = 512, 768
    plain = rtx.MXFP8Linear(k, n, device=dev)
    fused = rtx.MXFP8Linear(k, n, device=dev, backend="fused")
    with torch.no_grad():
        fused.weight.copy_(plain.weight)
    assert fused.explain()["backend"] == "fused"
    x = torch.randn(3, 100, k, device=dev).bfloat16()
    with torch.no_grad():
        want = plain(x)
        assert torch.equal(fused(x), want)
        assert torch.equal(rtx.mxfp8_linear(x, plain.weight, backend="fused"), want)
        packed = fused.to_quantized_weight()
        assert torch.equal(packed(x), want)
    xa, xb = x.clone().requires_grad_(True), x.clone().requires_grad_(True)
    ya, yb = plain(xa), fused(xb)
    ya.float().sum().backward()
    yb.float().sum().backward()
    assert torch.equal(ya, yb) and torch.equal(xa.grad, xb.grad) and torch.equal(plain.weight.grad, fused.weight.grad)
    _done(dev)


def test_quantized_weight_cache_is_bit_identical(dev):
    """Inside `quantized_weight_cache()` modules reuse the quantized weight across micro-batches; outputs,
    dX and accumulated dW equal the uncached run bit for bit, an in-place weight update is seen, and the
    scope saves exactly the weight quantizer launches."""
    import rtx_b200 as rtx

    torch.manual_seed(77)
    xs = [torch.randn(3, 50, 256).bfloat16().to(dev) for _ in range(3)]

    def run(module, cached):
        module.zero_grad(set_to_none=True)
        outs, dxs = [], []
        scope = rtx.quantized_weight_cache() if cached else None
        cache = scope.__enter__() if cached else None
        try:
            for x in xs:
                xg = x.clone().requires_grad_(True)
                y = module(xg)
                y.float().square().mean().backward()
                outs.append(y.detach().clone())
                dxs.append(xg.grad.clone())
            with torch.no_grad():
                outs.append(module(xs[0]).clone())
        finally:
            if cached:
                scope.__exit__(None, None, None)
        _done(dev)
        return outs, dxs, module.weight.grad.clone(), (cache.stats.copy() if cached else None)

    for make in (lambda: rtx.MXFP8Linear(256, 384, device=dev), lambda: rtx.NVFP4Linear(256, 384, device=dev)):
        module = make()
        outs0, dxs0, dw0, _ = run(module, False)
        outs1, dxs1, dw1, stats = run(module, True)
        for a, b in zip(outs0 + dxs0 + [dw0], outs1 + dxs1 + [dw1]):
            assert torch.equal(a, b)
        # forward operand: 1 miss + 3 hits; dX operand: 1 miss + 2 hits
        assert stats == {"hits": 5, "misses": 2}, stats
        # an optimizer-style update inside a scope is seen through the version counter
        with rtx.quantized_weight_cache() as cache:
            with torch.no_grad():
                before = module(xs[0]).clone()
                module.weight.mul_(0.5)
                after = module(xs[0]).clone()
            assert cache.stats["misses"] == 2
        with torch.no_grad():
            want = module(xs[0])
        _done(dev)
        assert torch.equal(after, want) and not torch.equal(before, after)

    # the fused SwiGLU inference path
    blk = rtx.SwiGLU(256, 384, device=dev)
    with torch.no_grad():
        want = blk(xs[0])
        with rtx.quantized_weight_cache() as cache:
            got = [blk(xs[0]).clone() for _ in range(2)]
        assert cache.stats == {"hits": 2, "misses": 2}
    _done(dev)
    assert torch.equal(got[0], want) and torch.equal(got[1], want)
    # under torch.compile the scope is ignored, not traced
    lin = rtx.MXFP8Linear(256, 384, device=dev)
    with torch.no_grad(), rtx.quantized_weight_cache() as cache:
        y_c = torch.compile(lin, fullgraph=True, dynamic=False)(xs[0])
        y_e = lin(xs[0])
    _done(dev)
    assert torch.equal(y_c, y_e)
