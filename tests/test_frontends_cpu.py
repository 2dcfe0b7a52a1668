"""CPU contract tests of the Python boundary (mirrors rtx tests/test_linear_frontends.py,
test_runtime_contract.py and the config halves of test_mxfp8_fwd.py / test_nvfp4.py):
no GPU, no kernel launch."""
import json
import os
import subprocess
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_lazy_import_touches_neither_cuda_nor_the_library():
    code = ("import sys; sys.path.insert(0, %r); import rtx_b200; "
            "assert 'rtx_b200.fp8' not in sys.modules and 'rtx_b200._native' not in sys.modules; "
            "assert 'MXFP8Linear' in dir(rtx_b200); print(rtx_b200.__version__)") % ROOT
    out = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=120)
    assert out.returncode == 0, out.stderr
    with pytest.raises(AttributeError):
        import rtx_b200

        rtx_b200.not_a_symbol


def test_public_names_match_the_reference_surface():
    import rtx_b200

    for name in ("MXFP8Linear", "NVFP4Linear", "mxfp8_linear", "nvfp4_linear", "quantize_mxfp8", "quantize_nvfp4",
                 "mxfp8_linear_backward", "MXTensor", "MXFP8Tensor", "NVFP4Tensor", "MXFP8QuantConfig",
                 "MXFP8GemmConfig", "MXFP8FwdConfig", "MXFP8Problem", "MXFP8BwdConfig", "NVFP4QuantConfig",
                 "NVFP4GemmConfig", "NVFP4Problem", "clear_runtime_caches", "validate_runtime_environment",
                 "DEFAULT_MXFP8_BWD_CONFIG", "DEFAULT_NVFP4_X_SCALE_REGION_ROWS"):
        assert getattr(rtx_b200, name) is not None


def test_configs_round_trip_and_reject_explicitly():
    from rtx_b200 import configs as C

    for cfg in (C.MXFP8FwdConfig(), C.MXFP8PrequantConfig(), C.MXFP8BwdConfig(streams="dual_stream"),
                C.NVFP4DynamicConfig(), C.MXFP8QuantConfig(scale_rounding="floor", scale_layout="row_major")):
        key = cfg.to_key()
        assert json.loads(key)["type"] == type(cfg).__name__
        assert C.config_from_key(key) == cfg
        assert hash(cfg) == hash(C.config_from_key(key))
    assert C.MXFP8QuantConfig(scale_layout="mma64").rejection(128, 128).startswith("mma64")
    assert "rounding" in C.MXFP8QuantConfig(scale_rounding="nearest").rejection(1, 1)
    assert "no kernel is built" in C.MXFP8GemmConfig(tile_n=128).rejection()
    assert C.MXFP8GemmConfig(tile_m=256, cta_group=2, stages=6).rejection() is None
    assert C.MXFP8GemmConfig().rejection(C.MXFP8Problem(0, 1, 1)) == "m, n and k must be positive"
    # a named schedule selects one built kernel and must state that kernel's tile shape
    for name in ("single", "pair", "stream"):
        assert C.MXFP8GemmConfig.for_schedule(name).rejection() is None
        assert C.NVFP4GemmConfig.for_schedule(name).rejection() is None
        assert C.config_from_key(C.MXFP8GemmConfig.for_schedule(name).to_key()).schedule == name
    assert "unknown GEMM schedule" in C.MXFP8GemmConfig(schedule="wide").rejection()
    assert "tile shape" in C.MXFP8GemmConfig(schedule="pair").rejection()
    assert "M <= 128" in C.MXFP8GemmConfig.for_schedule("stream").rejection(C.MXFP8Problem(256, 64, 64))
    assert "M <= 128" in C.NVFP4GemmConfig.for_schedule("stream").rejection(C.NVFP4Problem(256, 64, 64))
    assert C.MXFP8FwdConfig(pipeline="fused").rejection() == "forward pipeline 'fused' is not built"
    assert C.NVFP4ScaleConfig(policy="delayed").rejection() is None
    assert "history_len" in C.NVFP4ScaleConfig(policy="delayed", amax_history_len=3).rejection()
    assert "history_algo" in C.NVFP4ScaleConfig(policy="delayed", amax_history_algo="mean").rejection()
    assert "unknown NVFP4 scaling policy" in C.NVFP4ScaleConfig(policy="per_channel").rejection()
    assert C.NVFP4ScaleConfig(policy="jit_row_region").rejection() is None
    # region sizes travel in the forward schedule and go with the jit_row_region policy only
    region = C.NVFP4DynamicConfig(scale=C.NVFP4ScaleConfig(policy="jit_row_region"), x_scale_region_rows=5,
                                  weight_scale_region_rows=4)
    assert region.rejection() is None and region.jit_row_region
    assert C.config_from_key(region.to_key()) == region
    assert "both operands" in C.NVFP4DynamicConfig(scale=C.NVFP4ScaleConfig(policy="jit_row_region"),
                                                   x_scale_region_rows=5).rejection()
    assert "only with it" in C.NVFP4DynamicConfig(x_scale_region_rows=5, weight_scale_region_rows=4).rejection()
    assert "only with it" in C.NVFP4DynamicConfig(scale=C.NVFP4ScaleConfig(policy="jit_row_region")).rejection()
    assert C.NVFP4QuantConfig(scale_reciprocal="rcp_approx").rejection() is not None
    assert C.MXFP8Problem(3, 5, 1).storage_k == 32 and C.NVFP4Problem(1, 1, 129).storage_k == 160
    assert C.MXFP8GemmConfig().smem_bytes() <= C.SMEM_CAPACITY_BYTES


def test_bounded_cache_lru_and_env_limits(monkeypatch):
    from rtx_b200.runtime import BoundedCache, runner_cache_limit

    cache = BoundedCache(2)
    cache["a"], cache["b"] = 1, 2
    assert cache["a"] == 1
    cache["c"] = 3                       # evicts b (least recently used)
    assert "b" not in cache and set(cache) == {"a", "c"}
    assert cache.get("zz") is None
    stats = cache.stats()
    assert stats["evictions"] == 1 and stats["hits"] == 1 and stats["misses"] >= 1 and stats["max_entries"] == 2
    zero = BoundedCache(0)
    zero["k"] = 1
    assert len(zero) == 0
    with pytest.raises(ValueError):
        BoundedCache(-1)
    monkeypatch.setenv("RTX_MXFP8_PREQUANT_CACHE_ENTRIES", "3")
    assert runner_cache_limit("prequant") == 3
    monkeypatch.setenv("RTX_MXFP8_PREQUANT_CACHE_ENTRIES", "x")
    with pytest.raises(ValueError, match="must be an integer"):
        runner_cache_limit("prequant")
    monkeypatch.delenv("RTX_MXFP8_PREQUANT_CACHE_ENTRIES")
    monkeypatch.setenv("RTX_NVFP4_RUNNER_CACHE_ENTRIES", "5")
    assert runner_cache_limit("dynamic", namespace="NVFP4") == 5


def test_runtime_environment_contract(native_lib):
    from rtx_b200.runtime import validate_runtime_environment

    facts = validate_runtime_environment()
    assert facts["abi_version"] >= 100 and facts["torch_cuda"]
    if not torch.cuda.is_available():
        with pytest.raises(RuntimeError, match="no CUDA device"):
            validate_runtime_environment(require_device=True)


def test_module_constructors_and_state_dict_schema():
    from rtx_b200 import MXFP8Linear, NVFP4Linear

    with pytest.raises(NotImplementedError):
        MXFP8Linear(8, 8, bias=True)
    with pytest.raises(TypeError):
        MXFP8Linear(8, 8, dtype=torch.float16)
    with pytest.raises(ValueError, match="unknown MXFP8 backend"):
        MXFP8Linear(8, 8, backend="cutlass")
    from rtx_b200.configs import MXFP8FwdConfig, MXFP8GemmConfig, MXFP8PrequantConfig, NVFP4ScaleConfig

    # backend="fused" = the reference's one-kernel forward: the GEMM that quantizes X itself, unless the config
    # already names a schedule; auto / materialized = quantize once, packed GEMM (rtx/fp8.py:292-312)
    import json as _json

    sched = lambda mod: _json.loads(mod._forward_config_key)["gemm"]["schedule"]
    assert sched(MXFP8Linear(64, 64, device="meta", backend="fused")) == "fused_x"
    assert sched(MXFP8Linear(64, 64, device="meta", backend="auto")) == "auto"
    assert sched(MXFP8Linear(64, 64, device="meta", backend="materialized")) == "auto"
    assert sched(MXFP8Linear(64, 64, device="meta", backend="fused",
                             dynamic_config=MXFP8PrequantConfig(gemm=MXFP8GemmConfig.for_schedule("pair")))) == "pair"

    with pytest.raises(ValueError, match="both config aliases"):
        MXFP8Linear(8, 8, config=MXFP8FwdConfig(), forward_config=MXFP8FwdConfig())
    with pytest.raises(ValueError, match="materialized config aliases"):
        MXFP8Linear(8, 8, prequant_config=MXFP8PrequantConfig(), dynamic_config=MXFP8PrequantConfig())
    layer = MXFP8Linear(64, 32)
    assert list(layer.state_dict()) == ["weight"] and layer.weight.dtype is torch.bfloat16
    assert layer.weight.shape == (32, 64) and layer.weight_mode == "dynamic"
    assert "weight_mode=dynamic" in repr(layer) and layer.explain()["format"] == "mxfp8"
    ref = torch.nn.Linear(64, 32, bias=False)
    assert torch.equal(MXFP8Linear.from_float(ref).weight, ref.weight.bfloat16())
    with pytest.raises(NotImplementedError):
        MXFP8Linear.from_float(torch.nn.Linear(4, 4, bias=True))
    nv = NVFP4Linear(64, 32)
    # dynamic operands default to the row-region policy with the asymmetric X = 5, W = 4 regions
    assert list(nv.state_dict()) == ["weight"] and nv.scaling == "jit_row_region"
    assert (nv.x_scale_region_rows, nv.weight_scale_region_rows) == (5, 4)
    assert nv._dynamic_config.x_scale_region_rows == 5 and nv.explain()["weight_scale_region_rows"] == 4
    shared = NVFP4Linear(8, 8, scale_region_rows=4, x_scale_region_rows=8)
    assert (shared.x_scale_region_rows, shared.weight_scale_region_rows) == (8, 4)
    assert NVFP4Linear(8, 8, scaling="current")._dynamic_config.x_scale_region_rows == 0
    with pytest.raises(ValueError, match="positive"):
        NVFP4Linear(8, 8, scale_region_rows=0)
    delayed = NVFP4Linear(8, 8, scaling="delayed", scale_config=NVFP4ScaleConfig(amax_history_len=4))
    assert delayed._dynamic_config.scale.policy == "delayed" and delayed._dynamic_config.scale.amax_history_len == 4
    assert not delayed._delayed_initialized and list(delayed.state_dict()) == ["weight"]   # histories are not state
    delayed._delayed_initialized = True
    delayed.load_state_dict(nv.state_dict() if nv.weight.shape == delayed.weight.shape else delayed.state_dict())
    assert not delayed._delayed_initialized          # loading a checkpoint drops the histories
    delayed._delayed_initialized = True
    delayed.eval()
    delayed.train()
    assert not delayed._delayed_initialized          # so does re-entering training
    with pytest.raises(ValueError):
        NVFP4Linear(8, 8, scaling="per_channel")
    # BF16 / MXFP8 / NVFP4 dynamic modules share checkpoints
    nv.load_state_dict(layer.state_dict())
    assert torch.equal(nv.weight, layer.weight)


def test_functional_argument_errors_before_any_launch():
    from rtx_b200 import mxfp8_linear, mxfp8_linear_backward, nvfp4_linear, quantize_mxfp8, quantize_nvfp4

    x, w = torch.zeros(4, 32, dtype=torch.bfloat16), torch.zeros(8, 32, dtype=torch.bfloat16)
    with pytest.raises(ValueError, match="CUDA"):
        mxfp8_linear(x, w)
    with pytest.raises(ValueError, match="K mismatch"):
        mxfp8_linear(x, torch.zeros(8, 64, dtype=torch.bfloat16))
    with pytest.raises(ValueError, match="unknown MXFP8 backend"):
        mxfp8_linear(x, w, backend="x")
    with pytest.raises(ValueError, match="CUDA"):
        quantize_mxfp8(x)
    with pytest.raises(TypeError):
        quantize_nvfp4(x.float())
    with pytest.raises(ValueError, match="CUDA"):
        nvfp4_linear(x, w, scaling="jit_row_region")
    with pytest.raises(ValueError, match="scaling must be"):
        nvfp4_linear(x, w, scaling="nope")
    assert callable(mxfp8_linear_backward)


def test_custom_ops_dispatch_on_fake_cuda_tensors():
    """rtx tests/test_linear_frontends.py:362-441: every op has a schema and a fake kernel."""
    from torch._subclasses.fake_tensor import FakeTensorMode

    import rtx_b200.fp4  # noqa: F401
    import rtx_b200.fp8  # noqa: F401
    import rtx_b200.fp8_bwd  # noqa: F401
    from rtx_b200.configs import MXFP8BwdConfig, MXFP8PrequantConfig, NVFP4DynamicConfig

    fk, bk, nk = MXFP8PrequantConfig().to_key(), MXFP8BwdConfig().to_key(), NVFP4DynamicConfig().to_key()
    with FakeTensorMode():
        x = torch.empty(48, 96, dtype=torch.bfloat16, device="cuda")
        w = torch.empty(80, 96, dtype=torch.bfloat16, device="cuda")
        g = torch.empty(48, 80, dtype=torch.bfloat16, device="cuda")
        s = torch.empty(1, dtype=torch.float32, device="cuda")
        ops = torch.ops.rtx
        assert ops.mxfp8_linear_fwd(x, w, fk).shape == (48, 80)
        assert ops.mxfp8_linear_prequant(x, w, fk).dtype is torch.bfloat16
        assert ops.mxfp8_linear_train(x, w, fk, bk).shape == (48, 80)
        dx, dw = ops.mxfp8_linear_bwd(g, x, w, bk)
        assert dx.shape == x.shape and dw.shape == w.shape and dw.dtype is torch.bfloat16
        assert ops.mxfp8_linear_bwd_packed(g, x, w, bk).numel() == 48 * 96 + 80 * 96
        assert ops.mxfp8_linear_dx(g, x, w, bk).shape == (48, 96)
        assert ops.mxfp8_linear_dw(g, x, w, bk).shape == (80, 96)
        dx_buf, dw_buf = torch.empty_like(x), torch.empty_like(w)
        got = torch.ops.rtx.mxfp8_linear_bwd.out(g, x, w, bk, grad_x=dx_buf, grad_weight=dw_buf)
        assert got[0] is dx_buf and got[1] is dw_buf
        assert torch.ops.rtx.mxfp8_linear_dx.out(g, x, w, bk, grad_x=dx_buf) is dx_buf
        assert torch.ops.rtx.mxfp8_linear_dw.out(g, x, w, bk, grad_weight=dw_buf) is dw_buf
        assert torch.ops.rtx.mxfp8_linear_fwd_out(x, w, fk, torch.empty(48, 80, dtype=torch.bfloat16, device="cuda")) is None
        assert torch.ops.rtx.mxfp8_linear_prequant_out(x, w, fk, torch.empty(48, 80, dtype=torch.bfloat16, device="cuda")) is None
        assert ops.mxfp8_linear_dw_f32(g, x, bk).dtype is torch.float32
        q = torch.empty(80, 96, dtype=torch.uint8, device="cuda")
        sc = torch.empty(512 * 1, dtype=torch.uint8, device="cuda")
        assert ops.mxfp8_linear_dynamic_x_prequant_w(x, q, sc, 80, 96, "mma128", fk).shape == (48, 80)
        assert ops.mxfp8_linear_prequantized(q, q, sc, sc, 80, 80, 96, "mma128", "mma128", fk).shape == (80, 80)
        assert ops.nvfp4_linear_materialized_fwd(x, w, s, s, s, nk).shape == (48, 80)
        assert ops.nvfp4_linear_materialized_train(x, w, s, s, s, nk, bk).shape == (48, 80)
        assert ops.nvfp4_linear_block_fwd(x, w, nk).shape == (48, 80)
        assert ops.nvfp4_linear_block_train(x, w, nk, bk).shape == (48, 80)
        assert ops.nvfp4_linear_dynamic_x_prequant_w(x, q, sc, s, s, 80, 96, "mma128", nk).shape == (48, 80)
        assert ops.nvfp4_linear_prequantized(q, q, sc, sc, s, 80, 80, 96, "mma128", "mma128", nk).shape == (80, 80)
    schema = str(torch.ops.rtx.mxfp8_linear_fwd.default._schema)
    assert "Tensor x, Tensor weight, str config_key" in schema
    # declared with the dispatcher directly (rtx_b200/_oplib.py): compile-safe tag, and no kernel for CPU tensors —
    # the product path has no CPU fallback
    assert torch.Tag.pt2_compliant_tag in torch.ops.rtx.mxfp8_linear_fwd.default.tags
    assert torch.Tag.pt2_compliant_tag in torch.ops.rtx.nvfp4_linear_prequant_w_current.default.tags
    with pytest.raises(NotImplementedError):
        torch.ops.rtx.mxfp8_linear_fwd(torch.zeros(32, 32, dtype=torch.bfloat16), torch.zeros(32, 32, dtype=torch.bfloat16), fk)


def test_scale_layout_conversion_matches_the_oracle():
    from oracle import mx_oracle as O
    from rtx_b200.formats import scales_mma128_to_row_major, scales_row_major_to_mma128

    s = (torch.arange(300 * 9) % 251).to(torch.uint8).reshape(300, 9)
    tiles = scales_row_major_to_mma128(s, 300, 9, 3)
    assert torch.equal(tiles.reshape(3, 3, 512), O.scales_to_mma128(s))
    assert torch.equal(scales_mma128_to_row_major(tiles, 300, 9, 3), s)
    # NVFP4: tiles along K padded to whole 256-value K steps (4 tiles)
    s4 = (torch.arange(130 * 10) % 200).to(torch.uint8).reshape(130, 10)
    tiles4 = scales_row_major_to_mma128(s4, 130, 10, 4)
    assert tiles4.numel() == 2 * 4 * 512
    assert torch.equal(scales_mma128_to_row_major(tiles4, 130, 10, 4), s4)


def test_packed_tensor_containers_validate_storage():
    from rtx_b200.formats import make_mxfp8_tensor, make_nvfp4_tensor, mxfp8_scale_layout

    q = torch.zeros(8, 64, dtype=torch.uint8)
    t = make_mxfp8_tensor(q, torch.zeros(8 * 2, dtype=torch.uint8), (2, 4, 40), "row_major")
    assert tuple(t.shape) == (2, 4, 40) and t.qdata.shape == (2, 4, 64) and t.block_size == 32
    assert t.scale.dtype is torch.float8_e8m0fnu and mxfp8_scale_layout(t) == "row_major"
    with pytest.raises(ValueError, match="expected"):
        make_mxfp8_tensor(q, torch.zeros(7, dtype=torch.uint8), (8, 40), "row_major")
    with pytest.raises(ValueError, match="mma64"):
        make_mxfp8_tensor(q, torch.zeros(512, dtype=torch.uint8), (8, 40), "mma64")
    nv = make_nvfp4_tensor(torch.zeros(8, 16, dtype=torch.uint8), torch.zeros(8 * 2, dtype=torch.uint8),
                           torch.ones(1), (8, 17), "row_major")
    assert nv.block_size == 16 and tuple(nv.shape) == (8, 17)
    with pytest.raises(ValueError, match="storage K"):
        make_nvfp4_tensor(torch.zeros(8, 8, dtype=torch.uint8), torch.zeros(8, dtype=torch.uint8), torch.ones(1),
                          (8, 17), "row_major")


def test_autotune_adapter_and_winner_cache(tmp_path):
    from rtx_b200 import autotune as A

    adapter = A.make_mxfp8_prequant_fwd_adapter()
    assert isinstance(adapter, A.KernelAdapter)
    ctx = A.KernelContext("mxfp8_prequant_fwd", 8192, 28672, 4096)
    cands = adapter.candidates(ctx)
    # the library's own choice plus one candidate per built kernel that serves the shape
    assert [c.gemm.schedule for c in cands] == ["auto", "single", "pair", "fused_x"]
    assert all(adapter.rejection(c, ctx) is None for c in cands)
    small = adapter.candidates(A.KernelContext("mxfp8_prequant_fwd", 64, 8192, 4096))
    assert [c.gemm.schedule for c in small] == ["auto", "single", "pair", "stream", "fused_x"]
    nv = A.make_nvfp4_dynamic_fwd_adapter()
    assert [c.gemm.schedule for c in nv.candidates(A.KernelContext("nvfp4_dynamic_fwd", 8, 8192, 8192))] == [
        "auto", "single", "pair", "stream"]
    assert adapter.decode(adapter.encode(cands[1])) == cands[1]
    assert A.pick(ctx, adapter, None, mode="off") == adapter.default(ctx)
    assert A.pick(ctx, adapter, None, mode="cache", cache_dir=tmp_path) == adapter.default(ctx)
    times = {adapter.encode(cands[0]): 2.0, adapter.encode(cands[1]): 1.0, adapter.encode(cands[2]): 1.5,
             adapter.encode(cands[3]): 9.0}
    calls = []

    def evaluate(cfg):
        calls.append(cfg)
        return A.TrialOutcome("ok", median_ms=times[adapter.encode(cfg)])

    best = A.pick(ctx, adapter, evaluate, mode="balanced", cache_dir=tmp_path)
    assert best == cands[1] and len(calls) == 4
    path = A.runtime_winner_path(ctx, tmp_path)
    assert path.name == "m8192_n28672_k4096_hot_default_rev1.json" and path.parent.name == "b200"
    assert A.pick(ctx, adapter, None, mode="cache", cache_dir=tmp_path) == cands[1]
    assert set(A.ADAPTERS) == set(A.FAMILIES)
    failing = A.pick(A.KernelContext("mxfp8_prequant_fwd", 1, 1, 1), adapter,
                     lambda c: A.TrialOutcome("failed", detail="x"), mode="balanced", cache_dir=tmp_path)
    assert failing == adapter.default(ctx)


def test_model_conversion_keeps_parameters_and_is_all_or_nothing():
    """rtx/ptq.py semantics: training conversion keeps the Parameter objects (optimizer references, sharing,
    state-dict keys), shared modules are replaced at every alias, and nothing is touched when a selected
    layer is invalid."""
    import rtx_b200 as rtx
    from torch import nn

    class Block(nn.Module):
        def __init__(self):
            super().__init__()
            self.up = nn.Linear(32, 64, bias=False, dtype=torch.bfloat16)
            self.down = nn.Linear(64, 32, bias=False, dtype=torch.bfloat16)
            self.tied = self.up                      # an alias of a shared module
            self.head = nn.Linear(32, 8, bias=True, dtype=torch.bfloat16)

    model = Block()
    params = {n: p for n, p in model.named_parameters()}
    keys = list(model.state_dict())
    no_head = lambda m, fqn: isinstance(m, nn.Linear) and fqn != "head"
    out = rtx.convert_to_mxfp8_training(model, module_filter_fn=no_head)
    assert out is model and isinstance(model.up, rtx.MXFP8Linear) and model.tied is model.up
    assert isinstance(model.head, nn.Linear) and list(model.state_dict()) == keys
    assert all(params[n] is p for n, p in model.named_parameters())
    # the default filter reaches the biased head: refused before anything changes
    model2 = Block()
    with pytest.raises(NotImplementedError, match="bias"):
        rtx.convert_to_nvfp4_training(model2)
    assert type(model2.up) is nn.Linear
    with pytest.raises(ValueError, match="only some aliases"):
        rtx.convert_to_nvfp4_training(model2, module_filter_fn=lambda m, fqn: fqn == "up")
    nv = rtx.convert_to_nvfp4_training(model2, module_filter_fn=no_head,
                                       config=rtx.NVFP4TrainingConfig(scaling="delayed", scale_region_rows=None))
    assert isinstance(nv.down, rtx.NVFP4Linear) and nv.down.scaling == "delayed" and nv.down.weight is not None
    # PTQ needs CUDA weights and one of the two weight-only policies
    with pytest.raises(ValueError, match="CUDA"):
        rtx.quantize_(Block(), rtx.MXFP8WeightOnlyConfig(), filter_fn=no_head)
    with pytest.raises(TypeError, match="WeightOnlyConfig"):
        rtx.quantize_(Block(), object())
    with pytest.raises(ValueError, match="current or block"):
        rtx.NVFP4WeightOnlyConfig(scaling="delayed")
    # a root that is itself a linear is returned replaced
    root = nn.Linear(32, 32, bias=False, dtype=torch.bfloat16)
    assert isinstance(rtx.convert_to_mxfp8_training(root), rtx.MXFP8Linear)


def test_quantized_weight_cache_scope_and_invalidation():
    """Host logic of the step-scoped weight cache: entries follow the parameter's storage and autograd
    version, scopes nest onto the outermost cache, the scope is per thread and empties on exit."""
    import threading

    import rtx_b200 as rtx
    from rtx_b200 import weight_cache as W

    assert W.active() is None
    w = torch.nn.Parameter(torch.zeros(4, 4))
    other = torch.nn.Parameter(torch.zeros(4, 4))
    made = []

    def make(tag):
        return lambda: made.append(tag) or [tag]

    with rtx.quantized_weight_cache() as cache:
        assert W.active() is cache and cache.alive
        assert cache.get(w, "rows", make("a")) is cache.get(w, "rows", make("b"))
        assert cache.get(w, "transposed", make("c")) == ["c"]          # parts are independent
        assert cache.get(other, "rows", make("d")) == ["d"]            # so are parameters
        assert cache.get(w.detach(), "rows", make("e")) == ["a"]       # same storage and version: same entry
        with torch.no_grad():
            w.add_(1)                                                  # what an optimizer does
        assert cache.get(w, "rows", make("f")) == ["f"]
        assert cache.get(w, "transposed", make("g")) == ["g"]
        with rtx.quantized_weight_cache() as inner:
            assert inner is cache
        assert W.active() is cache
        seen = []
        t = threading.Thread(target=lambda: seen.append(W.active()))
        t.start()
        t.join()
        assert seen == [None]
        assert cache.stats == {"hits": 2, "misses": 5}
    assert made == ["a", "c", "d", "f", "g"]
    assert W.active() is None and not cache.alive and not cache.entries


def test_numa_local_is_a_no_op_without_a_gpu(monkeypatch):
    """`numa_local` narrows the thread's CPU affinity only when NVML names CPUs next to the GPU that the
    process may use; otherwise, and with RTXB_HOST_NUMA=0, the affinity is left alone.  It is restored on exit."""
    import os

    from rtx_b200 import host

    before = os.sched_getaffinity(0)
    with host.numa_local(torch.device("cuda", 0)) as scope:
        assert scope.cpus is None or set(scope.cpus) <= before
    assert os.sched_getaffinity(0) == before
    one = sorted(before)[:1]
    monkeypatch.setattr(host, "gpu_local_cpus", lambda device: one)
    with host.numa_local(torch.device("cuda", 0)) as scope:
        assert scope.cpus == one and os.sched_getaffinity(0) == set(one)
    assert os.sched_getaffinity(0) == before
    monkeypatch.setenv("RTXB_HOST_NUMA", "0")
    with host.numa_local(torch.device("cuda", 0)) as scope:
        assert scope.cpus is None and os.sched_getaffinity(0) == before


def test_stored_winner_changes_what_the_module_runs(tmp_path):
    """`autotune="cache"` on MXFP8Linear resolves the stored winner of the call's (M, N, K) (rtx/fp8.py:804-886,
    rtx/autotune/winners.py:26-45): explain() names the winner's GEMM schedule for that M and the configured one for
    an M without a winner; the quantizer settings of the module's own schedule are kept."""
    import rtx_b200 as rtx
    from rtx_b200 import autotune as A
    from rtx_b200 import configs as C

    n, k = 384, 256
    adapter = A.ADAPTERS["mxfp8_prequant_fwd"]()
    ctx = A.KernelContext("mxfp8_prequant_fwd", 512, n, k)
    winner = C.MXFP8PrequantConfig(gemm=C.MXFP8GemmConfig.for_schedule("single"))
    assert "fused_x" in C.MXFP8GemmConfig.SCHEDULES and any(
        c.gemm.schedule == "fused_x" for c in adapter.candidates(ctx))
    A.save_runtime_winner(ctx, adapter, winner, 0.123, tmp_path)
    floor = C.MXFP8PrequantConfig(quant=C.MXFP8QuantConfig(scale_rounding="floor"))
    tuned = rtx.MXFP8Linear(k, n, autotune="cache", autotune_cache_dir=tmp_path, dynamic_config=floor)
    plain = rtx.MXFP8Linear(k, n, dynamic_config=floor)
    hit, miss = tuned.explain(m=512), tuned.explain(m=256)
    assert hit["gemm_schedule"] == "single" and hit["schedule_source"] == "stored winner"
    assert miss["gemm_schedule"] == "auto" and miss["forward_key"] == plain.explain()["forward_key"]
    assert hit["forward_key"] != miss["forward_key"]
    assert C.config_from_key(hit["forward_key"]).quant.scale_rounding == "floor"
    assert plain.explain(m=512)["gemm_schedule"] == "auto" and plain.explain()["autotune"] == "off"


def test_install_as_rtx_aliases_the_package():
    """Code written against the reference's package name imports this package after `install_as_rtx()`."""
    import subprocess
    import sys

    code = ("import rtx_b200, torch; rtx_b200.install_as_rtx(); import rtx, rtx.fp8, rtx.formats; "
            "assert rtx.MXFP8Linear is rtx_b200.MXFP8Linear and rtx.fp8.mxfp8_linear is rtx_b200.mxfp8_linear; "
            "assert torch._rtx_mxfp8_launchers is torch._rtx_b200_launchers['mxfp8_fwd']; print('ok')")
    root = __import__("os").path.dirname(__import__("os").path.dirname(__import__("os").path.abspath(__file__)))
    out = subprocess.run([sys.executable, "-c", code], cwd=root, capture_output=True, text=True, timeout=300)
    assert out.returncode == 0 and out.stdout.strip().endswith("ok"), out.stderr[-2000:]


def test_stored_winner_reaches_nvfp4_modules(tmp_path):
    """`autotune="cache"` on NVFP4Linear: a winner stored for (family, M, N, K, policy) changes the schedule explain()
    reports for that M; other policies and other M keep the configured schedule (rtx/fp4.py:1065-1207)."""
    import rtx_b200 as rtx
    from rtx_b200 import autotune as A
    from rtx_b200 import configs as C

    n, k = 256, 128
    adapter = A.ADAPTERS["nvfp4_dynamic_fwd"]()
    ctx = A.KernelContext("nvfp4_dynamic_fwd", 64, n, k, variant="jit_row_region")
    winner = C.NVFP4DynamicConfig(gemm=C.NVFP4GemmConfig.for_schedule("stream"))
    A.save_runtime_winner(ctx, adapter, winner, 0.01, tmp_path)
    tuned = rtx.NVFP4Linear(k, n, autotune="cache", autotune_cache_dir=tmp_path)
    hit, miss = tuned.explain(m=64), tuned.explain(m=4096)
    assert hit["gemm_schedule"] == "stream" and hit["schedule_source"] == "stored winner"
    assert miss["gemm_schedule"] == "auto"
    kept = C.config_from_key(hit["forward_key"])
    assert kept.scale.policy == "jit_row_region" and kept.x_scale_region_rows == tuned.x_scale_region_rows
    other = rtx.NVFP4Linear(k, n, scaling="current", autotune="cache", autotune_cache_dir=tmp_path)
    assert other.explain(m=64)["gemm_schedule"] == "auto"          # a different policy is a different variant
    assert rtx.NVFP4Linear(k, n).explain()["autotune"] == "off"
    # the functional form resolves stored winners the same way (no first-use tuning there)
    from rtx_b200 import fp4

    base = tuned._dynamic_config
    got = fp4._stored_winner_config(base, 64, n, k, tmp_path, False, "jit_row_region")
    assert got.gemm.schedule == "stream" and got.scale.policy == "jit_row_region"
    assert fp4._stored_winner_config(base, 4096, n, k, tmp_path, False, "jit_row_region").gemm.schedule == "auto"
    assert fp4._stored_winner_config(base, 64, n, k, tmp_path, True, "current").gemm.schedule == "auto"


def test_row_block_of_a_global_draw_equals_the_slice():
    """workloads.make_inputs(rows=(lo, hi)): a rank of a weak-scaling run keeps only its block of the global
    tensors, with the values of the full draw (never seeded by rank); weights are unaffected."""
    from rtx_b200.workloads import make_inputs

    full = make_inputs(2, m=8192 + 4096, k=256, inter=128)
    part = make_inputs(2, m=8192 + 4096, k=256, inter=128, rows=(3000, 9000))
    assert torch.equal(full["x"][3000:9000], part["x"]) and torch.equal(full["w_gate_up"], part["w_gate_up"])
    assert torch.equal(full["w_down"], part["w_down"])
    full = make_inputs(4, m=12288, k=128, n=256)
    part = make_inputs(4, m=12288, k=128, n=256, rows=(4096, 12288))
    assert torch.equal(full["x"][4096:], part["x"]) and torch.equal(full["dy"][4096:], part["dy"])
    assert torch.equal(full["w"], part["w"])
