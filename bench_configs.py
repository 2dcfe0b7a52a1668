"""Device-timed measurements of benchmark configurations 3, 4 and 5 (configuration 2 is `bench.py`).

    python bench_configs.py --config 3            # NVFP4 forward 16384 x 28672 x 8192
    python bench_configs.py --config 4            # MXFP8 backward dX + dW, 16384 x 4096 x 4096
    python bench_configs.py --config 5            # NVFP4 decode, packed weights, M in {1, 8, 16, 64}
    python bench_configs.py --config 6            # configuration 2's shapes with the step-scoped weight cache
    python bench_configs.py --config 7            # host <-> device copies of the end-to-end step alone, one process, all GPUs
    python -m torch.distributed.run --nproc-per-node N ... bench_configs.py --config 4
    python -m torch.distributed.run --nproc-per-node N ... bench_configs.py --config 8   # phases of that backward step

One JSON line per measured case (rank 0).  Token rows are sharded over ranks (weak scaling: the
configuration's M per GPU); configuration 4 reduces dW across ranks inside the timed region (through peer
memory by default, `--dw-route nccl` for the all-reduce).  Timing: CUDA events around K steps after W warm-ups, max over ranks; inputs exceed L2 for
configurations 3 and 4; configuration 5 rotates over enough weight copies to exceed L2.
"""

from __future__ import annotations

import argparse
import json
import os

import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

from rtx_b200 import _native as N  # noqa: E402
from rtx_b200 import ops, parallel  # noqa: E402
from rtx_b200.workloads import CONFIG_NAMES, make_inputs  # noqa: E402

NOMINAL = {"fp8": 4500.0, "fp4": 9000.0, "hbm": 8000.0}


def _peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        d["source"] = "measured"
        return d
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


def _time(fn, steps, warmup, world, dev):
    for _ in range(max(warmup, 3)):
        fn()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier(device_ids=[dev.index])
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) / steps], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ops.check_device_status(dev)
    return float(t.item())


def _time_graph(fn, steps, dev):
    """Capture `steps` calls of fn in one CUDA graph and time its replay: removes the host launch cost,
    which exceeds the kernel time on the microsecond-scale decode shapes."""
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(3):
            fn()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for _ in range(steps):
            fn()
    graph.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(5):
        graph.replay()
    e1.record()
    torch.cuda.synchronize()
    ops.check_device_status(dev)
    return e0.elapsed_time(e1) / (5 * steps)


def config3(args, rank, world, dev):
    m, n, k = 16384, 28672, 8192
    inp = make_inputs(3, m=m)            # every rank: the same tensors; weak scaling keeps M per GPU
    x, w = inp["x"].to(dev), inp["w"].to(dev)
    ws = ops.Workspace(dev)
    out = torch.empty(m, n, dtype=torch.bfloat16, device=dev)
    ms = _time(lambda: ops.nvfp4_linear_fwd(x, w, ws, out), args.steps, args.warmup, world, dev)
    sx = ops.nvfp4_tensor_scale(x)
    sw, so = ops.nvfp4_tensor_scale(w, other_scale=sx)
    qa, sa = ops.nvfp4_quantize(x, sx)
    qb, sb = ops.nvfp4_quantize(w, sw)
    gemm_ms = _time(lambda: ops.nvfp4_gemm(qa, sa, qb, sb, m, n, k, so, out=out), args.steps, args.warmup, world, dev)
    flops = 2.0 * m * n * k
    peak = 4.0 * _peaks()["bf16_tflops"]
    # the same forward under the row-region policy (the module default): X regions of 8 rows, W of 4
    # (the default X = 5 does not divide 16384 rows and would fall back to one region)
    region_ms = _time(lambda: ops.nvfp4_linear_fwd_regions(x, w, ws, 8, 4, out), args.steps, args.warmup, world, dev)
    xs, wsc = ops.nvfp4_region_scales(x, 8), ops.nvfp4_region_scales(w, 4)
    qa2, sa2 = ops.nvfp4_quantize_regions(x, xs, 8)
    qb2, sb2 = ops.nvfp4_quantize_regions(w, wsc, 4)
    region_gemm_ms = _time(lambda: ops.nvfp4_gemm_regions(qa2, sa2, qb2, sb2, m, n, k, xs, 8, wsc, 4, out=out),
                           args.steps, args.warmup, world, dev)
    region_line = {
        "metric": "fused quant+GEMM TFLOPS (NVFP4 linear forward, row-region outer scales + quantization included)",
        "value": flops * world / (region_ms * 1e-3) / 1e12, "unit": "TFLOP/s", "n_gpus": world,
        "ms_per_step": region_ms, "scaling": "weak", "dtype": "nvfp4 (e2m1 x e4m3 x f32 per row region), fp32 accumulate",
        "data": "synthetic",
        "config": {"workload": "nvfp4_linear_fwd_m16384_n28672_k8192", "m_per_gpu": m,
                   "scaling_policy": "jit_row_region/power2, X regions of 8 rows, W regions of 4 rows"},
        "pct_of_nominal_fp4_peak": 100.0 * flops / (region_ms * 1e-3) / 1e12 / NOMINAL["fp4"],
        "gpu_launches_per_step": 5,
        "roofline": {"kernel": "gemm_blockscaled_pair_kernel<nvfp4, region_bf16>", "bound": "tensor",
                     "achieved": flops / (region_gemm_ms * 1e-3) / 1e12, "peak": peak, "unit": "TFLOP/s",
                     "frac": flops / (region_gemm_ms * 1e-3) / 1e12 / peak, "ms_per_launch": region_gemm_ms,
                     "traffic": None},
    }
    # delayed policy: the outer scales come from the |max| history, no reduction before the quantizers
    hx = x.float().abs().amax().reshape(1).expand(16).clone()
    hw = w.float().abs().amax().reshape(1).expand(16).clone()
    hist = {"x": [hx, torch.empty_like(hx)], "w": [hw, torch.empty_like(hw)]}

    def delayed_step():
        ops.nvfp4_linear_fwd_delayed(x, w, ws, hist["x"][0], hist["w"][0], hist["x"][1], hist["w"][1], out=out)
        hist["x"].reverse()
        hist["w"].reverse()

    delayed_ms = _time(delayed_step, args.steps, args.warmup, world, dev)
    delayed_line = {
        "metric": "fused quant+GEMM TFLOPS (NVFP4 linear forward, delayed outer scales, quantization + |max| "
                  "observation included)",
        "value": flops * world / (delayed_ms * 1e-3) / 1e12, "unit": "TFLOP/s", "n_gpus": world,
        "ms_per_step": delayed_ms, "scaling": "weak", "dtype": "nvfp4 (e2m1 x e4m3 x f32), fp32 accumulate",
        "data": "synthetic",
        "config": {"workload": "nvfp4_linear_fwd_m16384_n28672_k8192", "m_per_gpu": m,
                   "scaling_policy": "delayed/power2, history 16, window max"},
        "pct_of_nominal_fp4_peak": 100.0 * flops / (delayed_ms * 1e-3) / 1e12 / NOMINAL["fp4"],
        "gpu_launches_per_step": 3,
        "roofline": {"kernel": "gemm_blockscaled_pair_kernel<nvfp4, bf16>", "bound": "tensor",
                     "achieved": flops / (gemm_ms * 1e-3) / 1e12, "peak": peak, "unit": "TFLOP/s",
                     "frac": flops / (gemm_ms * 1e-3) / 1e12 / peak, "ms_per_launch": gemm_ms, "traffic": None},
    }
    return [region_line, delayed_line, {
        "metric": "fused quant+GEMM TFLOPS (NVFP4 linear forward, outer scales + quantization included)",
        "value": flops * world / (ms * 1e-3) / 1e12, "unit": "TFLOP/s", "n_gpus": world, "ms_per_step": ms,
        "scaling": "weak", "dtype": "nvfp4 (e2m1 x e4m3 x f32), fp32 accumulate", "data": "synthetic",
        "config": {"workload": "nvfp4_linear_fwd_m16384_n28672_k8192", "m_per_gpu": m, "scaling_policy": "current/power2"},
        "pct_of_nominal_fp4_peak": 100.0 * flops / (ms * 1e-3) / 1e12 / NOMINAL["fp4"], "gpu_launches_per_step": 7,
        "roofline": {"kernel": "gemm_blockscaled_pair_kernel<nvfp4, bf16>", "bound": "tensor",
                     "achieved": flops / (gemm_ms * 1e-3) / 1e12, "peak": peak, "unit": "TFLOP/s",
                     "frac": flops / (gemm_ms * 1e-3) / 1e12 / peak, "ms_per_launch": gemm_ms, "traffic": None,
                     "peak_note": "4 x measured cuBLAS bf16 burst as the dense FP4 proxy; nominal dense FP4 is 9000"},
    }]


def config4(args, rank, world, dev):
    m, n, k = 16384, 4096, 4096
    inp = make_inputs(4, m=m)
    x, w, dy = inp["x"].to(dev), inp["w"].to(dev), inp["dy"].to(dev)
    ws = ops.Workspace(dev)

    def step():
        # one rank: one call for both products (dY read once for its two quantizations, dW rounded to BF16 in
        # the epilogue); more: FP32 dW all-reduced band by band beside the rest of the step
        return parallel.data_parallel_linear_backward(dy, x, w)

    ms = _time(step, args.steps, args.warmup, world, dev)
    qc, sc = ops.mxfp8_quantize_transposed(dy)
    qd, sd = ops.mxfp8_quantize_transposed(x)
    dwbuf = torch.empty(n, k, dtype=torch.float32, device=dev)
    gemm_ms = _time(lambda: ops.mxfp8_gemm(qc, sc, qd, sd, n, k, m, out=dwbuf), args.steps, args.warmup, world, dev)
    flops = 4.0 * m * n * k
    peak = 2.0 * _peaks()["bf16_tflops"]
    return [{
        "metric": "fused quant+GEMM TFLOPS (MXFP8 backward dX + dW, four operand quantizations included)",
        "value": flops * world / (ms * 1e-3) / 1e12, "unit": "TFLOP/s", "n_gpus": world, "ms_per_step": ms,
        "scaling": "weak", "dtype": "mxfp8 (e4m3 x e8m0), fp32 accumulate", "data": "synthetic",
        "config": {"workload": "mxfp8_linear_bwd_m16384_n4096_k4096", "m_per_gpu": m,
                   "collective": parallel.backward_collective(n, k, dev)},
        "pct_of_nominal_fp8_peak": 100.0 * flops / (ms * 1e-3) / 1e12 / NOMINAL["fp8"],
        "gpu_launches_per_step": 5 if world == 1 else 7,
        "roofline": {"kernel": "gemm_blockscaled_pair_kernel<mxfp8, f32> (dW, K = 16384)", "bound": "tensor",
                     "achieved": flops / 2 / (gemm_ms * 1e-3) / 1e12, "peak": peak, "unit": "TFLOP/s",
                     "frac": flops / 2 / (gemm_ms * 1e-3) / 1e12 / peak, "ms_per_launch": gemm_ms, "traffic": None},
    }]


def config5(args, rank, world, dev):
    lines = []
    k = 8192
    hbm = _peaks()["hbm_gbs"]
    ws = ops.Workspace(dev)
    for n in (8192, 28672):
        inp = make_inputs(5, m=64, n=n)
        w = inp["w"].to(dev)
        w_scale = ops.nvfp4_tensor_scale(w, N.TENSOR_SCALE_EXACT)
        qw, sw = ops.nvfp4_quantize(w, w_scale)
        # rotate over copies of the packed weight so that every launch streams it from HBM
        copies = max(2, int(2 * 126e6 // (qw.numel() + sw.numel())) + 1)
        qws = [qw.clone() for _ in range(copies)]
        sws = [sw.clone() for _ in range(copies)]
        del w
        for m in (1, 8, 16, 64):
            x = inp["x"][:m].contiguous().to(dev)
            out = torch.empty(m, n, dtype=torch.bfloat16, device=dev)
            state = {"i": 0}

            def step():
                i = state["i"] = (state["i"] + 1) % copies
                ops.nvfp4_linear_fwd_prequant_w(x, qws[i], sws[i], w_scale, n, ws, out=out,
                                                scale_mode=N.TENSOR_SCALE_EXACT)

            eager_ms = _time(step, args.steps, args.warmup, world, dev)
            ms = _time_graph(step, args.steps, dev)
            x_scale, o_scale = ops.nvfp4_tensor_scale(x, N.TENSOR_SCALE_EXACT, other_scale=w_scale)
            qx, sx = ops.nvfp4_quantize(x, x_scale)

            def gemm_only():
                i = state["i"] = (state["i"] + 1) % copies
                ops.nvfp4_gemm(qx, sx, qws[i], sws[i], m, n, k, o_scale, out=out)

            gemm_ms = _time_graph(gemm_only, args.steps, dev)
            algo_bytes = n * k / 2 + n * k / 16 + m * k * 2 + m * n * 2
            lines.append({
                "metric": "NVFP4 decode GB/s (packed weights streamed once, activations quantized on the fly)",
                "value": algo_bytes / (ms * 1e-3) / 1e9, "unit": "GB/s", "n_gpus": world, "ms_per_step": ms,
                "dtype": "nvfp4", "data": "synthetic",
                "config": {"workload": f"nvfp4_decode_m{m}_n{n}_k{k}", "weight_copies_rotated": copies,
                           "timing": "CUDA-graph replay of the step: one kernel that also quantizes the activations "
                                     "(M <= 4, few column tiles), else |max| partials, scale + quantize, GEMM as "
                                     "three launches, each a programmatic dependent of the one before",
                           "eager_ms_per_step": eager_ms},
                "pct_of_nominal_hbm": 100.0 * algo_bytes / (ms * 1e-3) / 1e9 / NOMINAL["hbm"],
                "gpu_launches_per_step": 1 if (m <= 4 and (n + 255) // 256 < 74) else 3,
                "roofline": {"kernel": ("gemm_skinny_kernel" if (n + 255) // 256 < 74 else "gemm_blockscaled_kernel")
                             + "<nvfp4, bf16>", "bound": "hbm",
                             "achieved": algo_bytes / (gemm_ms * 1e-3) / 1e9, "peak": hbm, "unit": "GB/s",
                             "frac": algo_bytes / (gemm_ms * 1e-3) / 1e9 / hbm, "ms_per_launch": gemm_ms, "traffic": None,
                             "algorithmic_bytes": algo_bytes},
            })
    return lines


def config6(args, rank, world, dev):
    """Step-scoped quantized-weight cache on the shapes of configuration 2: (a) the SwiGLU block's fused
    inference forward, (b) a training step of the gate/up projection with four micro-batches (forward,
    dX, dW each).  Every case is timed without and inside `quantized_weight_cache()`; the outputs of the
    two are bit-identical.  The cached numbers skip work the uncached path does, so they are reported
    beside configuration 2's metric, never as it."""
    import rtx_b200 as rtx

    m, k, inter = 8192, 4096, 14336
    inp = make_inputs(2)
    x = inp["x"].to(dev)
    blk = rtx.SwiGLU(k, inter, device=dev)
    with torch.no_grad():
        blk.gate_up_proj.weight.copy_(inp["w_gate_up"].to(dev))
        blk.down_proj.weight.copy_(inp["w_down"].to(dev))
    lin = blk.gate_up_proj
    micro = 4
    xg = x.clone().requires_grad_(True)
    dy = (torch.randn(m, 2 * inter, device=dev) * 0.1).bfloat16()

    def infer():
        with torch.no_grad():
            return blk(x)

    def train_step():
        lin.weight.grad = None
        xg.grad = None
        for _ in range(micro):
            lin(xg).backward(dy)

    def scoped(fn):
        def run():
            with rtx.quantized_weight_cache():
                fn()
        return run

    lines = []
    with torch.no_grad():
        want = infer().clone()
    with rtx.quantized_weight_cache() as cache:
        same = torch.equal(infer(), want)
        t_inf_cached = _time(infer, args.steps, args.warmup, world, dev)      # warm cache: weights unchanged
    t_inf = _time(infer, args.steps, args.warmup, world, dev)
    flops_inf = 2.0 * m * (2 * inter) * k + 2.0 * m * k * inter
    lines.append({
        "metric": "fused quant+GEMM TFLOPS (MXFP8 SwiGLU block forward; weights quantized once per scope)",
        "value": flops_inf * world / (t_inf_cached * 1e-3) / 1e12, "unit": "TFLOP/s", "n_gpus": world,
        "ms_per_step": t_inf_cached, "scaling": "weak", "dtype": "mxfp8 (e4m3 x e8m0), fp32 accumulate",
        "data": "synthetic",
        "config": {"workload": "mxfp8_glu_mlp_fwd_m8192_k4096_i14336", "weights": "cached in scope (3 launches)",
                   "uncached_ms_per_step": t_inf, "uncached_tflops": flops_inf / (t_inf * 1e-3) / 1e12,
                   "bit_identical_to_uncached": bool(same)},
        "gpu_launches_per_step": 3})
    t_train = _time(train_step, max(args.steps // 4, 3), args.warmup, world, dev)
    t_train_cached = _time(scoped(train_step), max(args.steps // 4, 3), args.warmup, world, dev)
    flops_train = micro * 3 * 2.0 * m * (2 * inter) * k
    lines.append({
        "metric": "fused quant+GEMM TFLOPS (MXFP8 gate/up projection, forward + dX + dW, 4 micro-batches per step)",
        "value": flops_train * world / (t_train_cached * 1e-3) / 1e12, "unit": "TFLOP/s", "n_gpus": world,
        "ms_per_step": t_train_cached, "scaling": "weak", "dtype": "mxfp8 (e4m3 x e8m0), fp32 accumulate",
        "data": "synthetic",
        "config": {"workload": "mxfp8_linear_train_m8192_n28672_k4096_x4_microbatches",
                   "weights": "quantized once per step (row-wise and transposed), scope closed before the update",
                   "uncached_ms_per_step": t_train, "uncached_tflops": flops_train / (t_train * 1e-3) / 1e12}})
    return lines


def config7(args, rank, world, dev):
    """Host path alone: ONE process drives every visible GPU with the end-to-end step's copies (67 MB of pinned X in,
    67 MB of Y out per GPU and step, both directions at once, one stream pair per GPU) and no compute.  Separates
    "several processes contend for the host" from "the host's PCIe / memory path is the limit" when the
    end-to-end figure of bench.py does not scale with the GPU count."""
    import time

    n = torch.cuda.device_count()
    nbytes = 8192 * 4096 * 2
    lines = []
    for active in sorted({1, 2, 4, n} & set(range(1, n + 1))):
        devs = [torch.device("cuda", i) for i in range(active)]
        hx = [torch.empty(nbytes, dtype=torch.uint8).pin_memory() for _ in devs]
        hy = [torch.empty(nbytes, dtype=torch.uint8).pin_memory() for _ in devs]
        dx = [torch.empty(nbytes, dtype=torch.uint8, device=d) for d in devs]
        dy = [torch.empty(nbytes, dtype=torch.uint8, device=d) for d in devs]
        s_in = [torch.cuda.Stream(d) for d in devs]
        s_out = [torch.cuda.Stream(d) for d in devs]

        def run(steps):
            for i, d in enumerate(devs):
                with torch.cuda.stream(s_in[i]):
                    for _ in range(steps):
                        dx[i].copy_(hx[i], non_blocking=True)
                with torch.cuda.stream(s_out[i]):
                    for _ in range(steps):
                        hy[i].copy_(dy[i], non_blocking=True)
            for d in devs:
                torch.cuda.synchronize(d)

        run(3)
        t0 = time.perf_counter()
        run(args.steps)
        dt = time.perf_counter() - t0
        lines.append({
            "metric": "host <-> device copy GB/s per GPU and direction (pinned, both directions at once, no compute)",
            "value": nbytes * args.steps / dt / 1e9, "unit": "GB/s", "n_gpus": active, "ms_per_step": 1e3 * dt / args.steps,
            "config": {"workload": "host_copies_67MB_in_67MB_out_per_gpu", "processes": 1, "gpus_driven": active,
                       "aggregate_gbs_each_way": active * nbytes * args.steps / dt / 1e9}})
    return lines


def config8(args, rank, world, dev):
    """Where a data-parallel backward step (configuration 4, 16384 rows per GPU, peer-memory route) spends its
    time: one event per phase on the stream the phase runs on, averaged over the steps, as milliseconds since
    the step's start (slowest rank); and the dW GEMM alone with local outputs against outputs in the owners'
    (peer) slots."""
    if world < 2:
        raise SystemExit("--config 8 needs two or more ranks (torchrun)")
    m, n, k = 16384, 4096, 4096
    inp = make_inputs(4, m=m)
    x, w, dy = inp["x"].to(dev), inp["w"].to(dev), inp["dy"].to(dev)
    st = parallel._peer_state(n, k, dev, None)
    if st is None:
        raise SystemExit("the peer-memory route is not available for this shape / group")
    for _ in range(max(args.warmup, 3)):
        parallel._peer_backward(dy, x, w, st)
    torch.cuda.synchronize()
    acc = {}
    for _ in range(args.steps):
        dist.barrier()
        torch.cuda.synchronize()
        marks = {}
        parallel._peer_backward(dy, x, w, st, marks=marks)
        torch.cuda.synchronize()
        for name, ev in marks.items():
            if name != "start":
                acc[name] = acc.get(name, 0.0) + marks["start"].elapsed_time(ev) / args.steps
    names = list(acc)
    t = torch.tensor([acc[nm] for nm in names], dtype=torch.float64, device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    phases = {nm: round(float(v), 4) for nm, v in zip(names, t.tolist())}
    q_dy, s_dy, q_dyt, s_dyt = ops.mxfp8_quantize_dual(dy)
    q_xt, s_xt = ops.mxfp8_quantize_transposed(x)
    local = [torch.empty(st.rows, k, dtype=torch.float32, device=dev) for _ in range(world)]
    first = (rank + 1) % world
    t_local = _time(lambda: ops.mxfp8_gemm_row_blocks(q_dyt, s_dyt, q_xt, s_xt, n, k, m, local, first_block=first),
                    args.steps, args.warmup, world, dev)
    t_peer = _time(lambda: ops.mxfp8_gemm_row_blocks(q_dyt, s_dyt, q_xt, s_xt, n, k, m, st.peer_slot, first_block=first),
                   args.steps, args.warmup, world, dev)
    return [{"metric": "data-parallel MXFP8 backward: milliseconds from the step's start to the end of each phase "
                       "(slowest rank; a synchronised start per step, so the first kernel carries its launch latency)",
             "value": phases["end"], "unit": "ms", "n_gpus": world, "ms_per_step": phases["end"],
             "config": {"workload": CONFIG_NAMES[4], "rows_per_gpu": m, "phases_ms_since_start": phases,
                        "main_stream": ["quantized_dy_and_xt", "dw_gemm", "quantized_wt", "dx_gemm", "end"],
                        "side_streams": ["barrier_partials_landed", "owner_sum", "barrier_blocks_reduced", "blocks_copied"],
                        "dw_gemm_alone_ms": {"local_outputs": round(t_local, 4), "outputs_in_peer_slots": round(t_peer, 4)}}}]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--config", type=int, required=True, choices=(3, 4, 5, 6, 7, 8))
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--dw-route", choices=["peer", "nccl"], default="peer",
                    help="configuration 4 on several GPUs: reduce-scatter through peer memory in the dW GEMM, or NCCL all-reduce")
    args = ap.parse_args()
    parallel.P2P_REDUCE_SCATTER = args.dw_route == "peer"
    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("a CUDA device is required; there is no CPU fallback for the measured path")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev, pg_options=parallel.nccl_options())
    lines = {3: config3, 4: config4, 5: config5, 6: config6, 7: config7, 8: config8}[args.config](args, rank, world, dev)
    if rank == 0:
        for line in lines:
            line.update({"steps": args.steps, "warmup": max(args.warmup, 3), "higher_is_better": True})
            print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
