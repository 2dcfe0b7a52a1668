#!/usr/bin/env python
"""Benchmark of the block-scaled quantize+GEMM hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl own|reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

Headline workload: the MXFP8 SwiGLU MLP forward of benchmark configuration 2 — ONE batch
X bf16 [8192, 4096] (N(0,1), 0.1 % of entries x50), W_gate|W_up bf16 [28672, 4096], W_down bf16
[4096, 14336] — whose token rows are sharded over the ranks (strong scaling: 8192 / N rows per GPU),
weights replicated, no collective.  Every step quantizes X, both weights and H to MXFP8 and runs
the two block-scaled GEMMs (SiLU*up fused into the first epilogue).

The one JSON line rank 0 prints also carries, as named sub-records:
  weak       the same forward with 8192 rows PER GPU (per-GPU work fixed);
  sustained  the headline step looped for at least two seconds (clock and power under the cap);
  backward   configuration 4 (MXFP8 dX + dW, 16384 x 4096 x 4096) through
             rtx_b200.parallel.data_parallel_linear_backward, the FP32 dW all-reduced with NCCL
             inside the timed region, strong (16384 rows split) and weak (16384 rows per GPU),
             with a parity check of the sharded result against the unsharded one;
  configs    (1 GPU only) configurations 3 and 5 measured as bench_configs.py does.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

M, K, INTER, N_OUT = 8192, 4096, 14336, 4096
BWD_M, BWD_N, BWD_K = 16384, 4096, 4096
NOMINAL_FP8_TFLOPS = 4500.0
SUSTAINED_SECONDS = 2.2
METRIC = "fused quant+GEMM TFLOPS (MXFP8 SwiGLU MLP forward, quantization included)"


def mlp_flops(m: int) -> float:
    return 2.0 * m * (2 * INTER) * K + 2.0 * m * N_OUT * INTER


def measured_peaks() -> dict:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        d["source"] = "measured"
        return d
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clock, power and throttle reasons with `nvidia-smi -lms` (read-only) in a child process
    while the timed loops run; a sample counts for a label if its timestamp falls inside a region marked
    with that label."""

    FIELDS = ("timestamp,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int, period_ms: int = 10):
        self.index, self.period_ms = index, period_ms
        self.proc, self.path, self.regions = None, None, []

    def start(self):
        import subprocess
        import tempfile

        fd, self.path = tempfile.mkstemp(suffix=".csv")
        os.close(fd)
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", str(self.period_ms), "-f", self.path], stdout=subprocess.DEVNULL, stderr=subprocess.DEVNULL)
            time.sleep(0.3)   # let it print its first lines before the timed loops start
        except OSError:
            self.proc = None

    def mark(self, label: str, t0: float, t1: float):
        self.regions.append((label, t0, t1))

    def stop(self) -> dict:
        """{label: {sm_mhz, sm_max_mhz, power_w, reasons, samples}}"""
        import datetime

        labels = sorted({r[0] for r in self.regions})
        empty = {"sm_mhz": None, "sm_max_mhz": None, "power_w": None, "reasons": [], "samples": 0}
        if self.proc is None:
            return {label: dict(empty) for label in labels}
        time.sleep(0.05)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except Exception:
            self.proc.kill()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        try:
            lines = open(self.path).read().splitlines()
            os.unlink(self.path)
        except OSError:
            lines = []
        acc = {label: {"clocks": [], "powers": [], "reasons": set()} for label in labels}
        max_mhz, total = None, 0
        for line in lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 8:
                continue
            try:
                ts = datetime.datetime.strptime(parts[0], "%Y/%m/%d %H:%M:%S.%f").timestamp()
                mhz, mx, watts = float(parts[1]), float(parts[2]), float(parts[3])
            except ValueError:
                continue
            total += 1
            max_mhz = mx
            for label, t0, t1 in self.regions:
                if t0 - 0.005 <= ts <= t1 + 0.005:
                    a = acc[label]
                    a["clocks"].append(mhz)
                    a["powers"].append(watts)
                    a["reasons"].update(n for n, flag in zip(names, parts[4:8]) if flag.lower().startswith("active"))
        out = {}
        for label, a in acc.items():
            out[label] = {"sm_mhz": statistics.median(a["clocks"]) if a["clocks"] else None, "sm_max_mhz": max_mhz,
                          "power_w": statistics.median(a["powers"]) if a["powers"] else None,
                          "reasons": sorted(a["reasons"]), "samples": len(a["clocks"]), "samples_total": total}
        return out


def physical_gpu_index(local_rank: int) -> int:
    vis = os.environ.get("CUDA_VISIBLE_DEVICES")
    if vis:
        try:
            return int(vis.split(",")[local_rank])
        except (ValueError, IndexError):
            pass
    return local_rank


# --------------------------------------------------------------------------
# reference arm and CPU baseline: the reference's CPU path (oracle/cpu_path.py)
# --------------------------------------------------------------------------

def host_threads() -> int:
    """Host threads this process may use: the CPUs of its affinity mask (a container's share), not the machine's."""
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except (AttributeError, OSError):
        return os.cpu_count() or 1


def cpu_workload_run(m_rows: int, threads: int, repeats: int, warmup: int):
    """Times the reference's CPU formulation (encode + FP32 dequantized matmul) of the MLP forward on the
    first m_rows token rows of configuration 2 with the full weights.  -> (seconds per run, flop per run)"""
    import torch

    from oracle import cpu_path as C
    from rtx_b200.workloads import make_inputs

    torch.set_num_threads(threads)
    inp = make_inputs(2, m=m_rows, inter=INTER)
    x, wgu, wd = inp["x"], inp["w_gate_up"], inp["w_down"]
    times = []
    for i in range(warmup + repeats):
        t0 = time.perf_counter()
        C.mx_glu_mlp(x, wgu, wd)
        dt = time.perf_counter() - t0
        if i >= warmup:
            times.append(dt)
    return times, mlp_flops(m_rows)


def run_reference_arm(args) -> None:
    """The reference's own CPU path on the host cores, all threads, every step the WHOLE configuration-2
    batch (8192 rows, full weights): the same work per step as the own arm's global step at any N."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    threads = host_threads()
    times, flops = cpu_workload_run(M, threads, args.steps, max(min(args.warmup, 2), 1))
    total = sum(times)
    value = flops * len(times) / total / 1e12
    sample = (f"every step = the whole workload: X {M} rows, W_gate|W_up [{2 * INTER}, {K}], W_down [{N_OUT}, {INTER}], "
              f"{flops:.3e} flop; {len(times)} steps in {total:.1f} s")
    line = {
        "impl": "reference",
        "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": 1e3 * total / len(times), "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "mxfp8 (e4m3 x e8m0), fp32 accumulate", "data": "synthetic",
        "config": {"workload": f"mxfp8_glu_mlp_fwd_m{M}_k{K}_i{INTER}", "sample": sample,
                   "path": "reference CPU path: torch encode + FP32 dequantized matmul (oracle/cpu_path.py, pinned bit "
                           "for bit to the reference's rtx.autotune.legacy._torch_mxfp8_reference)"},
        "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# --------------------------------------------------------------------------
# own arm
# --------------------------------------------------------------------------

class Timer:
    """CUDA-event timing on the current stream between barriers; results are reduced (max over ranks)
    together at the end."""

    def __init__(self, torch, dist, world, local_rank, sampler):
        self.torch, self.dist, self.world, self.local_rank, self.sampler = torch, dist, world, local_rank, sampler
        self.results = {}

    def barrier(self):
        if self.world > 1:
            self.dist.barrier(device_ids=[self.local_rank])

    def run(self, name, fn, steps, warmup, label="burst", per_step=False):
        """per_step: an event after every step as well, so that the record can show median and worst step beside
        the mean (a single stall inside a 20-step region otherwise hides in the mean)."""
        torch = self.torch
        for _ in range(warmup):
            fn()
        torch.cuda.synchronize()
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        marks = [torch.cuda.Event(enable_timing=True) for _ in range(steps)] if per_step else None
        self.barrier()
        torch.cuda.synchronize()
        w0 = time.time()
        ev0.record()
        for i in range(steps):
            fn()
            if marks is not None:
                marks[i].record()
        ev1.record()
        torch.cuda.synchronize()
        self.sampler.mark(label, w0, time.time())
        self.barrier()
        self.results[name] = ev0.elapsed_time(ev1) / steps
        if marks is not None:
            each = sorted(a.elapsed_time(b) for a, b in zip([ev0] + marks[:-1], marks))
            self.results[name + "_median"] = each[len(each) // 2]
            self.results[name + "_max"] = each[-1]
        return self.results[name]

    def reduce(self, dev):
        names = sorted(self.results)
        t = self.torch.tensor([self.results[n] for n in names], dtype=self.torch.float64, device=dev)
        if self.world > 1:
            self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        self.results = dict(zip(names, (float(v) for v in t.tolist())))
        return self.results


def run_own_arm(args) -> None:
    import torch
    import torch.distributed as dist

    from rtx_b200 import _native as N
    from rtx_b200 import build, ops, parallel
    from rtx_b200.host import GluMlpHostSession, numa_local
    from rtx_b200.workloads import make_inputs

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device; there is no CPU fallback for the measured path")
    if not os.path.exists(N.LIB_PATH):
        build.build()
    N.load()
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev, pg_options=parallel.nccl_options())
    if M % (world * 128) or BWD_M % (world * 128):
        raise SystemExit(f"{M} and {BWD_M} token rows must split into whole 128-row tiles over {world} ranks")
    steps, warmup = args.steps, max(args.warmup, 3)
    sampler = ClockSampler(physical_gpu_index(local_rank), period_ms=args.sample_ms)
    timer = Timer(torch, dist, world, local_rank, sampler)
    ws = ops.Workspace(dev)

    # ---------------- forward inputs: one global draw, every rank slices its rows ----------------
    inp = make_inputs(2, m=M)             # the same batch and weights at every N
    numa = numa_local(dev)
    numa.__enter__()                       # host buffers next to this rank's GPU; restored before the CPU baseline
    per = M // world
    x_host = inp["x"][rank * per:(rank + 1) * per].contiguous().pin_memory()
    x = x_host.to(dev, non_blocking=True)
    # weak sub-record: M rows per GPU out of a global draw of M * world rows
    x_weak = make_inputs(2, m=M * world, rows=(rank * M, (rank + 1) * M))["x"].to(dev) if world > 1 else x
    wgu = inp["w_gate_up"].to(dev)
    wd = inp["w_down"].to(dev)
    del inp
    y = torch.empty(per, N_OUT, dtype=torch.bfloat16, device=dev)
    y_weak = torch.empty(M, N_OUT, dtype=torch.bfloat16, device=dev) if world > 1 else y
    y_host = torch.empty(per, N_OUT, dtype=torch.bfloat16).pin_memory()
    launches_per_step = 5  # quantize X, W_gate_up, W_down + gate/up GEMM (SiLU*up and H quantization fused) + down GEMM

    def step():
        with ops.gemm_schedule(args.schedule):
            ops.mxfp8_glu_mlp_fwd(x, wgu, wd, ws, None, y, want_hidden=False)

    def step_weak():
        with ops.gemm_schedule(args.schedule):
            ops.mxfp8_glu_mlp_fwd(x_weak, wgu, wd, ws, None, y_weak, want_hidden=False)

    sampler.start()
    timer.run("fwd", step, steps, warmup)
    ops.check_device_status(dev)
    if world > 1:
        timer.run("fwd_weak", step_weak, steps, warmup)
        ops.check_device_status(dev)

    # ---------------- dominant kernel alone: the gate/up GEMM with the fused SwiGLU epilogue ----------------
    qx, sx = ops.mxfp8_quantize(x)
    qg, sg = ops.mxfp8_quantize(wgu)
    if args.schedule == "fused_x":
        timer.run("gemm", lambda: ops.mxfp8_gemm_glu_mx_fused_x(x, qg, sg, INTER), steps, 3)
    else:
        with ops.gemm_schedule(args.schedule):
            timer.run("gemm", lambda: ops.mxfp8_gemm_glu_mx(qx, sx, qg, sg, per, INTER, K), steps, 3)
    ops.check_device_status(dev)
    del qx, sx, qg, sg
    if args.quick:
        clocks = sampler.stop()
        numa.__exit__(None, None, None)
        res = timer.reduce(dev)
        if rank == 0:
            print(json.dumps({
                "metric": METRIC, "value": mlp_flops(M) / (res["fwd"] * 1e-3) / 1e12, "unit": "TFLOP/s", "n_gpus": world,
                "steps": steps, "warmup": warmup, "ms_per_step": res["fwd"], "quick": True, "schedule": args.schedule,
                "config": {"workload": f"mxfp8_glu_mlp_fwd_m{M}_k{K}_i{INTER}", "m_per_gpu": per},
                "dominant_kernel": {"ms_per_launch": res["gemm"],
                                    "tflops": 2.0 * per * (2 * INTER) * K / (res["gemm"] * 1e-3) / 1e12},
                "clocks": clocks.get("burst")}), flush=True)
        if world > 1:
            dist.destroy_process_group()
        return

    # ---------------- end to end through host buffers (rtx_b200.host.GluMlpHostSession) ----------------
    # every step copies that step's X from pinned host memory to the device and its Y back; copy-in of step
    # i+1 and copy-out of step i-1 overlap the compute of step i (three streams, three device buffer sets)
    session = GluMlpHostSession(wgu, wd, per)
    x_hosts = [x_host, x_host.clone().pin_memory()]
    y_hosts = [y_host, torch.empty_like(y_host).pin_memory()]
    for i in range(3):
        session.submit(x_hosts[i % 2], y_hosts[i % 2])
    session.drain()
    timer.barrier()
    torch.cuda.synchronize()
    w0 = time.time()
    t0 = time.perf_counter()
    for i in range(steps):
        session.submit(x_hosts[i % 2], y_hosts[i % 2])
    session.drain()
    timer.results["e2e"] = (time.perf_counter() - t0) * 1e3 / steps   # spans three streams: host clock, submit..drain
    sampler.mark("burst", w0, time.time())
    timer.barrier()
    e2e_launches = session.launches_per_step
    del session

    # the copies of the end-to-end step alone (X in and Y out at the same time, no compute): its PCIe floor
    s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()
    c0, c1, c2, c3 = (torch.cuda.Event(enable_timing=True) for _ in range(4))
    torch.cuda.synchronize()
    with torch.cuda.stream(s_in):
        c0.record()
        for i in range(steps):
            x.copy_(x_hosts[i % 2], non_blocking=True)
        c1.record()
    with torch.cuda.stream(s_out):
        c2.record()
        for i in range(steps):
            y_hosts[i % 2].copy_(y, non_blocking=True)
        c3.record()
    torch.cuda.synchronize()
    timer.results["copies"] = max(c0.elapsed_time(c1), c2.elapsed_time(c3)) / steps
    numa.__exit__(None, None, None)

    del x_weak, y_weak

    # ---------------- backward (configuration 4): dX local, FP32 dW all-reduced inside the timed region ----------------
    bwd = make_inputs(4, m=BWD_M)          # the same 16384 rows and weight at every N
    bper = BWD_M // world
    w_b = bwd["w"].to(dev)
    shards = {"strong": (bwd["x"][rank * bper:(rank + 1) * bper].to(dev), bwd["dy"][rank * bper:(rank + 1) * bper].to(dev))}
    if world > 1:
        # weak: 16384 rows per GPU out of one global draw of 16384 * N rows (only this rank's block is held)
        wide = make_inputs(4, m=BWD_M * world, rows=(rank * BWD_M, (rank + 1) * BWD_M))
        shards["weak"] = (wide["x"].to(dev), wide["dy"].to(dev))
        del wide
    bwd_parity = None
    for mode, (xb, dyb) in shards.items():
        timer.run(f"bwd_{mode}", lambda: parallel.data_parallel_linear_backward(dyb, xb, w_b), steps, warmup,
                  per_step=True)
        ops.check_device_status(dev)
    if world > 1:
        # parity of the sharded step: dX rows bit-equal to the unsharded rows, all-reduced dW within the
        # output bar of the unsharded dW (only the FP32 summation order differs)
        from oracle.mx_oracle import parity_report

        xb, dyb = shards["strong"]
        dx_r, dw_r = parallel.data_parallel_linear_backward(dyb, xb, w_b)
        x_all, dy_all = bwd["x"].to(dev), bwd["dy"].to(dev)
        dx_1, dw_1 = ops.mxfp8_linear_bwd(dy_all, x_all, w_b, ws)
        torch.cuda.synchronize()
        rep = parity_report(dw_r.cpu(), dw_1.cpu())
        bwd_parity = {"dx_rows_bit_equal": bool(torch.equal(dx_r, dx_1[rank * bper:(rank + 1) * bper])),
                      "dw_rel_fro": rep["rel_fro"], "dw_frac_le_1ulp": rep["frac_le_1ulp"],
                      "against": "the unsharded rtxb_mxfp8_linear_bwd on the same 16384 rows (rank 0's comparison)"}
        del x_all, dy_all, dx_1, dw_1, dx_r, dw_r
    del bwd, shards
    bwd_route = parallel.backward_collective(BWD_N, BWD_K, dev)

    # ---------------- other configurations, one GPU only ----------------
    others = None
    if world == 1 and not args.no_other_configs:
        import bench_configs as BC

        sub = argparse.Namespace(steps=steps, warmup=3)
        keep = ("metric", "value", "unit", "ms_per_step", "config", "roofline", "gpu_launches_per_step")
        others = {"c3_nvfp4_forward": [{k: ln.get(k) for k in keep} for ln in BC.config3(sub, 0, 1, dev)],
                  "c5_nvfp4_decode": [{k: ln.get(k) for k in keep} for ln in BC.config5(sub, 0, 1, dev)]}

    # ---------------- sustained: the headline step for >= 2 s (last: everything above is measured from a cool start,
    # this loop leaves the part at its power-capped clock) ----------------
    t = torch.tensor([timer.results["fwd"]], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    sustained_steps = int(SUSTAINED_SECONDS * 1e3 / float(t.item())) + 1
    timer.run("sustained", step, sustained_steps, 0, label="sustained")
    ops.check_device_status(dev)

    clocks = sampler.stop()
    res = timer.reduce(dev)

    if rank == 0:
        peaks = measured_peaks()
        fp8_peak = 2.0 * peaks["bf16_tflops"]
        flops_global = mlp_flops(M)                       # strong scaling: the global batch is fixed
        value = flops_global / (res["fwd"] * 1e-3) / 1e12
        e2e_value = flops_global / (res["e2e"] * 1e-3) / 1e12
        gemm_tflops = 2.0 * per * (2 * INTER) * K / (res["gemm"] * 1e-3) / 1e12
        sus = clocks.get("sustained", {})
        sus_value = flops_global / (res["sustained"] * 1e-3) / 1e12
        traffic = None
        tpath = os.path.join(ROOT, "profiles", "roofline_traffic.json")
        if os.path.exists(tpath) and world == 1:
            with open(tpath) as f:
                traffic = json.load(f).get("gemm_glu_mxfp8_c2_dram_bytes_per_launch")
        bwd_flops = 4.0 * BWD_M * BWD_N * BWD_K
        backward = {
            "metric": "fused quant+GEMM TFLOPS (MXFP8 backward dX + dW, operand quantizations and the dW all-reduce included)",
            "workload": f"mxfp8_linear_bwd_m{BWD_M}_n{BWD_N}_k{BWD_K}",
            "api": "rtx_b200.parallel.data_parallel_linear_backward",
            "collective": bwd_route,
            "strong": {"rows_per_gpu": bper, "ms_per_step": res["bwd_strong"],
                       "ms_per_step_median": res["bwd_strong_median"], "ms_per_step_max": res["bwd_strong_max"],
                       "value": bwd_flops / (res["bwd_strong"] * 1e-3) / 1e12, "unit": "TFLOP/s"},
        }
        if world > 1:
            backward["weak"] = {"rows_per_gpu": BWD_M, "ms_per_step": res["bwd_weak"],
                                "ms_per_step_median": res["bwd_weak_median"], "ms_per_step_max": res["bwd_weak_max"],
                                "value": bwd_flops * world / (res["bwd_weak"] * 1e-3) / 1e12, "unit": "TFLOP/s"}
            backward["parity"] = bwd_parity
        line = {
            "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": steps,
            "warmup": warmup, "ms_per_step": res["fwd"], "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "mxfp8 (e4m3 x e8m0), fp32 accumulate",
            "data": "synthetic",
            "config": {"workload": f"mxfp8_glu_mlp_fwd_m{M}_k{K}_i{INTER}", "m_global": M, "m_per_gpu": per, "k": K,
                       "inter": INTER, "n_out": N_OUT,
                       "parallelism": f"dp{world} (one {M}-row batch, token rows sharded, weights replicated, no collective)",
                       "l2": "inputs exceed L2 (352 MB of bf16 weights + X re-read and re-quantized every step)",
                       "hidden": "H leaves the gate/up epilogue already MXFP8-encoded; no BF16 H is materialized"},
            "tflops_per_gpu": value / world,
            "pct_of_nominal_fp8_peak": 100.0 * value / world / NOMINAL_FP8_TFLOPS,
            "pct_of_measured_fp8_proxy": 100.0 * value / world / fp8_peak,
            "e2e": {"value": e2e_value, "unit": "TFLOP/s", "h2d_bytes_per_step": x_host.numel() * 2 * world,
                    "d2h_bytes_per_step": y_host.numel() * 2 * world, "ms_per_step": res["e2e"],
                    "api": "rtx_b200.host.GluMlpHostSession.submit/drain (copies overlapped with compute)",
                    "gpu_launches_per_step": e2e_launches,
                    "host_cpus": f"{len(numa.cpus)} CPUs next to the GPU" if numa.cpus else "unbound",
                    "copies_alone_ms_per_step": res["copies"],
                    "copies_alone_gbs_each_way": x_host.numel() * 2 / (res["copies"] * 1e-3) / 1e9,
                    "note": ("host path of this pool: the host side of a box delivers 50-87 GB/s each way in total "
                             "however many GPUs or processes share it (bench_configs.py --config 7), so the copies "
                             "alone bound this figure at N > 1" if world > 1 else
                             "bound by this rank's own PCIe copies (copies_alone_ms_per_step)")},
            "gpu_launches": launches_per_step * steps,
            "clocks": clocks.get("burst"),
            "schedule": args.schedule,
            "roofline": {"kernel": ("gemm_mxfp8_fused_a_pair_kernel<glu_mx>" if args.schedule == "fused_x" else
                                    "gemm_blockscaled_pair_kernel<mxfp8, glu_mx>") + " (gate/up GEMM + SiLU*up + MXFP8 encode of H)",
                         "bound": "tensor", "achieved": gemm_tflops, "peak": fp8_peak, "unit": "TFLOP/s",
                         "frac": gemm_tflops / fp8_peak, "frac_of_nominal": gemm_tflops / NOMINAL_FP8_TFLOPS,
                         "traffic": traffic, "ms_per_launch": res["gemm"], "rows": per,
                         "peak_note": f"2 x {peaks['source']} cuBLAS bf16 burst ({peaks['bf16_tflops']} TFLOP/s) as the "
                                      f"dense FP8 proxy (of measured); nominal dense FP8 is {NOMINAL_FP8_TFLOPS} TFLOP/s"},
            "sustained": {"value": sus_value, "unit": "TFLOP/s", "steps": sustained_steps, "ms_per_step": res["sustained"],
                          "seconds": res["sustained"] * sustained_steps * 1e-3, "sm_mhz": sus.get("sm_mhz"),
                          "power_w": sus.get("power_w"), "reasons": sus.get("reasons"), "samples": sus.get("samples"),
                          "ms_times_mhz": (res["sustained"] * sus["sm_mhz"]) if sus.get("sm_mhz") else None,
                          "burst_ms_times_mhz": (res["fwd"] * clocks["burst"]["sm_mhz"])
                          if clocks.get("burst", {}).get("sm_mhz") else None,
                          "pct_of_nominal_fp8_peak": 100.0 * sus_value / world / NOMINAL_FP8_TFLOPS},
            "backward": backward,
        }
        if world > 1:
            weak_value = mlp_flops(M) * world / (res["fwd_weak"] * 1e-3) / 1e12
            line["weak"] = {"value": weak_value, "unit": "TFLOP/s", "rows_per_gpu": M, "ms_per_step": res["fwd_weak"],
                            "tflops_per_gpu": weak_value / world}
        if others is not None:
            line["configs"] = others
        if world == 1 and not args.no_cpu_baseline:
            threads = host_threads()
            times, flops = cpu_workload_run(M, threads, 3, 1)
            line["cpu_baseline"] = {
                "value": flops * len(times) / sum(times) / 1e12, "unit": "TFLOP/s", "cores": threads, "kind": "port",
                "sample": f"{len(times)} runs (after 1 warm-up) of the reference CPU path on the whole workload: "
                          f"X {M} rows, full weights, {flops:.3e} flop per run, {sum(times):.1f} s in total"}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", choices=["own", "reference"], default="own")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--sample-ms", type=int, default=10, help="period of the clock / power sampler (nvidia-smi -lms)")
    ap.add_argument("--no-other-configs", action="store_true", help="skip configurations 3 and 5 (1-GPU runs)")
    ap.add_argument("--schedule", choices=["auto", "single", "pair", "fused_x"], default="auto",
                    help="GEMM schedule of the forward step (fused_x: X is quantized inside the gate/up GEMM)")
    ap.add_argument("--quick", action="store_true",
                    help="forward step and dominant kernel only (profiler-sized runs): no end-to-end, sustained or backward part")
    ap.add_argument("--m", type=int, default=M, help="token rows of the batch (smaller values give profiler-sized cases)")
    ap.add_argument("--inter", type=int, default=INTER, help="SwiGLU intermediate width")
    args = ap.parse_args()
    globals()["M"], globals()["INTER"] = args.m, args.inter
    if args.impl == "reference":
        run_reference_arm(args)
    else:
        run_own_arm(args)


if __name__ == "__main__":
    main()
