#!/usr/bin/env python
"""Benchmark of the block-scaled quantize+GEMM hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl own|reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

Workload (N=1 and per rank): the MXFP8 SwiGLU MLP forward of the benchmark
configuration — X bf16 [8192, 4096] (N(0,1), 0.1 % of entries x50), W_gate|W_up
bf16 [28672, 4096], W_down bf16 [4096, 14336]; every step quantizes X, both
weights and H to MXFP8 and runs the two block-scaled GEMMs (SiLU*up fused into
the first epilogue).  Token rows are sharded over ranks, weights replicated, no
collective on the forward path.  One JSON line is printed by rank 0.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

M, K, INTER, N_OUT = 8192, 4096, 14336, 4096
NOMINAL_FP8_TFLOPS = 4500.0
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
    while the timed loops run; samples are kept only if their timestamp falls inside a marked region."""

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

    def mark(self, t0: float, t1: float):
        self.regions.append((t0, t1))

    def stop(self) -> dict:
        import datetime

        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        time.sleep(0.05)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except Exception:
            self.proc.kill()
        clocks, powers, reasons, max_mhz, total = [], [], set(), None, 0
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        try:
            lines = open(self.path).read().splitlines()
            os.unlink(self.path)
        except OSError:
            lines = []
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
            if not any(t0 - 0.005 <= ts <= t1 + 0.005 for t0, t1 in self.regions):
                continue
            clocks.append(mhz)
            powers.append(watts)
            for name, flag in zip(names, parts[4:8]):
                if flag.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(clocks) if clocks else None, "sm_max_mhz": max_mhz,
                "power_w": statistics.median(powers) if powers else None, "reasons": sorted(reasons),
                "samples": len(clocks), "samples_total": total,
                "regions": "timed steps, end-to-end steps and the dominant-kernel loop"}


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

def cpu_sample_run(m_s: int, inter_s: int, threads: int, repeats: int, warmup: int):
    """Times the CPU path on a sample: the first m_s token rows, gate/up rows [0, inter_s) of each
    half and the matching inter_s columns of W_down.  Returns (seconds per run list, flops per run)."""
    import torch

    from oracle import cpu_path as C
    from rtx_b200.workloads import make_inputs

    torch.set_num_threads(threads)
    inp = make_inputs(2, m=m_s, inter=inter_s)
    x, wgu, wd = inp["x"], inp["w_gate_up"], inp["w_down"]
    flops = 2.0 * m_s * (2 * inter_s) * K + 2.0 * m_s * N_OUT * inter_s
    times = []
    for i in range(warmup + repeats):
        t0 = time.perf_counter()
        C.mx_glu_mlp(x, wgu, wd)
        dt = time.perf_counter() - t0
        if i >= warmup:
            times.append(dt)
    return times, flops


def run_reference_arm(args) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    m_s, inter_s = 2048, 2048
    times, flops = cpu_sample_run(m_s, inter_s, threads, args.steps, max(args.warmup, 1))
    total = sum(times)
    value = flops * len(times) / total / 1e12
    sample = (f"per step: X[:{m_s}] of {M} rows, gate/up rows [0,{inter_s}) of {INTER} each, "
              f"W_down[:, :{inter_s}]; K={K} and n_out={N_OUT} full; {flops:.3e} flop/step")
    line = {
        "impl": "reference",
        "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": 1e3 * total / len(times), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "mxfp8 (e4m3 x e8m0), fp32 accumulate", "data": "synthetic",
        "config": {"workload": "mxfp8_glu_mlp_fwd_m8192_k4096_i14336", "sample": sample,
                   "path": "reference CPU path: torch encode + FP32 dequantized matmul (oracle/cpu_path.py port)"},
        "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# --------------------------------------------------------------------------
# own arm
# --------------------------------------------------------------------------

def run_own_arm(args) -> None:
    import torch
    import torch.distributed as dist

    from rtx_b200 import _native as N
    from rtx_b200 import build, ops
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
        dist.init_process_group("nccl", device_id=dev)

    def barrier():
        if world > 1:
            dist.barrier(device_ids=[local_rank])

    # identical global tensors on every rank; each rank keeps its own M rows (weak scaling:
    # M rows per GPU whatever the GPU count)
    rows_global = M * world if args.scaling == "weak" else M
    inp = make_inputs(2, m=rows_global)
    per = rows_global // world
    # host buffers on the NUMA node of this rank's GPU (affinity restored before the CPU baseline runs)
    from rtx_b200.host import numa_local
    numa = numa_local(dev)
    numa.__enter__()
    x_host = inp["x"][rank * per:(rank + 1) * per].contiguous().pin_memory()
    x = x_host.to(dev, non_blocking=True)
    wgu = inp["w_gate_up"].to(dev)
    wd = inp["w_down"].to(dev)
    del inp
    m_local = per
    y = torch.empty(m_local, N_OUT, dtype=torch.bfloat16, device=dev)
    y_host = torch.empty(m_local, N_OUT, dtype=torch.bfloat16).pin_memory()
    ws = ops.Workspace(dev)
    launches_per_step = 5  # quantize X, W_gate_up, W_down + gate/up GEMM (SiLU*up and H quantization fused) + down GEMM

    def step():
        ops.mxfp8_glu_mlp_fwd(x, wgu, wd, ws, None, y, want_hidden=False)

    for _ in range(max(args.warmup, 3)):
        step()
    torch.cuda.synchronize()
    ops.check_device_status(dev)

    sampler = ClockSampler(physical_gpu_index(local_rank))
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    torch.cuda.synchronize()
    sampler.start()
    torch.cuda.synchronize()
    w0 = time.time()
    ev0.record()
    for _ in range(args.steps):
        step()
    ev1.record()
    torch.cuda.synchronize()
    sampler.mark(w0, time.time())
    barrier()
    ms_total = ev0.elapsed_time(ev1)
    ops.check_device_status(dev)

    # end to end through host buffers (rtx_b200.host.GluMlpHostSession): every step copies that step's X
    # from pinned host memory to the device and its Y back to pinned host memory; copy-in of step i+1 and
    # copy-out of step i-1 overlap the compute of step i (three streams, three device buffer sets)
    from rtx_b200.host import GluMlpHostSession

    session = GluMlpHostSession(wgu, wd, m_local)
    x_hosts = [x_host, x_host.clone().pin_memory()]
    y_hosts = [y_host, torch.empty_like(y_host).pin_memory()]
    for i in range(3):
        session.submit(x_hosts[i % 2], y_hosts[i % 2])
    session.drain()
    barrier()
    torch.cuda.synchronize()
    w0 = time.time()
    t0 = time.perf_counter()
    for i in range(args.steps):
        session.submit(x_hosts[i % 2], y_hosts[i % 2])
    session.drain()
    e2e_ms_total = (time.perf_counter() - t0) * 1e3   # spans three streams: host clock around submit..drain
    sampler.mark(w0, time.time())
    barrier()

    # the copies of the end-to-end step alone (X in and Y out at the same time, no compute): the PCIe
    # floor of the end-to-end number
    s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()
    c0, c1, c2, c3 = (torch.cuda.Event(enable_timing=True) for _ in range(4))
    torch.cuda.synchronize()
    with torch.cuda.stream(s_in):
        c0.record()
        for i in range(args.steps):
            x.copy_(x_hosts[i % 2], non_blocking=True)
        c1.record()
    with torch.cuda.stream(s_out):
        c2.record()
        for i in range(args.steps):
            y_hosts[i % 2].copy_(y, non_blocking=True)
        c3.record()
    torch.cuda.synchronize()
    copy_ms = max(c0.elapsed_time(c1), c2.elapsed_time(c3)) / args.steps

    # dominant kernel alone: the gate/up GEMM with the fused SwiGLU epilogue
    qx, sx = ops.mxfp8_quantize(x)
    qg, sg = ops.mxfp8_quantize(wgu)
    for _ in range(3):
        ops.mxfp8_gemm_glu_mx(qx, sx, qg, sg, m_local, INTER, K)
    torch.cuda.synchronize()
    w0 = time.time()
    ev0.record()
    for _ in range(args.steps):
        ops.mxfp8_gemm_glu_mx(qx, sx, qg, sg, m_local, INTER, K)
    ev1.record()
    torch.cuda.synchronize()
    sampler.mark(w0, time.time())
    clocks = sampler.stop()
    numa.__exit__(None, None, None)
    gemm_ms = ev0.elapsed_time(ev1) / args.steps
    ops.check_device_status(dev)

    t = torch.tensor([ms_total, e2e_ms_total, gemm_ms], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_total, e2e_ms_total, gemm_ms = (float(v) for v in t.tolist())

    if rank == 0:
        peaks = measured_peaks()
        flops_step_global = mlp_flops(m_local) * world
        value = flops_step_global * args.steps / (ms_total * 1e-3) / 1e12
        e2e_value = flops_step_global * args.steps / (e2e_ms_total * 1e-3) / 1e12
        gemm_tflops = 2.0 * m_local * (2 * INTER) * K / (gemm_ms * 1e-3) / 1e12
        fp8_peak = 2.0 * peaks["bf16_tflops"]
        traffic = None
        tpath = os.path.join(ROOT, "profiles", "roofline_traffic.json")
        if os.path.exists(tpath):
            with open(tpath) as f:
                traffic = json.load(f).get("gemm_glu_mxfp8_c2_dram_bytes_per_launch")
        line = {
            "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms_total / args.steps, "higher_is_better": True,
            "scaling": args.scaling, "vs_baseline": None, "dtype": "mxfp8 (e4m3 x e8m0), fp32 accumulate",
            "data": "synthetic",
            "config": {"workload": f"mxfp8_glu_mlp_fwd_m{M}_k{K}_i{INTER}", "m_per_gpu": m_local, "k": K,
                       "inter": INTER, "n_out": N_OUT, "parallelism": f"dp{world} (token rows sharded, weights replicated)",
                       "l2": "inputs exceed L2 (X 67 MB + weights 352 MB bf16 re-read every step)",
                       "hidden": "H leaves the gate/up epilogue already MXFP8-encoded; no BF16 H is materialized"},
            "tflops_per_gpu": value / world,
            "pct_of_nominal_fp8_peak": 100.0 * value / world / NOMINAL_FP8_TFLOPS,
            "pct_of_measured_fp8_proxy": 100.0 * value / world / fp8_peak,
            "e2e": {"value": e2e_value, "unit": "TFLOP/s", "h2d_bytes_per_step": x_host.numel() * 2 * world,
                    "d2h_bytes_per_step": y_host.numel() * 2 * world, "ms_per_step": e2e_ms_total / args.steps,
                    "api": "rtx_b200.host.GluMlpHostSession.submit/drain (copies overlapped with compute)",
                    "host_cpus": f"{len(numa.cpus)} CPUs next to the GPU" if numa.cpus else "unbound",
                    "copies_alone_ms_per_step": copy_ms,
                    "copies_alone_gbs_each_way": x_host.numel() * 2 / (copy_ms * 1e-3) / 1e9},
            "gpu_launches": launches_per_step * args.steps,
            "clocks": clocks,
            "roofline": {"kernel": "gemm_blockscaled_pair_kernel<mxfp8, glu_mx> (gate/up GEMM + SiLU*up + MXFP8 encode of H)", "bound": "tensor",
                         "achieved": gemm_tflops, "peak": fp8_peak, "unit": "TFLOP/s", "frac": gemm_tflops / fp8_peak,
                         "traffic": traffic, "ms_per_launch": gemm_ms,
                         "peak_note": f"2 x {peaks['source']} cuBLAS bf16 burst ({peaks['bf16_tflops']} TFLOP/s) as the "
                                      f"dense FP8 proxy; nominal dense FP8 is {NOMINAL_FP8_TFLOPS} TFLOP/s"},
        }
        if world == 1 and not args.no_cpu_baseline:
            threads = os.cpu_count() or 1
            m_s = M
            times, flops = cpu_sample_run(m_s, INTER, threads, 3, 1)
            line["cpu_baseline"] = {
                "value": flops * len(times) / sum(times) / 1e12, "unit": "TFLOP/s", "cores": threads, "kind": "port",
                "sample": f"{len(times)} runs (after 1 warm-up) of the reference CPU path on the whole workload: "
                          f"X {m_s} rows, full weights, {flops:.3e} flop per run, {sum(times):.1f} s in total"}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", choices=["own", "reference"], default="own")
    ap.add_argument("--scaling", choices=["weak", "strong"], default="weak")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--m", type=int, default=M, help="token rows per GPU (smaller values give profiler-sized cases)")
    ap.add_argument("--inter", type=int, default=INTER, help="SwiGLU intermediate width")
    args = ap.parse_args()
    globals()["M"], globals()["INTER"] = args.m, args.inter
    if args.impl == "reference":
        run_reference_arm(args)
    else:
        run_own_arm(args)


if __name__ == "__main__":
    main()
