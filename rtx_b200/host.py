"""Host-buffer entry point for the SwiGLU MLP: the call a user with activations in
host memory makes.  Each `submit` copies X from pinned host memory to the device,
runs the MXFP8 MLP (quantize, gate/up GEMM with fused SiLU*up, quantize, down GEMM)
and copies Y back to pinned host memory.  Three streams and three device buffer sets
let the copy-in of step i+1 and the copy-out of step i-1 overlap the compute of
step i (a buffer set's X is free again as soon as its previous compute has finished,
its Y once the previous copy-out has); optionally each step is itself cut into
blocks of token rows that are copied, computed and returned one after another;
`drain()` waits for everything submitted.
"""

from __future__ import annotations

from typing import List, Optional

import torch

from . import ops


def gpu_local_cpus(device: torch.device) -> Optional[List[int]]:
    """CPUs of this process's allowed set that sit on the NUMA node of `device` (NVML's CPU affinity of the
    GPU, looked up by UUID so that CUDA_VISIBLE_DEVICES does not matter); None when NVML, the UUID or an
    overlap with the allowed set is missing."""
    import os

    try:
        import pynvml

        pynvml.nvmlInit()
        uuid = str(torch.cuda.get_device_properties(device).uuid)
        handle = pynvml.nvmlDeviceGetHandleByUUID(("GPU-" + uuid) if not uuid.startswith("GPU-") else uuid)
        words = (os.cpu_count() or 64) // 64 + 1
        mask = pynvml.nvmlDeviceGetCpuAffinity(handle, words)
    except Exception:
        return None
    local = {64 * w + b for w, word in enumerate(mask) for b in range(64) if (int(word) >> b) & 1}
    cpus = sorted(local & os.sched_getaffinity(0))
    return cpus or None


class numa_local:
    """Context manager: run the calling thread on the CPUs next to `device` while pinned host buffers are
    allocated (first touch puts their pages on that NUMA node) and copies are submitted; the previous
    affinity is restored on exit.  With eight GPUs behind two sockets, host buffers on the far socket send
    every host-device copy across the socket interconnect."""

    def __init__(self, device: torch.device):
        import os

        # RTXB_HOST_NUMA=0 leaves the affinity alone
        self.cpus = None if os.environ.get("RTXB_HOST_NUMA") == "0" else gpu_local_cpus(device)
        self.prev = None

    def __enter__(self):
        import os

        if self.cpus:
            self.prev = os.sched_getaffinity(0)
            os.sched_setaffinity(0, self.cpus)
        return self

    def __exit__(self, *exc):
        import os

        if self.prev is not None:
            os.sched_setaffinity(0, self.prev)
        return False


class GluMlpHostSession:
    """`chunk_rows` > 0 (default: off) pipelines WITHIN a step as well: the weights are quantized once per step, then every
    block of `chunk_rows` token rows is copied in, run through the two GEMMs and copied out on its own, so the
    first bytes of Y leave while later rows of X are still arriving.  A step's latency drops from (copy in +
    compute + copy out) to about one chunk of each beyond the longest of the three; the bits are those of
    the whole-step call (rows are independent, K is accumulated in the same order)."""

    def __init__(self, w_gate_up: torch.Tensor, w_down: torch.Tensor, max_rows: int, depth: int = 3,
                 chunk_rows: Optional[int] = None):
        if w_gate_up.device.type != "cuda":
            raise ValueError("weights must already be resident on the GPU")
        if chunk_rows is not None and (chunk_rows < 0 or chunk_rows % 128):
            raise ValueError("chunk_rows must be a non-negative multiple of 128 (whole scale tiles)")
        self.device = w_gate_up.device
        self.w_gate_up, self.w_down = w_gate_up.contiguous(), w_down.contiguous()
        self.k = w_gate_up.shape[1]
        self.inter = w_gate_up.shape[0] // 2
        self.n_out = w_down.shape[0]
        self.max_rows = max_rows
        self.depth = depth
        self.chunk_rows = chunk_rows
        with torch.cuda.device(self.device):
            self.copy_in, self.compute, self.copy_out = (torch.cuda.Stream() for _ in range(3))
        self.x = [torch.empty(max_rows, self.k, dtype=torch.bfloat16, device=self.device) for _ in range(depth)]
        self.y = [torch.empty(max_rows, self.n_out, dtype=torch.bfloat16, device=self.device) for _ in range(depth)]
        self.ws = ops.Workspace(self.device)
        self._compute_done: List[Optional[torch.cuda.Event]] = [None] * depth
        self._out_done: List[Optional[torch.cuda.Event]] = [None] * depth
        self._step = 0
        self.launches_per_step = 0      # kernels launched by the last submit

    def submit(self, x_host: torch.Tensor, y_host: torch.Tensor) -> None:
        """Enqueue one MLP forward; `x_host` / `y_host` must be pinned and stay alive until `drain()`."""
        if not (x_host.is_pinned() and y_host.is_pinned()):
            raise ValueError("host buffers must be pinned for asynchronous copies")
        m = x_host.shape[0]
        if m > self.max_rows or x_host.shape[1] != self.k:
            raise ValueError("activation shape does not fit this session")
        b = self._step % self.depth
        # Whole steps by default.  Blocks of 2048 rows on 8192-row steps measured 1.39-1.56 ms per step against
        # 1.48-1.51 whole on the same box (shorter fill and drain, but four times the dependencies between the
        # three streams): within noise; at 4096 rows and below the step is compute bound and blocks are slower.
        chunk = self.chunk_rows if self.chunk_rows else m
        if chunk <= 0 or chunk >= m:
            chunk = m
        with torch.cuda.device(self.device):
            # x[b] is free once the previous occupant's kernels have read it; y[b] once it has been copied out
            if self._compute_done[b] is not None:
                self.copy_in.wait_event(self._compute_done[b])
            if self._out_done[b] is not None:
                self.compute.wait_event(self._out_done[b])
            launches = 0
            if chunk < m:
                with torch.cuda.stream(self.compute):   # the step's weights, quantized once
                    qg, sg = ops.mxfp8_quantize(self.w_gate_up)
                    qd, sd = ops.mxfp8_quantize(self.w_down)
                launches += 2
            for r0 in range(0, m, chunk):
                r1 = min(r0 + chunk, m)
                with torch.cuda.stream(self.copy_in):
                    self.x[b][r0:r1].copy_(x_host[r0:r1], non_blocking=True)
                    arrived = torch.cuda.Event()
                    arrived.record(self.copy_in)
                self.compute.wait_event(arrived)
                with torch.cuda.stream(self.compute):
                    if chunk < m:
                        qx, sx = ops.mxfp8_quantize(self.x[b][r0:r1])
                        qh, sh, _ = ops.mxfp8_gemm_glu_mx(qx, sx, qg, sg, r1 - r0, self.inter, self.k)
                        ops.mxfp8_gemm(qh, sh, qd, sd, r1 - r0, self.n_out, self.inter, out=self.y[b][r0:r1])
                        launches += 3
                    else:
                        ops.mxfp8_glu_mlp_fwd(self.x[b][:m], self.w_gate_up, self.w_down, self.ws, None, self.y[b][:m],
                                              want_hidden=False)
                        launches += 5
                    computed = torch.cuda.Event()
                    computed.record(self.compute)
                self.copy_out.wait_event(computed)
                with torch.cuda.stream(self.copy_out):
                    y_host[r0:r1].copy_(self.y[b][r0:r1], non_blocking=True)
            self._compute_done[b] = computed
            self._out_done[b] = torch.cuda.Event()
            self._out_done[b].record(self.copy_out)
            self.launches_per_step = launches
        self._step += 1

    def drain(self) -> None:
        for s in (self.copy_in, self.compute, self.copy_out):
            s.synchronize()
        ops.check_device_status(self.device)
