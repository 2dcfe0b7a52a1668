"""Row-sharded MXFP8 backward on two real GPUs: dX local, FP32 partial dW summed by NCCL.

Needs two visible GPUs (skipped otherwise).  Each rank runs in its own process, one GPU each, and
leaves only between steps with nothing in flight.  NVLS is turned off for the ranks: a two-rank
correctness check does not need in-switch reduction.
"""

import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import mx_oracle as O

pytestmark = pytest.mark.gpu


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, out_dir: str, route: str):
    os.environ.update({"MASTER_ADDR": "127.0.0.1", "MASTER_PORT": str(port), "NCCL_NVLS_ENABLE": "0"})
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    from rtx_b200 import ops, parallel

    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev, pg_options=parallel.nccl_options())
    try:
        inp = O.make_inputs(4, m=512, n=1024, k=384)
        x, w, dy = inp["x"], inp["w"], inp["dy"]
        xs = parallel.shard_rows(x, rank, world).to(dev)
        gs = parallel.shard_rows(dy, rank, world).to(dev)
        parallel.DW_BAND_ROWS = 256          # NCCL route: four bands of dW, four all-reduces
        parallel.P2P_REDUCE_SCATTER = route == "peer"
        for _ in range(3):                    # repeated steps reuse the staging slots
            dx, dw = parallel.data_parallel_linear_backward(gs, xs, w.to(dev))
        torch.cuda.synchronize()
        ops.check_device_status(dev)
        took = parallel.backward_collective(1024, 384, dev)
        assert took.startswith("reduce-scatter" if route == "peer" else "NCCL all-reduce"), took
        torch.save({"dx": dx.cpu(), "dw": dw.cpu()}, os.path.join(out_dir, f"rank{rank}.pt"))
        dist.barrier(device_ids=[rank])
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("route", ["peer", "nccl"])
def test_dw_all_reduce_matches_single_gpu_two_ranks(tmp_path, route):
    """Both routes of the data-parallel dW: the reduce-scatter through peer memory inside the GEMM epilogue
    (+ BF16 all-gather) and the banded NCCL all-reduce."""
    if not torch.cuda.is_available() or torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    world = 2
    mp.start_processes(_worker, args=(world, _free_port(), str(tmp_path), route), nprocs=world, join=True,
                       start_method="spawn")
    inp = O.make_inputs(4, m=512, n=1024, k=384)    # dW [1024, 384]: several bands, each with its own all-reduce
    x, w, dy = inp["x"], inp["w"], inp["dy"]
    want_dx, want_dw = O.mxfp8_backward(x, w, dy)
    parts = [torch.load(os.path.join(str(tmp_path), f"rank{r}.pt")) for r in range(world)]
    # dW: identical on both ranks; equal to the single-GPU oracle up to FP32 summation order
    assert torch.equal(parts[0]["dw"], parts[1]["dw"])
    rep = O.parity_report(parts[0]["dw"], want_dw)
    assert rep["rel_fro"] <= 1e-3 and rep["frac_le_1ulp"] >= 0.999, rep
    # dX: each rank's rows are exactly the single-GPU rows (no collective, same blocks)
    got_dx = torch.cat([p["dx"] for p in parts], dim=0)
    rep = O.parity_report(got_dx, want_dx)
    assert rep["rel_fro"] <= 1e-3 and rep["frac_le_1ulp"] >= 0.999, rep
