"""The data-parallel dW path on two CPU ranks (gloo): shard the token rows, compute per-rank
partial dW with the CPU oracle, all-reduce in FP32, and compare with the unsharded result.
The reference has no distributed tests (it is single GPU); this covers the new N > 1 logic."""
import os
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank: int, world: int, port: int, out_dir: str):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from oracle import mx_oracle as O
        from rtx_b200 import parallel as P

        torch.set_num_threads(2)
        inp = O.make_inputs(4, m=256, n=96, k=160)        # identical global tensors on every rank
        x, w, dy = inp["x"], inp["w"], inp["dy"]
        xs, dys = P.shard_rows(x, rank, world), P.shard_rows(dy, rank, world)
        assert xs.shape[0] == 256 // world and xs.shape[0] % 32 == 0

        def compute(g, xx, ww):
            dx, dw = O.mxfp8_backward(xx, ww, g, dw_dtype=torch.float32)
            return dx, dw

        dx, dw = P.data_parallel_linear_backward(dys, xs, w, compute=compute)
        dx_full, dw_full = O.mxfp8_backward(x, w, dy, dw_dtype=torch.float32)
        lo, hi = P.shard_bounds(256, rank, world)
        # dX rows are independent of the sharding: bit equal
        assert torch.equal(dx, dx_full[lo:hi])
        # dW: same quantized blocks (32-row blocks stay whole), FP32 summation order differs
        assert dw.dtype is torch.bfloat16
        rel = ((dw.float() - dw_full).norm() / dw_full.norm()).item()
        assert rel < 4e-3, rel
        assert (O.bf16_ulp_distance(dw, dw_full.bfloat16()) <= 1).float().mean() > 0.999
        # every rank holds the same reduced dW
        gathered = [torch.empty_like(dw) for _ in range(world)]
        dist.all_gather(gathered, dw)
        assert all(torch.equal(gathered[0], t) for t in gathered)
        # payload of a shard equals the payload of the same rows in the unsharded tensor
        q_shard, s_shard = O.mxfp8_quantize_transposed(xs)
        q_full, s_full = O.mxfp8_quantize_transposed(x)
        assert torch.equal(q_shard, q_full[:, lo:hi]) and torch.equal(s_shard, s_full[:, lo // 32:hi // 32])
        open(os.path.join(out_dir, f"ok{rank}"), "w").write("ok")
    finally:
        dist.destroy_process_group()


def test_dw_all_reduce_two_ranks(tmp_path):
    world, port = 2, 29500 + (os.getpid() % 400)
    mp.spawn(_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    assert all((tmp_path / f"ok{r}").exists() for r in range(world))


def test_shard_bounds_reject_partial_mx_blocks():
    from rtx_b200 import parallel as P

    assert P.shard_bounds(16384, 3, 8) == (6144, 8192)
    with pytest.raises(ValueError, match="32-row"):
        P.shard_bounds(100, 0, 2)
    with pytest.raises(TypeError, match="FP32"):
        P.all_reduce_dw(torch.zeros(2, 2, dtype=torch.bfloat16))
    assert P.all_reduce_dw(torch.zeros(2, 2)) is None      # no process group: nothing to do


def test_peer_reduce_scatter_block_rows():
    from rtx_b200 import parallel as P

    assert P.p2p_block_rows(4096, 8) == 512 and P.p2p_block_rows(4096, 2) == 2048
    assert P.p2p_block_rows(4096, 1) == 0          # one rank: nothing to scatter
    assert P.p2p_block_rows(1000, 2) == 0          # ragged: blocks must be whole 256-row tiles
    assert P.backward_collective(4096, 4096, torch.device("cpu")) == "none (one rank)"


def test_dw_bands_cover_the_rows_in_whole_tile_rows():
    from rtx_b200 import parallel as P

    # one wave per band (band_rows < 0): K = 4096 is 16 column tiles, 64 pairs hold 4 tile rows = 1024 rows
    assert P.dw_bands(4096, 4096, band_rows=-1, margin=20) == [(0, 1024), (1024, 2048), (2048, 3072), (3072, 4096)]
    # wide K: one tile row per band; ragged N: the last band takes the rest
    assert P.dw_bands(700, 14336, band_rows=-1, margin=20) == [(0, 256), (256, 512), (512, 700)]
    assert P.dw_bands(4096, 4096, band_rows=2048) == [(0, 2048), (2048, 4096)]
    assert P.dw_bands(4096, 4096) == [(0, 4096)] and P.dw_bands(700, 300) == [(0, 700)]      # default: one band
    for n, k in ((4096, 4096), (1000, 300), (256, 256), (5, 7)):
        bands = P.dw_bands(n, k)
        assert bands[0][0] == 0 and bands[-1][1] == n
        assert all(a[1] == b[0] for a, b in zip(bands, bands[1:])) and all(lo % 256 == 0 for lo, _ in bands)
