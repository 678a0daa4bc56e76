"""Column sharding of the LM head / large-N projections: slab arithmetic, and the gather on the
gloo backend with two CPU ranks (the same host code the NCCL path runs)."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from libr3d_b200.shard import gather_columns, gather_topk, slab_of
from oracle import oracle as orc


@pytest.mark.parametrize("n,world", [(151936, 1), (151936, 2), (151936, 4), (151936, 8), (27648, 8),
                                     (5120, 8), (130, 4), (128, 8)])
def test_slabs_cover_rows_once(n, world):
    slabs = [slab_of(n, world, r) for r in range(world)]
    assert len({s.padded for s in slabs}) == 1 and slabs[0].padded % 128 == 0
    covered = np.zeros(n, np.int32)
    for s in slabs:
        assert 0 <= s.rows <= s.padded and s.start + s.rows <= n
        covered[s.start:s.start + s.rows] += 1
    assert (covered == 1).all()
    assert all(slabs[i].start <= slabs[i + 1].start for i in range(world - 1))
    # 151936 = 1187 tiles of 128: eight ranks take 149 tiles each, the last one 144
    if (n, world) == (151936, 8):
        assert slabs[0].padded == 149 * 128 and slabs[7].rows == 144 * 128


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank(rank, world, port, n, M, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        g = torch.Generator().manual_seed(7)
        full = torch.randn((M, n), generator=g)                      # the unsharded result
        s = slab_of(n, world, rank)
        local = torch.full((M, s.padded), float("nan"))               # padding columns are don't-care
        local[:, :s.rows] = full[:, s.start:s.start + s.rows]
        got = gather_columns(local, n)
        out[rank] = bool(torch.equal(got, full))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("n,M", [(1000, 3), (151936, 1), (256, 16)])
def test_gather_equals_unsharded_two_ranks(n, M):
    mgr = mp.Manager()
    out = mgr.dict()
    port = _free_port()
    mp.spawn(_rank, args=(2, port, n, M, out), nprocs=2, join=True)
    assert dict(out) == {0: True, 1: True}


def _rank_topk(rank, world, port, n, M, R, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        rng = np.random.default_rng(3)
        # few distinct bf16 values: ties inside a slab and across slabs; one row with a single finite value
        bits = orc.f32_to_bf16_bits((np.round(rng.standard_normal((M, n)) * 4) / 2).astype(np.float32))
        bits[-1, :] = 0xFF80
        bits[-1, n // 2 + 3] = 0x3F80
        s = slab_of(n, world, rank)
        # what this rank's row_topk row would write (the CPU oracle stands in for the GPU kernel here)
        idx, val = orc.row_topk(np.ascontiguousarray(bits[:, s.start:s.start + s.rows]), R, s.start)
        pairs = np.stack([idx.view(np.float32), val], axis=-1)
        gi, gv = gather_topk(torch.from_numpy(pairs))
        wi, wv = orc.row_topk(bits, R, 0)
        out[rank] = bool(np.array_equal(gi.numpy(), wi) and np.array_equal(gv.numpy().view(np.uint32), wv.view(np.uint32)))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("n,M,R", [(1024, 3, 8), (4096, 2, 32), (256, 4, 32)])
def test_sharded_topk_pairs_merge_two_ranks(n, M, R):
    mgr = mp.Manager()
    out = mgr.dict()
    port = _free_port()
    mp.spawn(_rank_topk, args=(2, port, n, M, R, out), nprocs=2, join=True)
    assert dict(out) == {0: True, 1: True}
