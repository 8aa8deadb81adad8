"""CPU, 2 processes over gloo: the batch-sharding helpers used by the multi-GPU launcher."""
import os
import socket

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from coda_gqa_l_b200.sharding import gather_rows, max_over_ranks, shard_bounds, shard_of, sum_over_ranks


def test_shard_bounds_cover_the_batch():
    assert shard_bounds(256, 8) == [(32 * r, 32 * r + 32) for r in range(8)]
    assert shard_bounds(5, 2) == [(0, 3), (3, 5)]
    assert shard_bounds(1, 4) == [(0, 1), (1, 1), (1, 1), (1, 1)]


def _worker(rank, world, port, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        full = torch.arange(5 * 3, dtype=torch.float32).view(5, 3)
        mine = shard_of(full, rank, world)
        assert mine.shape[0] == (3 if rank == 0 else 2)
        back = gather_rows(mine * 2)
        assert torch.equal(back, full * 2)
        assert max_over_ranks(1.0 + rank) == 2.0
        assert sum_over_ranks(float(mine.shape[0])) == 5.0
        ret[rank] = 1
    finally:
        dist.destroy_process_group()


def test_two_rank_shard_and_gather():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    ret = ctx.Manager().dict()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, ret)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    assert dict(ret) == {0: 1, 1: 1}
