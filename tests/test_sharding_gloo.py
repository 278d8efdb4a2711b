"""The multi-GPU decomposition (no data-path collective): shards partition the units exactly, and
the max-over-ranks reduction used for timing works over a real 2-process group (gloo, CPU)."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from mxdsa_b200 import sharding


def test_shards_partition_units():
    for n in (0, 1, 7, 64, 262144):
        for world in (1, 2, 3, 4, 8):
            pieces = [sharding.shard_range(n, r, world) for r in range(world)]
            assert pieces[0][0] == 0 and pieces[-1][1] == n
            assert all(pieces[i][1] == pieces[i + 1][0] for i in range(world - 1))
            sizes = [e - b for b, e in pieces]
            assert max(sizes) - min(sizes) <= 1
    assert sharding.shard_query_tokens(524288, 3, 8) == (196608, 262144)
    with pytest.raises(ValueError):
        sharding.shard_query_tokens(7, 0, 2)
    with pytest.raises(ValueError):
        sharding.shard_range(8, 2, 2)


def _worker(rank, world, port, out):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        b, e = sharding.shard_query_tokens(20, rank, world)
        sizes = [torch.zeros(2, dtype=torch.int64) for _ in range(world)]
        dist.all_gather(sizes, torch.tensor([b, e]))
        mx = sharding.max_over_ranks(10.0 + rank)
        dist.barrier()
        if rank == 0:
            out.put(([tuple(int(v) for v in s) for s in sizes], mx))
    finally:
        dist.destroy_process_group()


def test_two_rank_group_gloo():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    sizes, mx = out.get(timeout=120)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert sizes == [(0, 10), (10, 20)]
    assert mx == 11.0
