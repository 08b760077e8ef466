"""Host logic of the (batch x head) partition, on CPU: head ranges, and the all-gather of
per-rank outputs with two gloo ranks reproducing the single-rank tensor bit for bit."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from logos_b200 import sharding


def test_head_ranges_cover_and_partition():
    for world in (1, 2, 4, 8, 16):
        seen = []
        for r in range(world):
            lo, hi = sharding.head_range(16, r, world)
            assert hi - lo == 16 // world
            seen += list(range(lo, hi))
        assert seen == list(range(16))
    with pytest.raises(ValueError):
        sharding.head_range(16, 0, 3)       # ranks must divide the heads
    with pytest.raises(ValueError):
        sharding.head_range(16, 2, 2)


def test_shard_then_gather_single_rank_is_identity():
    x = torch.arange(2 * 4 * 3, dtype=torch.float32).reshape(2, 4, 3)
    assert torch.equal(sharding.all_gather_heads(sharding.shard_heads(x, 0, 1), 1), x)


def _worker(rank, world, port, ok):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        full = torch.arange(3 * 8 * 5, dtype=torch.float32).reshape(3, 8, 5) * 0.5
        mine = sharding.shard_heads(full, rank, world)
        assert mine.shape == (3, 8 // world, 5)
        got = sharding.all_gather_heads(mine, world)
        ok[rank] = int(torch.equal(got, full))
        # a rank whose slice has the wrong shape is caught before the collective
        lo, hi = sharding.head_range(8, rank, world)
        ok[world + rank] = int((lo, hi) == (rank * 4, rank * 4 + 4))
    finally:
        dist.destroy_process_group()


def test_all_gather_heads_two_gloo_ranks():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    world = 2
    ok = mp.get_context("spawn").Array("i", [0] * (2 * world))
    mp.spawn(_worker, args=(world, port, ok), nprocs=world, join=True)
    assert list(ok) == [1] * (2 * world)
