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


def _wrong_shape_worker(rank, world, port, ok):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        # rank 1 brings one head too many: every rank learns of it BEFORE the data collective
        mine = torch.zeros((3, 4 + rank, 5))
        try:
            sharding.check_slices(mine, world)
        except ValueError as e:
            ok[rank] = int("rank(s) [1]" in str(e))
        # equal slices pass
        sharding.check_slices(torch.zeros((3, 4, 5)), world)
        ok[world + rank] = 1
    finally:
        dist.destroy_process_group()


def test_mismatched_slice_is_reported_on_every_rank_before_the_collective():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    world = 2
    ok = mp.get_context("spawn").Array("i", [0] * (2 * world))
    mp.spawn(_wrong_shape_worker, args=(world, port, ok), nprocs=world, join=True)
    assert list(ok) == [1] * (2 * world)


def _absent_rank_worker(rank, world, port, ok, mode):
    import datetime
    import time
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=4))
    full = torch.arange(2 * 4 * 3, dtype=torch.float32).reshape(2, 4, 3)
    mine = sharding.shard_heads(full, rank, world)
    if mode == "late":
        if rank == 1:
            time.sleep(1.0)                 # late, but inside the limit: the step still completes
        ok[rank] = int(torch.equal(sharding.all_gather_heads(mine, world), full))
        dist.destroy_process_group()
        return
    # mode "missing": rank 1 leaves between steps without entering the collective
    if rank == 1:
        ok[rank] = 1
        return
    t0 = time.time()
    try:
        sharding.all_gather_heads(mine, world)
        ok[rank] = 0                        # must not "succeed" with a rank missing
    except Exception:
        ok[rank] = int(time.time() - t0 < 30)          # an error inside the limit, not an endless wait


@pytest.mark.parametrize("mode", ["late", "missing"])
def test_late_rank_is_waited_for_and_missing_rank_ends_in_an_error(mode):
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    world = 2
    ok = mp.get_context("spawn").Array("i", [0] * world)
    ctx = mp.spawn(_absent_rank_worker, args=(world, port, ok, mode), nprocs=world, join=False)
    ctx.join(timeout=60) if False else [p.join(60) for p in ctx.processes]
    for p in ctx.processes:
        if p.is_alive():
            p.terminate()
    assert list(ok) == [1] * world
