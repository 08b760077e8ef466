"""The head exchange over peer-mapped memory (logos_comm) and the decode kernel's peer epilogue.

On one GPU the ranks are contexts of one process whose kernels are issued in an order in which no
kernel ever has to wait for a later one: all ranks' producing kernels first, then all ranks' wait
kernels.  (Ranks as separate processes on ONE GPU would make one launch wait for another one's, which
nothing guarantees to run.)  With two or more GPUs the same path runs as one process per GPU, with the
blocks shared through CUDA IPC handles; that test needs `torch.cuda.device_count() >= 2`.
"""
import os
import socket

import numpy as np
import pytest
import torch

import oracle as O
from logos_b200 import lib as L
from logos_b200.engine import Comm, Engine
from helpers import assert_close

pytestmark = pytest.mark.gpu


def _inputs(B, H, S, seed, device="cuda"):
    g = torch.Generator(device=device).manual_seed(seed)
    kq = torch.randint(-127, 128, (B, H, S, 64), dtype=torch.int8, device=device, generator=g)
    vq = torch.randint(-127, 128, (B, H, S, 64), dtype=torch.int8, device=device, generator=g)
    ks = torch.rand((B, H), device=device, generator=g) * 0.02 + 0.01
    vs = torch.rand((B, H), device=device, generator=g) * 0.02 + 0.01
    q = torch.randn((B, H, 64), device=device, generator=g).half()
    qp = torch.randn((B, H, 64), device=device, generator=g).half()
    lens = torch.randint(1, S + 1, (B,), dtype=torch.int32, device=device, generator=g)
    lens[0] = S
    return q, qp, kq, vq, ks, vs, lens


def _slice(t, lo, hi):
    return t[:, lo:hi].contiguous()


@pytest.fixture()
def ranks():
    """`world` contexts on cuda:0 with their comms; closed afterwards."""
    made = []

    def make(world, gathered_bytes, chunk=256):
        engs = [Engine(0) for _ in range(world)]
        for e in engs:
            e.set_option(L.OPT_DECODE_CHUNK, chunk)
        comms = [Comm(e, r, world, gathered_bytes) for r, e in enumerate(engs)]
        Comm.connect_local(comms)
        made.append((engs, comms))
        return engs, comms

    yield make
    torch.cuda.synchronize()
    for engs, comms in made:
        for c in comms:
            c.close()
        for e in engs:
            e.close()


@pytest.mark.parametrize("world,window", [(2, 0), (4, 0), (2, 16)])
def test_local_ranks_match_one_gpu_bit_for_bit(engine, ranks, world, window):
    B, H, S = 3, 8, 2048
    p = L.Params.make(0.125, True, window, 4 if window else 0, 0.1, 0.05, 1.0, L.DIFFUSE_CAUSAL)
    engs, comms = ranks(world, B * H * 64 * 4)
    engine.set_option(L.OPT_DECODE_CHUNK, 256)
    engine.reserve(engine.decode_workspace_bytes(B, H, S, 64))
    per = H // world
    for e in engs:
        e.reserve(e.decode_workspace_bytes(B, per, S, 64))
    try:
        for step in range(3):               # three steps: both staging slots, the counter moves on
            q, qp, kq, vq, ks, vs, lens = _inputs(B, H, S, 100 + step)
            want = engine.decode_int8(q, qp, kq, vq, ks, vs, lens, p)
            outs = [torch.full((B, H, 64), float("nan"), device="cuda") for _ in range(world)]
            for r, e in enumerate(engs):    # every rank's rows leave first ...
                lo, hi = r * per, (r + 1) * per
                e.decode_int8_push(comms[r], _slice(q, lo, hi), _slice(qp, lo, hi), _slice(kq, lo, hi),
                                   _slice(vq, lo, hi), _slice(ks, lo, hi), _slice(vs, lo, hi), lens, p)
            for r in range(world):          # ... then nobody has to wait
                engs[r].decode_int8_collect(comms[r], outs[r])
            for e in engs:
                e.synchronize()
            for r in range(world):
                assert torch.equal(outs[r], want), f"step {step}, rank {r}: gathered rows differ from the one-GPU result"
        # and the one-GPU result itself against the oracle (last step's inputs)
        op = O.attn_params(0.125, True, window, 4 if window else 0, 0.1, 0.05, 1.0, O.DIFFUSE_CAUSAL)
        n = B * H
        ref = O.decode_int8_batch(q.float().cpu().numpy().reshape(n, 64), qp.float().cpu().numpy().reshape(n, 64),
                                  kq.cpu().numpy().reshape(n, S, 64), vq.cpu().numpy().reshape(n, S, 64),
                                  ks.cpu().numpy().reshape(n), vs.cpu().numpy().reshape(n),
                                  np.repeat(lens.cpu().numpy(), H), op).reshape(B, H, 64)
        assert_close(outs[0].cpu().numpy(), ref, "gathered rows vs oracle")
    finally:
        engine.set_option(L.OPT_DECODE_CHUNK, 0)


def test_any_per_head_tensor_is_gathered(ranks):
    B, Hl, world = 2, 3, 2
    local = [torch.randn((B, Hl, 40, 64), device="cuda").bfloat16() for _ in range(world)]
    engs, comms = ranks(world, B * Hl * world * 40 * 64 * 2)
    outs = [torch.zeros((B, Hl * world, 40, 64), dtype=torch.bfloat16, device="cuda") for _ in range(world)]
    for rep in range(2):
        for r in range(world):
            comms[r].push(local[r])
        for r in range(world):
            comms[r].wait(outs[r])
        torch.cuda.synchronize()
        want = torch.cat(local, dim=1)
        for r in range(world):
            assert torch.equal(outs[r], want)
        local = [t * 2 for t in local]


def test_wait_gives_up_when_a_rank_never_arrives(ranks):
    """Rank 1 never produces: rank 0's wait kernel runs into its time limit, returns, and the
    context reports which rank was missing.  The GPU is never left waiting: the limit is 50 ms."""
    B, Hl, world = 1, 1, 2
    engs, comms = ranks(world, B * Hl * world * 64 * 4)
    engs[0].set_option(L.OPT_PEER_WAIT_MS, 50)
    local = torch.ones((B, Hl, 64), device="cuda")
    out = torch.zeros((B, Hl * world, 64), device="cuda")
    comms[0].push(local)
    comms[0].wait(out)
    with pytest.raises(L.LogosError) as err:
        engs[0].synchronize()
    assert err.value.status == L.ERR_KERNEL_TIMEOUT and "rank 1" in str(err.value)
    engs[0].synchronize()                   # the status was cleared by the report; the context still works


def test_comm_argument_checks(engine):
    lib = L.load_library()
    import ctypes as C
    h = C.c_void_p()
    assert lib.logos_comm_create(engine.h, 2, 2, 1024, C.byref(h)) == L.ERR_INVALID_ARG      # rank outside the world
    assert lib.logos_comm_create(engine.h, 0, 9, 1024, C.byref(h)) == L.ERR_INVALID_ARG      # at most 8 ranks
    c = Comm(engine, 0, 2, 4096)
    try:
        t = torch.zeros((1, 1, 64), device="cuda")
        with pytest.raises(L.LogosError):    # not connected to its peer yet
            c.push(t)
    finally:
        c.close()
    one = Comm(engine, 0, 1, 4096)           # a world of one needs no connection
    try:
        t = torch.arange(64, device="cuda", dtype=torch.float32).view(1, 1, 64)
        out = torch.zeros_like(t)
        one.all_gather_heads(t, out)
        engine.synchronize()
        assert torch.equal(out, t)
        big = torch.zeros((1, 1, 4096), device="cuda")
        with pytest.raises(L.LogosError):    # larger than the slot
            one.push(big)
    finally:
        one.close()


# ---- one process per GPU -------------------------------------------------------------------------

def _rank_main(rank, world, port, results):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    import datetime
    import torch.distributed as dist
    from logos_b200.sharding import ShardedDecoder, head_range
    torch.cuda.set_device(rank)
    dist.init_process_group("cpu:gloo,cuda:nccl", rank=rank, world_size=world,
                            timeout=datetime.timedelta(seconds=60))
    eng = None
    try:
        eng = Engine(rank)
        eng.set_option(L.OPT_DECODE_CHUNK, 256)
        B, H, S = 4, 8, 4096
        p = L.Params.make(0.125, True, 0, 0, 0.1, 0.05, 1.0, L.DIFFUSE_CAUSAL)
        dev = f"cuda:{rank}"
        full = [t.to(dev) for t in _inputs(B, H, S, 7, device="cpu")]     # the same tensors on every rank
        q, qp, kq, vq, ks, vs, lens = full
        eng.reserve(eng.decode_workspace_bytes(B, H, S, 64))
        want = eng.decode_int8(q, qp, kq, vq, ks, vs, lens, p)             # all heads on this GPU
        lo, hi = head_range(H, rank, world)
        sl = lambda t: t[:, lo:hi].contiguous()
        gen = torch.Generator(device="cpu").manual_seed(8)               # the same new token on every rank
        knew, vnew = (torch.randn((B, H, 64), generator=gen).half().to(dev) for _ in range(2))
        passed = 0          # bit 0: peer exchange, bit 1: the same step as a graph, bit 2: library all-gather
        for mode in ("peer", "nccl"):
            kc, vc = sl(kq).clone(), sl(vq).clone()
            d = ShardedDecoder(eng, kc, vc, sl(ks), sl(vs), p, rank, world, gather=mode)
            for step in range(3):          # the same token three times: the append is idempotent
                got = d.step(sl(q), sl(qp), sl(knew), sl(vnew), lens)
                eng.synchronize()
            # the appended row replaced position len-1: recompute the one-GPU answer on the same cache
            kq2, vq2 = kq.clone(), vq.clone()
            eng.kv_append(knew, vnew, kq2, vq2, ks, vs, lens - 1)
            want2 = eng.decode_int8(q, qp, kq2, vq2, ks, vs, lens, p)
            eng.synchronize()
            if torch.equal(got, want2):
                passed |= 1 if mode == "peer" else 4
            else:
                print(f"rank {rank} {mode}: max-abs difference {float((got - want2).abs().max()):.3e}", flush=True)
            if mode == "peer":             # the same step replayed as a graph, twice
                d.capture(sl(q), sl(qp), sl(knew), sl(vnew), lens)
                for _ in range(2):
                    got_g = d.replay()
                eng.synchronize()
                if torch.equal(got_g, want2):
                    passed |= 2
            dist.barrier()
            d.close()
        results[rank] = passed
        del want
    finally:
        if eng is not None:
            torch.cuda.synchronize()
            eng.close()
        dist.destroy_process_group()


def test_one_process_per_gpu_bit_identical_to_one_gpu():
    world = min(torch.cuda.device_count(), 4)
    if world < 2:
        pytest.skip("needs at least two GPUs")
    import torch.multiprocessing as mp
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    results = mp.get_context("spawn").Array("i", [0] * world)
    mp.spawn(_rank_main, args=(world, port, results), nprocs=world, join=True)
    assert list(results) == [7] * world, "bit 0: peer exchange, bit 1: as a graph, bit 2: library all-gather"
