"""Failure handling on the host side and memory-safety checks that fault nothing: an allocator that
refuses, canary-padded output buffers around the kernels at odd shapes.  (The kernels' own bounded waits
are exercised in test_umma_selftest_gpu.py and test_comm_gpu.py.)"""
import ctypes as C

import numpy as np
import pytest
import torch

from logos_b200 import lib as L
from logos_b200.engine import Engine

pytestmark = pytest.mark.gpu


def test_reserve_through_a_caller_allocator_that_can_refuse():
    eng = Engine(0)
    try:
        held = {}                       # pointer -> tensor that backs it
        state = {"refuse": False, "calls": 0, "freed": 0}

        @L.ALLOC_FN
        def alloc(pptr, nbytes, user):
            state["calls"] += 1
            if state["refuse"]:
                return 1
            t = torch.empty((nbytes + 255,), dtype=torch.uint8, device="cuda")
            p = (t.data_ptr() + 255) & ~255
            held[p] = t
            pptr[0] = p
            return 0

        @L.FREE_FN
        def free(ptr, user):
            state["freed"] += 1
            held.pop(ptr, None)

        assert eng.lib.logos_ctx_set_allocator(eng.h, alloc, free, None) == L.OK
        small = eng.decode_workspace_bytes(2, 2, 256, 64)
        eng.reserve(small)
        assert state["calls"] == 1 and len(held) == 1
        # the pool runs dry: the call fails with a clear status and the context keeps its workspace
        state["refuse"] = True
        with pytest.raises(L.LogosError) as err:
            eng.reserve(small * 64)
        assert err.value.status == L.ERR_WORKSPACE and "allocator" in str(err.value)
        assert len(held) == 1 and state["freed"] == 0
        # ... and still works with what it has
        g = torch.Generator(device="cuda").manual_seed(1)
        kq = torch.randint(-127, 128, (2, 2, 256, 64), dtype=torch.int8, device="cuda", generator=g)
        sc = torch.full((2, 2), 0.02, device="cuda")
        q = torch.randn((2, 2, 64), device="cuda", generator=g).half()
        lens = torch.tensor([256, 100], dtype=torch.int32, device="cuda")
        p = L.Params.make(0.125, True, 0, 0, 0.0, 0.0, 1.0, L.DIFFUSE_NONE)
        eng.set_option(L.OPT_DECODE_CHUNK, 128)          # two splits: the workspace is really used
        out = eng.decode_int8(q, None, kq, kq, sc, sc, lens, p)
        eng.synchronize()
        assert bool(torch.isfinite(out).all())
        # a larger request once the pool has room again: new block first, then the old one goes back
        state["refuse"] = False
        eng.reserve(small * 4)
        assert state["freed"] == 1 and len(held) == 1
    finally:
        eng.close()
    assert state["freed"] == 2 and not held          # destroying the context returned the last block


class Guarded:
    """A tensor inside a larger buffer whose margins carry a pattern; check() proves nothing wrote there."""

    def __init__(self, shape, dtype, pad_bytes=4096):
        n = int(np.prod(shape)) * torch.empty((), dtype=dtype).element_size()
        self.raw = torch.full((pad_bytes + n + pad_bytes,), 0xA5, dtype=torch.uint8, device="cuda")
        self.pad, self.n = pad_bytes, n
        self.t = self.raw[pad_bytes:pad_bytes + n].view(dtype).view(shape)

    def check(self, what):
        lo, hi = self.raw[:self.pad], self.raw[self.pad + self.n:]
        assert bool((lo == 0xA5).all()) and bool((hi == 0xA5).all()), f"{what}: wrote outside its output"


@pytest.mark.parametrize("S,window,stride", [(1, 0, 0), (129, 0, 0), (257, 0, 0), (300, 64, 0), (333, 64, 16), (77, 8, 5)])
def test_attention_kernels_stay_inside_their_output(engine, S, window, stride):
    B, H = 2, 3
    g = torch.Generator(device="cuda").manual_seed(S)
    Q, K, V = (torch.randn((B, H, S, 64), device="cuda", generator=g).bfloat16() for _ in range(3))
    p = L.Params.make(0.125, True, window, stride, 0.1, 0.05, 1.0, L.DIFFUSE_CAUSAL)
    for dt in (torch.bfloat16, torch.float32):
        out = Guarded((B, H, S, 64), dt)
        engine.attention(Q, K, V, p, out=out.t)
        engine.synchronize()
        out.check(f"attention S={S} window={window} stride={stride} {dt}")
        assert bool(torch.isfinite(out.t.float()).all())


def test_cache_kernels_stay_inside_their_outputs(engine):
    B, H, S, S_max = 3, 2, 101, 130
    g = torch.Generator(device="cuda").manual_seed(9)
    x = torch.randn((B, H, S, 64), device="cuda", generator=g)
    cache = Guarded((B * H, S_max, 64), torch.int8)
    cache.t.zero_()
    _, ks = engine.nikhilam_compress(x, cache=cache.t)
    engine.synchronize()
    cache.check("kv_quantize")
    assert bool((cache.t[:, S:] == 0).all())                 # rows beyond S are not touched either
    kc = cache.t.view(B, H, S_max, 64)
    new = torch.randn((B, H, 64), device="cuda", generator=g).half()
    pos = torch.tensor([S, S_max - 1, S_max + 7], dtype=torch.int32, device="cuda")      # the last one is out of range
    engine.kv_append(new, new, kc, kc, ks, ks, pos)
    engine.synchronize()
    cache.check("kv_append")                                 # the out-of-range row was rejected, not written
    lens = torch.tensor([S + 1, S_max, 5], dtype=torch.int32, device="cuda")
    out = Guarded((B, H, 64), torch.float32)
    engine.reserve(engine.decode_workspace_bytes(B, H, S_max, 64))
    q = torch.randn((B, H, 64), device="cuda", generator=g).half()
    for w, st in ((0, 0), (16, 4)):
        p = L.Params.make(0.125, True, w, st, 0.1, 0.05, 1.0, L.DIFFUSE_CAUSAL)
        engine.decode_int8(q, q, kc, kc, ks, ks, lens, p, out=out.t)
        engine.synchronize()
        out.check(f"decode window={w}")
    deq = Guarded((B * H, S, 64), torch.float32)
    engine.lib.logos_kv_dequantize(engine.h, C.c_void_p(kc.data_ptr()), S_max * 64, C.c_void_p(ks.data_ptr()),
                                   C.c_void_p(deq.t.data_ptr()), S * 64, B * H, S * 64)
    engine.synchronize()
    deq.check("kv_dequantize")


def test_projection_stays_inside_its_outputs(engine):
    B, S, H, D = 2, 77, 3, 136
    g = torch.Generator(device="cuda").manual_seed(3)
    X = torch.randn((B * S, D), device="cuda", generator=g).bfloat16()
    Wt = (torch.randn((3 * H * 64, D), device="cuda", generator=g) * 0.05).bfloat16()
    outs = [Guarded((B, H, S, 64), torch.bfloat16) for _ in range(3)]
    rc = engine.lib.logos_qkv_project(engine.h, L.BF16, C.c_void_p(X.data_ptr()), C.c_void_p(Wt.data_ptr()),
                                      *(C.c_void_p(o.t.data_ptr()) for o in outs), B, S, H, D, None, None)
    assert rc == L.OK
    engine.synchronize()
    for o in outs:
        o.check("qkv_project")
    C_out = Guarded((B * S, 192), torch.float32)
    engine.project(X, (torch.randn((192, D), device="cuda", generator=g) * 0.05).bfloat16(), out=C_out.t)
    engine.synchronize()
    C_out.check("project")
