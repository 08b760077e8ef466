"""INT8-KV decode attention on the GPU against the CPU oracle (dequantize + Navier-Stokes
terms + last attention row), through the C ABI."""
import numpy as np
import pytest
import torch

import oracle as O
from logos_b200 import lib as L
from logos_b200 import synthetic as syn
from helpers import assert_close

pytestmark = pytest.mark.gpu

MODES = [L.DIFFUSE_NONE, L.DIFFUSE_CAUSAL, L.DIFFUSE_CENTRAL]


def make_cache(B, H, S_max, lens, seed, DH=64):
    """Pre-quantization K/V ~ N(0,1) with 1 % x8 outliers, quantized per (b,h) over the valid rows."""
    k = syn.normal_with_outliers((B, H, S_max, DH), seed, 1)
    v = syn.normal_with_outliers((B, H, S_max, DH), seed, 2)
    kq = np.zeros((B, H, S_max, DH), np.int8)
    vq = np.zeros_like(kq)
    ks = np.zeros((B, H), np.float32)
    vs = np.zeros_like(ks)
    for b in range(B):
        for h in range(H):
            n = lens[b]
            kq[b, h, :n], ks[b, h] = O.nikhilam_compress(k[b, h, :n])
            vq[b, h, :n], vs[b, h] = O.nikhilam_compress(v[b, h, :n])
    return kq, vq, ks, vs


def run_case(engine, B, H, S_max, lens, params, seed, tight=2e-5, DH=64):
    lens = np.asarray(lens, np.int32)
    kq, vq, ks, vs = make_cache(B, H, S_max, lens, seed, DH)
    q = syn.normal((B, H, DH), seed, 3).astype(np.float16)
    qp = syn.normal((B, H, DH), seed, 4).astype(np.float16)
    engine.reserve(engine.decode_workspace_bytes(B, H, S_max, DH))
    dev = lambda a: torch.from_numpy(a).cuda()
    out = engine.decode_int8(dev(q), dev(qp), dev(kq), dev(vq), dev(ks), dev(vs), dev(lens), params)
    op = O.attn_params(params.scale, params.causal, params.window, params.stride, params.ns_eta, params.ns_nu,
                       params.ns_alpha, params.diffuse_mode)
    n = B * H
    want = O.decode_int8_batch(q.astype(np.float32).reshape(n, DH), qp.astype(np.float32).reshape(n, DH),
                               kq.reshape(n, S_max, DH), vq.reshape(n, S_max, DH), ks.reshape(n), vs.reshape(n),
                               np.repeat(lens, H), op).reshape(B, H, DH)
    got = out.cpu().numpy()
    assert_close(got, want, f"decode lens={list(lens)}")
    assert np.abs(got - want).max() < tight * max(1.0, np.abs(want).max()), np.abs(got - want).max()
    return got


@pytest.mark.parametrize("mode", MODES)
@pytest.mark.parametrize("alpha", [1.0, 0.3])
def test_dense_small_and_ragged(engine, mode, alpha):
    p = L.Params.make(0.125, True, 0, 0, 0.1, 0.05, alpha, mode)
    run_case(engine, 4, 2, 128, [1, 2, 63, 128], p, seed=11)
    run_case(engine, 3, 3, 320, [65, 200, 320], p, seed=12)


@pytest.mark.parametrize("mode", MODES)
def test_dense_split_k(engine, mode):
    # few pairs and a long context: the engine splits the key axis into many chunks
    p = L.Params.make(0.125, True, 0, 0, 0.1, 0.05, 1.0, mode)
    run_case(engine, 2, 2, 4096, [4096, 1500], p, seed=13)
    run_case(engine, 1, 1, 8192, [8192], p, seed=14)
    # chunk boundaries: lengths one below / at / one above a multiple of every chunk size
    run_case(engine, 6, 1, 2048, [127, 128, 129, 1023, 1024, 1025], p, seed=15)


def test_dense_blend_split_k(engine):
    p = L.Params.make(0.125, True, 0, 0, 0.1, 0.05, 0.3, L.DIFFUSE_CENTRAL)
    run_case(engine, 2, 2, 4096, [4096, 777], p, seed=16)


def test_ns_off_variants(engine):
    # alpha 0 or eta = nu = 0 is plain softmax attention over the dequantized cache
    for p in (L.Params.make(0.125, True, 0, 0, 0.0, 0.0, 1.0, L.DIFFUSE_NONE),
              L.Params.make(0.125, True, 0, 0, 0.1, 0.05, 0.0, L.DIFFUSE_CAUSAL)):
        run_case(engine, 2, 2, 512, [512, 100], p, seed=17)


@pytest.mark.parametrize("mode", MODES)
@pytest.mark.parametrize("alpha", [1.0, 0.3])
def test_shunyam_window_and_landmarks(engine, mode, alpha):
    # window 64 / stride 16 is the reference's production setting (cuda/train_gpu.cu:1172-1173);
    # lens at and around the window switch the rule on and off (seq > window)
    p = L.Params.make(0.125, True, 64, 16, 0.1, 0.05, alpha, mode)
    run_case(engine, 6, 2, 1024, [1, 64, 65, 66, 500, 1024], p, seed=18)
    p = L.Params.make(0.125, True, 8, 5, 0.1, 0.05, alpha, mode)      # stride does not divide anything
    run_case(engine, 4, 2, 256, [9, 10, 77, 256], p, seed=19)
    p = L.Params.make(0.125, True, 32, 0, 0.1, 0.05, alpha, mode)     # pure window: no landmarks
    run_case(engine, 3, 2, 256, [33, 100, 256], p, seed=20)


def test_full_size_benchmark_shape(engine):
    """64 sequences x 16 heads x 8192 cached tokens (1 GiB of int8 K+V): a sample of pairs
    against the oracle, plus a property that needs no oracle -- permuting the cached
    tokens of a pair (keys and values together) leaves plain softmax attention unchanged."""
    B, H, S, DH = 64, 16, 8192, 64
    g = torch.Generator(device="cuda").manual_seed(4)
    kq = torch.randint(-127, 128, (B, H, S, DH), dtype=torch.int8, device="cuda", generator=g)
    vq = torch.randint(-127, 128, (B, H, S, DH), dtype=torch.int8, device="cuda", generator=g)
    ks = torch.rand((B, H), device="cuda", generator=g) * 0.02 + 0.01
    vs = torch.rand((B, H), device="cuda", generator=g) * 0.02 + 0.01
    q = torch.randn((B, H, DH), device="cuda", generator=g).half()
    qp = torch.randn((B, H, DH), device="cuda", generator=g).half()
    lens = torch.full((B,), S, dtype=torch.int32, device="cuda")
    engine.reserve(engine.decode_workspace_bytes(B, H, S, DH))
    p = L.Params.make(0.125, True, 0, 0, 0.1, 0.05, 1.0, L.DIFFUSE_CAUSAL)
    out = engine.decode_int8(q, qp, kq, vq, ks, vs, lens, p).cpu().numpy()
    op = O.attn_params(0.125, True, 0, 0, 0.1, 0.05, 1.0, O.DIFFUSE_CAUSAL)
    for (b, h) in [(0, 0), (17, 5), (63, 15)]:
        want = O.decode_int8_batch(q[b, h][None].float().cpu().numpy(), qp[b, h][None].float().cpu().numpy(),
                                   kq[b, h][None].cpu().numpy(), vq[b, h][None].cpu().numpy(),
                                   [ks[b, h].item()], [vs[b, h].item()], [S], op)
        assert_close(out[b, h], want[0], f"pair {(b, h)}")
    # permutation invariance of plain attention (no advection, no diffusion)
    p0 = L.Params.make(0.125, True, 0, 0, 0.0, 0.0, 1.0, L.DIFFUSE_NONE)
    a = engine.decode_int8(q, None, kq, vq, ks, vs, lens, p0).cpu().numpy()
    perm = torch.randperm(S, device="cuda", generator=g)
    kq.copy_(kq[:, :, perm].clone())
    vq.copy_(vq[:, :, perm].clone())
    b_ = engine.decode_int8(q, None, kq, vq, ks, vs, lens, p0).cpu().numpy()
    assert np.abs(a - b_).max() < 1e-5


@pytest.mark.parametrize("pinned", [True, False, "one block", "one block with the lengths"])
def test_host_step_entry_point(engine, pinned):
    """logos_decode_step_int8_host == append + decode on device tensors, with page-locked host
    buffers (separate allocations, which may be neighbours in address space but must not be copied as one),
    with pageable ones, with the four tensors in one page-locked block (sent as one copy), and with the lengths
    directly behind them in that block."""
    B, H, S_max, DH = 4, 4, 512, 64
    lens0 = np.array([10, 100, 300, 511], np.int32)
    kq, vq, ks, vs = make_cache(B, H, S_max, lens0, 21)
    dev = lambda a: torch.from_numpy(a).cuda()
    kc, vc, ksd, vsd = dev(kq), dev(vq), dev(ks), dev(vs)
    kc2, vc2 = kc.clone(), vc.clone()
    host = (lambda t: t.pin_memory()) if pinned else (lambda t: t)
    lens = None
    if pinned == "one block":
        block = torch.randn(4, B, H, DH).half().pin_memory()
        q, qp, kn, vn = block[0], block[1], block[2], block[3]
    elif pinned == "one block with the lengths":
        n16 = 4 * B * H * DH * 2
        buf = torch.empty(n16 + 4 * B, dtype=torch.uint8).pin_memory()
        block = buf[:n16].view(torch.float16).view(4, B, H, DH)
        block.copy_(torch.randn(4, B, H, DH).half())
        q, qp, kn, vn = block[0], block[1], block[2], block[3]
        lens = buf[n16:].view(torch.int32)
        lens.copy_(torch.from_numpy(lens0 + 1))
    else:
        q = host(torch.randn(B, H, DH).half())
        qp = host(torch.randn(B, H, DH).half())
        kn = host(torch.randn(B, H, DH).half())
        vn = host(torch.randn(B, H, DH).half())
    if lens is None:
        lens = host(torch.from_numpy(lens0 + 1))
    out = host(torch.full((B, H, DH), float("nan")))
    p = L.Params.make(0.125, True, 0, 0, 0.1, 0.05, 1.0, L.DIFFUSE_CAUSAL)
    engine.reserve(engine.decode_workspace_bytes(B, H, S_max, DH))
    engine.decode_step_host(q, qp, kn, vn, kc, vc, ksd, vsd, lens, p, out)
    engine.kv_append(kn.cuda(), vn.cuda(), kc2, vc2, ksd, vsd, dev(lens0))
    want = engine.decode_int8(q.cuda(), qp.cuda(), kc2, vc2, ksd, vsd, lens.cuda(), p)
    assert torch.equal(kc, kc2) and torch.equal(vc, vc2)
    assert torch.equal(out, want.cpu())


def test_argument_errors(engine):
    B, H, S, DH = 1, 1, 64, 64
    z8 = torch.zeros((B, H, S, DH), dtype=torch.int8, device="cuda")
    one = torch.ones((B, H), device="cuda")
    q = torch.zeros((B, H, DH), dtype=torch.float16, device="cuda")
    lens = torch.ones(B, dtype=torch.int32, device="cuda")
    p = L.Params.make(0.125, True, 0, 0, 0.1, 0.05, 1.0, L.DIFFUSE_CAUSAL)
    with pytest.raises(L.LogosError) as e:
        engine.decode_int8(q, None, z8, z8, one, one, lens, p)      # advection needs q_prev
    assert e.value.status == L.ERR_INVALID_ARG
    bad = L.Params.make(0.125, True, 0, 0, 0.1, 0.05, 1.0, 7)
    with pytest.raises(L.LogosError):
        engine.decode_int8(q, q, z8, z8, one, one, lens, bad)
    z8_24 = torch.zeros((B, H, S, 24), dtype=torch.int8, device="cuda")     # not a multiple of 16
    with pytest.raises(L.LogosError) as e:
        engine.decode_int8(q[..., :24].contiguous(), q[..., :24].contiguous(), z8_24, z8_24, one, one, lens, p)
    assert e.value.status == L.ERR_UNSUPPORTED


@pytest.mark.parametrize("DH", [16, 32, 96, 128])
def test_other_head_dimensions(engine, DH):
    """Head dimensions the model does not use (the reference's attention takes any DH <= 128): the general
    kernel, every switch, ragged lengths, against the same oracle."""
    sc = 1.0 / np.sqrt(DH)
    for mode in MODES:
        p = L.Params.make(sc, True, 0, 0, 0.1, 0.05, 1.0, mode)
        run_case(engine, 3, 2, 300, [1, 2, 300], p, seed=400 + DH + mode, DH=DH)
    run_case(engine, 2, 2, 700, [700, 333], L.Params.make(sc, True, 0, 0, 0.1, 0.05, 0.3, L.DIFFUSE_CENTRAL), seed=410 + DH, DH=DH)
    run_case(engine, 2, 2, 600, [600, 64], L.Params.make(sc, True, 64, 16, 0.1, 0.05, 1.0, L.DIFFUSE_CAUSAL), seed=420 + DH, DH=DH)
    run_case(engine, 1, 2, 600, [599], L.Params.make(sc, True, 32, 0, 0.1, 0.05, 0.6, L.DIFFUSE_CAUSAL), seed=430 + DH, DH=DH)
    run_case(engine, 1, 1, 4096, [4096], L.Params.make(sc, True, 0, 0, 0.0, 0.0, 1.0, L.DIFFUSE_NONE), seed=440 + DH, DH=DH)


def test_decode_step_replayed_as_cuda_graph(engine):
    """ShardedDecoder.capture / replay: the graph's inputs are refilled in place between replays and
    every replay gives bit for bit what the eager step gives on the same inputs."""
    from logos_b200.sharding import ShardedDecoder
    B, H, S_max, DH = 3, 4, 600, 64
    g = torch.Generator(device="cuda").manual_seed(77)
    kc = torch.randint(-127, 128, (B, H, S_max, DH), generator=g, device="cuda", dtype=torch.int8)
    vc = torch.randint(-127, 128, (B, H, S_max, DH), generator=g, device="cuda", dtype=torch.int8)
    ks = torch.rand((B, H), generator=g, device="cuda") * 0.05 + 0.01
    vs = torch.rand((B, H), generator=g, device="cuda") * 0.05 + 0.01
    p = L.Params.make(0.125, True, 0, 0, 0.1, 0.05, 1.0, L.DIFFUSE_CAUSAL)
    dec = ShardedDecoder(engine, kc.clone(), vc.clone(), ks, vs, p)
    ref = ShardedDecoder(engine, kc.clone(), vc.clone(), ks, vs, p)
    q, qp, kn, vn = (torch.randn((B, H, DH), generator=g, device="cuda").half() for _ in range(4))
    lens = torch.tensor([600, 333, 17], dtype=torch.int32, device="cuda")
    out = dec.capture(q, qp, kn, vn, lens)
    for rnd in range(3):
        for t in (q, qp, kn, vn):
            t.copy_(torch.randn((B, H, DH), generator=g, device="cuda").half())
        lens.copy_(torch.tensor([600 - rnd, 333 + rnd, 17 + 5 * rnd], dtype=torch.int32, device="cuda"))
        got = dec.replay().clone()
        want = ref.step(q, qp, kn, vn, lens).clone()
        torch.cuda.synchronize()
        assert got.data_ptr() != want.data_ptr() and out is dec.out_local
        assert torch.equal(got, want), f"round {rnd}"
        assert torch.equal(dec.kc, ref.kc) and torch.equal(dec.vc, ref.vc)
    # while a captured graph is alive the workspace it points into cannot be replaced
    with pytest.raises(L.LogosError) as err:
        engine.reserve(engine.decode_workspace_bytes(64, 16, 8192, DH) * 4)
    assert err.value.status == L.ERR_WORKSPACE
    dec.release()
    ref.release()


def test_dense_decode_rejects_viscosity_outside_unit_interval(engine):
    """The dense kernel carries the diffusion-folded weights as unsigned digits, which only holds for
    nu in [0, 1]; anything else is refused instead of being clipped silently."""
    dev = lambda a: torch.from_numpy(a).cuda()
    B, H, S = 1, 1, 64
    kq, vq, ks, vs = make_cache(B, H, S, [S], 31)
    q = dev(syn.normal((B, H, 64), 31, 3).astype(np.float16))
    engine.reserve(engine.decode_workspace_bytes(B, H, S, 64))
    for nu in (-0.1, 1.5):
        p = L.Params.make(0.125, True, 0, 0, 0.1, nu, 1.0, L.DIFFUSE_CAUSAL)
        with pytest.raises(L.LogosError) as err:
            engine.decode_int8(q, q, dev(kq), dev(vq), dev(ks), dev(vs), dev(np.array([S], np.int32)), p)
        assert err.value.status == L.ERR_UNSUPPORTED
    p = L.Params.make(0.125, True, 0, 0, 0.1, 1.5, 0.0, L.DIFFUSE_CAUSAL)    # alpha 0: diffusion is off, nu is unused
    engine.decode_int8(q, q, dev(kq), dev(vq), dev(ks), dev(vs), dev(np.array([S], np.int32)), p)
    engine.synchronize()


@pytest.mark.parametrize("chunk", [128, 192, 256, 512, 768, 960, 1024])
def test_every_split_size_against_the_oracle(engine, chunk):
    p = L.Params.make(0.125, True, 0, 0, 0.1, 0.05, 1.0, L.DIFFUSE_CAUSAL)
    engine.set_option(L.OPT_DECODE_CHUNK, chunk)
    try:
        run_case(engine, 2, 3, 2048, [2048, 777], p, seed=32)
    finally:
        engine.set_option(L.OPT_DECODE_CHUNK, 0)
    with pytest.raises(L.LogosError):
        engine.set_option(L.OPT_DECODE_CHUNK, 300)


def test_prefetch_depth_does_not_change_the_bits(engine):
    """LOGOS_OPT_DECODE_DEPTH only changes how many tiles a warp has in flight: same arithmetic, same order."""
    outs = []
    for depth in (2, 4):
        engine.set_option(L.OPT_DECODE_DEPTH, depth)
        try:
            outs.append([run_case(engine, 3, 2, 2048, [2048, 1, 777], L.Params.make(0.125, True, 0, 0, 0.1, 0.05, a, m), seed=33)
                         for a, m in ((1.0, L.DIFFUSE_CAUSAL), (0.4, L.DIFFUSE_CENTRAL))])
        finally:
            engine.set_option(L.OPT_DECODE_DEPTH, 0)
    for x, y in zip(*outs):
        assert np.array_equal(x, y)
    with pytest.raises(L.LogosError):
        engine.set_option(L.OPT_DECODE_DEPTH, 3)


@pytest.mark.parametrize("window,stride", [(0, 0), (64, 16)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_decode_step_with_16_bit_rows(engine, dtype, window, stride):
    """logos_decode_step_int8_to: the same step, the rows stored as the one rounding of the fp32 rows (dense and
    sparse kernel); a 16-bit type with another head dimension is refused."""
    B, H, S_max, DH = 3, 4, 700, 64
    g = torch.Generator(device="cuda").manual_seed(17 + window)
    kc = torch.randint(-127, 128, (B, H, S_max, DH), dtype=torch.int8, device="cuda", generator=g)
    vc = torch.randint(-127, 128, (B, H, S_max, DH), dtype=torch.int8, device="cuda", generator=g)
    ks = torch.rand((B, H), device="cuda", generator=g) + 0.5
    vs = torch.rand((B, H), device="cuda", generator=g) + 0.5
    q, qp, kn, vn = (torch.randn((B, H, DH), device="cuda", generator=g).half() for _ in range(4))
    lens = torch.tensor([700, 65, 1], dtype=torch.int32, device="cuda")
    p = L.Params.make(0.125, True, window, stride, 0.1, 0.05, 1.0, L.DIFFUSE_CAUSAL)
    engine.reserve(engine.decode_workspace_bytes(B, H, S_max, DH))
    kc2, vc2 = kc.clone(), vc.clone()
    want = engine.decode_step(q, qp, kn, vn, kc, vc, ks, vs, lens, p)
    got = engine.decode_step(q, qp, kn, vn, kc2, vc2, ks, vs, lens, p, out_dtype=dtype)
    engine.synchronize()
    assert got.dtype == dtype and torch.equal(got, want.to(dtype))
    assert torch.equal(kc, kc2) and torch.equal(vc, vc2)
    z = torch.zeros((1, 1, 64, 32), dtype=torch.int8, device="cuda")
    one = torch.ones((1, 1), device="cuda")
    q32 = torch.zeros((1, 1, 32), dtype=torch.float16, device="cuda")
    with pytest.raises(L.LogosError) as e:
        engine.decode_step(q32, q32, q32, q32, z, z, one, one, torch.ones(1, dtype=torch.int32, device="cuda"), p, out_dtype=dtype)
    assert e.value.status == L.ERR_UNSUPPORTED


@pytest.mark.parametrize("alpha,mode", [(1.0, L.DIFFUSE_CAUSAL), (0.4, L.DIFFUSE_CENTRAL), (1.0, L.DIFFUSE_NONE)])
def test_window_step_appends_inside_the_decode_kernel(engine, alpha, mode):
    """With a window the step is one kernel that quantises the new rows itself: the cache bytes and the rows are those
    of logos_kv_append followed by logos_decode_int8, also at position 0, at the last row of the cache, for a
    sequence shorter than the window and for a length outside the cache (rejected, nothing written)."""
    B, H, S_max, DH = 6, 3, 400, 64
    g = torch.Generator(device="cuda").manual_seed(23 + int(alpha * 10) + mode)
    kc = torch.randint(-127, 128, (B, H, S_max, DH), dtype=torch.int8, device="cuda", generator=g)
    vc = torch.randint(-127, 128, (B, H, S_max, DH), dtype=torch.int8, device="cuda", generator=g)
    ks = torch.rand((B, H), device="cuda", generator=g) * 0.05 + 0.01
    vs = torch.rand((B, H), device="cuda", generator=g) * 0.05 + 0.01
    q, qp = (torch.randn((B, H, DH), device="cuda", generator=g).half() for _ in range(2))
    kn, vn = (torch.randn((B, H, DH), device="cuda", generator=g).half() * 3.0 for _ in range(2))   # some values saturate
    lens = torch.tensor([400, 1, 2, 66, 200, 401], dtype=torch.int32, device="cuda")
    p = L.Params.make(0.125, True, 64, 16, 0.1, 0.05, alpha, mode)
    engine.reserve(engine.decode_workspace_bytes(B, H, S_max, DH))
    kc2, vc2 = kc.clone(), vc.clone()
    got = engine.decode_step(q, qp, kn, vn, kc, vc, ks, vs, lens, p)
    engine.kv_append(kn, vn, kc2, vc2, ks, vs, lens - 1)
    want = engine.decode_int8(q, qp, kc2, vc2, ks, vs, lens, p)
    engine.synchronize()
    assert torch.equal(kc, kc2) and torch.equal(vc, vc2)
    assert torch.equal(got, want)
