"""Nikhilam INT8 KV on the GPU: bytes and scales bit-exact against the CPU oracle and
against the reference's own kernels compiled for sm_100a."""
import ctypes as C

import numpy as np
import pytest
import torch

import oracle as O
from logos_b200 import synthetic as syn

pytestmark = pytest.mark.gpu


def oracle_compress(x):
    qs, ss = [], []
    for t in x.reshape(-1, x.shape[-2] * x.shape[-1]):
        q, s = O.nikhilam_compress(t)
        qs.append(q)
        ss.append(s)
    return np.stack(qs).reshape(x.shape), np.array(ss, np.float32).reshape(x.shape[:-2])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("shape", [(1, 1, 1, 64), (2, 3, 17, 64), (4, 16, 512, 64), (1, 2, 33, 7)])
def test_compress_bit_exact(engine, dtype, shape):
    x = syn.normal_with_outliers(shape, 4, 1)
    xt = torch.from_numpy(x).cuda().to(dtype)
    xr = xt.float().cpu().numpy()          # what the kernel really sees
    q, s = engine.nikhilam_compress(xt)
    qo, so = oracle_compress(xr)
    assert np.array_equal(s.cpu().numpy().view(np.uint32), so.view(np.uint32)), "scales differ"
    assert np.array_equal(q.cpu().numpy(), qo), "int8 bytes differ"


def test_compress_edge_values(engine):
    cases = {
        "zeros": np.zeros((1, 16, 64), np.float32),
        "ties": (np.arange(1024, dtype=np.float32).reshape(1, 16, 64) - 512) * np.float32(0.5),
        "tiny": np.full((1, 16, 64), 1e-30, np.float32),
        "huge": np.full((1, 16, 64), 3e38, np.float32) * np.sign(np.random.default_rng(0).standard_normal((1, 16, 64))).astype(np.float32),
        "one_outlier": np.concatenate([np.full((1, 15, 64), 0.01, np.float32), np.full((1, 1, 64), 900.0, np.float32)], 1),
    }
    for name, x in cases.items():
        q, s = engine.nikhilam_compress(torch.from_numpy(x).cuda())
        qo, so = oracle_compress(x)
        assert np.array_equal(s.cpu().numpy().view(np.uint32), so.view(np.uint32)), name
        assert np.array_equal(q.cpu().numpy(), qo), name


def test_reference_test_fixtures_on_gpu(engine):
    # S13 ramp, M5 sine, MEM3 sawtooth (see tests/test_oracle_cpu.py for the citations)
    ramp = (5.0 + np.arange(2048, dtype=np.float32) * (4.84 / 2047)).astype(np.float32).reshape(1, 32, 64)
    sine = (7.5 * np.sin(np.arange(4096) * 0.01)).astype(np.float32).reshape(1, 64, 64)
    saw = ((np.arange(1 << 20) % 201) - 100).astype(np.float32).reshape(1, 1 << 14, 64)
    for x in (ramp, sine, saw):
        xt = torch.from_numpy(x).cuda()
        q, s = engine.nikhilam_compress(xt)
        xd = engine.nikhilam_decompress(q, s).cpu().numpy()
        qo, so = oracle_compress(x)
        assert np.array_equal(q.cpu().numpy(), qo)
        assert np.array_equal(xd, np.stack([O.nikhilam_dequantize(qo[0], so[0])]))
    assert np.abs(xd - saw).max() < 1.0


def test_cache_layout_and_append(engine):
    B, H, S, S_max, DH = 3, 4, 37, 64, 64
    k = syn.normal_with_outliers((B, H, S, DH), 4, 2)
    v = syn.normal_with_outliers((B, H, S, DH), 4, 3)
    kc = torch.zeros((B, H, S_max, DH), dtype=torch.int8, device="cuda")
    vc = torch.zeros_like(kc)
    _, ks = engine.nikhilam_compress(torch.from_numpy(k).cuda(), cache=kc)
    _, vs = engine.nikhilam_compress(torch.from_numpy(v).cuda(), cache=vc)
    qo, so = oracle_compress(k)
    assert np.array_equal(kc[:, :, :S].cpu().numpy(), qo) and not kc[:, :, S:].any()
    assert np.array_equal(ks.cpu().numpy(), so)
    # append one row per (b,h) at different positions, including a value far beyond the scale
    k_new = syn.normal((B, H, DH), 4, 4)
    k_new[0, 0, 0] = 1e4
    k_new[1, 1, 1] = -1e4
    v_new = syn.normal((B, H, DH), 4, 5)
    pos = np.array([S, S + 1, 0], np.int32)
    for dt in (torch.float32, torch.float16):
        kn, vn = torch.from_numpy(k_new).cuda().to(dt), torch.from_numpy(v_new).cuda().to(dt)
        kc2, vc2 = kc.clone(), vc.clone()
        engine.kv_append(kn, vn, kc2, vc2, ks, vs, torch.from_numpy(pos).cuda())
        knr, vnr = kn.float().cpu().numpy(), vn.float().cpu().numpy()
        exp_k, exp_v = kc.cpu().numpy().copy(), vc.cpu().numpy().copy()
        for b in range(B):
            for h in range(H):
                exp_k[b, h, pos[b]] = O.nikhilam_quantize(knr[b, h], ks[b, h].item())
                exp_v[b, h, pos[b]] = O.nikhilam_quantize(vnr[b, h], vs[b, h].item())
        assert np.array_equal(kc2.cpu().numpy(), exp_k)
        assert np.array_equal(vc2.cpu().numpy(), exp_v)
    assert exp_k[0, 0, S, 0] == 127 and exp_k[1, 1, S + 1, 1] == -127


def test_full_size_properties(engine):
    """One layer's worth of cache at the decode benchmark's size (64 x 16 x 8192 x 64 per
    tensor kind is 512 MiB of int8): checked through size-independent properties."""
    B, H, S, DH = 16, 16, 8192, 64
    g = torch.Generator(device="cuda").manual_seed(40)
    x = torch.randn((B, H, S, DH), device="cuda", generator=g)
    x[torch.rand(x.shape, device="cuda", generator=g) < 0.01] *= 8
    q, s = engine.nikhilam_compress(x)
    amax = x.abs().amax(dim=(-1, -2))
    want = (amax.cpu().numpy() + np.float32(1e-8)) / np.float32(127.5)   # IEEE fp32, as the reference's host code
    assert np.array_equal(s.cpu().numpy(), want)
    assert int(q.abs().max()) <= 127
    # every tensor uses its full range: the absmax element maps to +-127
    assert torch.equal(q.abs().amax(dim=(-1, -2)).to(torch.int32), torch.full((B, H), 127, dtype=torch.int32, device="cuda"))
    xd = engine.nikhilam_decompress(q, s)
    assert bool(((xd - x).abs() <= 0.5 * s[..., None, None] * 1.0001 + 1e-7).all())
    # idempotence: re-quantizing the dequantized tensor with the same scale returns the bytes
    samp = xd[3, 5].cpu().numpy()
    assert np.array_equal(O.nikhilam_quantize(samp, s[3, 5].item()), q[3, 5].cpu().numpy())
    # sampled tensors against the oracle, bit for bit
    for (b, h) in [(0, 0), (7, 9), (15, 15)]:
        qo, so = O.nikhilam_compress(x[b, h].cpu().numpy())
        assert so == s[b, h].item() and np.array_equal(qo, q[b, h].cpu().numpy())


@pytest.mark.skipif(O.refgpu() is None, reason="reference kernels not built")
def test_reference_kernels_second_witness(engine):
    """The reference's absmax/quantize/dequantize kernels (built without fast-math for
    sm_100a) give the same bytes as the oracle and as this engine."""
    R = O.refgpu()
    x = torch.from_numpy(syn.normal_with_outliers((8192, 64), 4, 7)).cuda()
    n = x.numel()
    amax = torch.zeros(1, device="cuda")
    assert R.refgpu_absmax(x.data_ptr(), amax.data_ptr(), n) == 0
    torch.cuda.synchronize()
    scale = np.float32((np.float32(amax.item()) + np.float32(1e-8)) / np.float32(127.5))
    q_ref = torch.empty(n, dtype=torch.int8, device="cuda")
    assert R.refgpu_quantize(x.data_ptr(), q_ref.data_ptr(), float(scale), n) == 0
    d_ref = torch.empty(n, device="cuda")
    assert R.refgpu_dequantize(q_ref.data_ptr(), d_ref.data_ptr(), float(scale), n) == 0
    torch.cuda.synchronize()
    q, s = engine.nikhilam_compress(x[None])
    qo, so = O.nikhilam_compress(x.cpu().numpy())
    assert s.item() == scale == so
    assert np.array_equal(q_ref.cpu().numpy().reshape(8192, 64), qo)
    assert torch.equal(q[0].reshape(-1), q_ref)
    assert torch.equal(engine.nikhilam_decompress(q, s).reshape(-1), d_ref)
