"""The whole-model INT8 KV cache container driven by the engine's kernels: a two-layer
prefill -> append -> decode loop over arena slices, and a trip through the disk format."""
import numpy as np
import pytest
import torch

import oracle as O
from logos_b200 import lib as L
from logos_b200 import synthetic as syn
from logos_b200.kvcache import KVCache
from helpers import assert_close

pytestmark = pytest.mark.gpu


def test_two_layer_generation_over_the_arena(engine, tmp_path):
    LAYERS, B, H, S0, S_max, DH, steps = 2, 2, 3, 70, 128, 64, 3
    cache = KVCache(LAYERS, B, H, S_max, DH)
    dev = lambda a: torch.from_numpy(a).cuda()
    ref = []          # per layer: oracle-side int8 rows and scales
    for l in range(LAYERS):
        k = syn.normal_with_outliers((B, H, S0, DH), 91 + l, 1)
        v = syn.normal_with_outliers((B, H, S0, DH), 91 + l, 2)
        cache.fill(engine, l, dev(k), dev(v))
        kq = np.zeros((B, H, S_max, DH), np.int8)
        vq = np.zeros_like(kq)
        ks = np.zeros((B, H), np.float32)
        vs = np.zeros_like(ks)
        for b in range(B):
            for h in range(H):
                kq[b, h, :S0], ks[b, h] = O.nikhilam_compress(k[b, h])
                vq[b, h, :S0], vs[b, h] = O.nikhilam_compress(v[b, h])
        ref.append((kq, vq, ks, vs))
    cache.set_lens(S0)
    for l in range(LAYERS):      # bit-exact bytes and scales in the arena slices
        kc, vc, ks, vs = cache.layer(l)
        assert np.array_equal(kc.cpu().numpy(), ref[l][0]) and np.array_equal(vc.cpu().numpy(), ref[l][1])
        assert np.array_equal(ks.cpu().numpy(), ref[l][2]) and np.array_equal(vs.cpu().numpy(), ref[l][3])

    engine.reserve(engine.decode_workspace_bytes(B, H, S_max, DH))
    p = L.Params.make(0.125, True, 0, 0, 0.1, 0.05, 1.0, L.DIFFUSE_CAUSAL)
    op = O.attn_params(0.125, True, 0, 0, 0.1, 0.05, 1.0, L.DIFFUSE_CAUSAL)
    n = B * H
    qp = [syn.normal((B, H, DH), 95, 3 + l).astype(np.float16) for l in range(LAYERS)]
    for step in range(steps):
        pos = S0 + step
        if step == 1:            # the cache survives a trip to disk in the middle of a generation
            path = str(tmp_path / "kv.bin")
            cache.dump(path)
            cache = KVCache.load(path)
        for l in range(LAYERS):
            q = syn.normal((B, H, DH), 96 + l, 10 + step).astype(np.float16)
            kn = syn.normal((B, H, DH), 96 + l, 30 + step).astype(np.float16)
            vn = syn.normal((B, H, DH), 96 + l, 50 + step).astype(np.float16)
            cache.append(engine, l, dev(kn), dev(vn))
            kq, vq, ks, vs = ref[l]
            for b in range(B):
                for h in range(H):
                    kq[b, h, pos] = O.nikhilam_quantize(kn[b, h].astype(np.float32), ks[b, h])
                    vq[b, h, pos] = O.nikhilam_quantize(vn[b, h].astype(np.float32), vs[b, h])
            kc, vc, ksd, vsd = cache.layer(l)
            lens = cache.lens + 1
            out = engine.decode_int8(dev(q), dev(qp[l]), kc, vc, ksd, vsd, lens, p).cpu().numpy()
            want = O.decode_int8_batch(q.astype(np.float32).reshape(n, DH), qp[l].astype(np.float32).reshape(n, DH),
                                       kq.reshape(n, S_max, DH), vq.reshape(n, S_max, DH), ks.reshape(n), vs.reshape(n),
                                       np.full(n, pos + 1, np.int32), op).reshape(B, H, DH)
            assert_close(out, want, f"layer {l} step {step}", 2e-5, 1e-5)
            qp[l] = q
        cache.advance()
    assert int(cache.lens[0]) == S0 + steps
    for l in range(LAYERS):
        kc, vc, _, _ = cache.layer(l)
        assert np.array_equal(kc.cpu().numpy(), ref[l][0]) and np.array_equal(vc.cpu().numpy(), ref[l][1])


def test_prefill_in_one_call_fills_the_cache(engine):
    """logos_prefill_fwd = logos_kv_quantize of the raw K and V + logos_attention_fwd, bit for bit."""
    B, H, S, S_max, DH = 2, 3, 200, 256, 64
    dev = lambda a: torch.from_numpy(a).cuda().bfloat16()
    Q, K, V = (dev(syn.normal_with_outliers((B, H, S, DH), 97, t)) for t in (1, 2, 3))
    p = L.Params.make(0.125, True, 0, 0, 0.1, 0.05, 1.0, L.DIFFUSE_CAUSAL)
    kc = torch.zeros((B, H, S_max, DH), dtype=torch.int8, device="cuda")
    vc = torch.zeros_like(kc)
    ks = torch.zeros((B, H), dtype=torch.float32, device="cuda")
    vs = torch.zeros_like(ks)
    out = engine.prefill(Q, K, V, p, kc, vc, ks, vs, out_dtype=torch.float32)
    engine.synchronize()
    kq, ks2 = engine.nikhilam_compress(K)
    vq, vs2 = engine.nikhilam_compress(V)
    want = engine.attention(Q, K, V, p, out_dtype=torch.float32)
    engine.synchronize()
    assert torch.equal(kc[:, :, :S], kq) and torch.equal(vc[:, :, :S], vq)
    assert int(kc[:, :, S:].abs().sum()) == 0 and int(vc[:, :, S:].abs().sum()) == 0
    assert torch.equal(ks, ks2) and torch.equal(vs, vs2)
    assert torch.equal(out, want)
    # the cache bytes against the oracle as well, for one head
    q_o, s_o = O.nikhilam_compress(K[1, 2].float().cpu().numpy())
    assert np.array_equal(kc[1, 2, :S].cpu().numpy(), q_o) and np.float32(ks[1, 2].item()) == s_o
    # caches and scales travel together
    rc = engine.lib.logos_prefill_fwd(engine.h, L.BF16, L.F32, Q.data_ptr(), K.data_ptr(), V.data_ptr(), out.data_ptr(),
                                      B, H, S, DH, __import__("ctypes").byref(p), kc.data_ptr(), None, ks.data_ptr(),
                                      vs.data_ptr(), S_max)
    assert rc == L.ERR_INVALID_ARG
