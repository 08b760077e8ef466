"""Model-level parity on the GPU: the whole multi-head forward of the reference's CPU model
(configuration 1 of the benchmark list, at a reduced and at the full size), a generation loop
(prefill into the INT8 cache, then append + decode steps), and the kernel time-out channel."""
import ctypes as C

import numpy as np
import pytest
import torch

import oracle as O
from logos_b200 import lib as L
from logos_b200 import synthetic as syn
from logos_b200.attention import MultiHeadAttention
from helpers import assert_close

pytestmark = pytest.mark.gpu


def mha_case(engine, seq, d_model, H, alpha, sparse, seed):
    dk = d_model // H
    X = syn.normal((seq, d_model), seed, 1)
    W = {k: syn.normal(shape, seed, t, std=0.02) for t, (k, shape) in enumerate(
        dict(WQ=(H, d_model, dk), WK=(H, d_model, dk), WV=(H, d_model, dk), WO=(H, dk, d_model),
             Wp=(d_model, d_model)).items(), start=2)}
    cfg = O.HeadCfg(int(sparse), 8, 4, 1, alpha, 0.1, 0.05, 1, O.lib().lo_max_threads())
    want = np.empty((seq, d_model), np.float32)
    O.lib().lo_mha_forward(X, W["WQ"], W["WK"], W["WV"], W["WO"], W["Wp"], seq, d_model, H, C.byref(cfg), want)
    dev = lambda a: torch.from_numpy(a).cuda()
    mha = MultiHeadAttention(engine, dev(W["WQ"]), dev(W["WK"]), dev(W["WV"]), dev(W["WO"]), dev(W["Wp"]),
                             use_sparse=sparse, sparse_window=8, sparse_stride=4, use_navier_stokes=True,
                             ns_alpha=alpha, ns_eta=0.1, ns_nu=0.05, diffuse_mode=L.DIFFUSE_CENTRAL, kv_int8=True)
    torch.backends.cuda.matmul.allow_tf32 = False
    got = mha.forward(dev(X)).cpu().numpy()
    assert_close(got, want, f"MHA seq={seq} d={d_model} alpha={alpha} sparse={sparse}")


def test_mha_forward_small(engine):
    for alpha, sparse in [(1.0, False), (0.3, False), (0.3, True)]:
        mha_case(engine, 96, 128, 4, alpha, sparse, 81)


def test_mha_forward_configuration_1(engine):
    # B=1, seq=512, d_model=1024, H=16, DH=64, fp32; X ~ N(0,1), weights ~ N(0,0.02); causal full
    # attention with Q-advection 0.1 and (central) V-diffusion 0.05; K/V through the INT8 round trip
    mha_case(engine, 512, 1024, 16, 1.0, False, 82)


def test_generation_loop_prefill_then_decode(engine):
    """Prefill S0 tokens, fill the INT8 cache, then 6 steps of append + decode; every step is
    compared with the oracle's decode over the oracle-quantized cache, and the cache bytes with
    the oracle's quantization of the appended rows."""
    B, H, S0, S_max, DH, steps = 2, 3, 70, 128, 64, 6
    k = syn.normal_with_outliers((B, H, S0, DH), 83, 1)
    v = syn.normal_with_outliers((B, H, S0, DH), 83, 2)
    kc = torch.zeros((B, H, S_max, DH), dtype=torch.int8, device="cuda")
    vc = torch.zeros_like(kc)
    _, ks = engine.nikhilam_compress(torch.from_numpy(k).cuda(), cache=kc)
    _, vs = engine.nikhilam_compress(torch.from_numpy(v).cuda(), cache=vc)
    kc_o, vc_o = kc.cpu().numpy().copy(), vc.cpu().numpy().copy()
    ks_o, vs_o = ks.cpu().numpy(), vs.cpu().numpy()
    engine.reserve(engine.decode_workspace_bytes(B, H, S_max, DH))
    q_prev = syn.normal((B, H, DH), 83, 3).astype(np.float16)
    n = B * H
    for (w, s_, mode) in [(0, 0, L.DIFFUSE_CAUSAL), (64, 16, L.DIFFUSE_CAUSAL)]:
        p = L.Params.make(0.125, True, w, s_, 0.1, 0.05, 1.0, mode)
        op = O.attn_params(0.125, True, w, s_, 0.1, 0.05, 1.0, mode)
        kc_t, vc_t = kc.clone(), vc.clone()
        kco, vco = kc_o.copy(), vc_o.copy()
        qp = q_prev
        for step in range(steps):
            pos = S0 + step
            q = syn.normal((B, H, DH), 83, 10 + step).astype(np.float16)
            kn = syn.normal((B, H, DH), 83, 30 + step).astype(np.float16)
            vn = syn.normal((B, H, DH), 83, 50 + step).astype(np.float16)
            dev = lambda a: torch.from_numpy(a).cuda()
            engine.kv_append(dev(kn), dev(vn), kc_t, vc_t, ks, vs, torch.full((B,), pos, dtype=torch.int32, device="cuda"))
            lens = torch.full((B,), pos + 1, dtype=torch.int32, device="cuda")
            out = engine.decode_int8(dev(q), dev(qp), kc_t, vc_t, ks, vs, lens, p).cpu().numpy()
            for b in range(B):
                for h in range(H):
                    kco[b, h, pos] = O.nikhilam_quantize(kn[b, h].astype(np.float32), ks_o[b, h])
                    vco[b, h, pos] = O.nikhilam_quantize(vn[b, h].astype(np.float32), vs_o[b, h])
            assert np.array_equal(kc_t.cpu().numpy(), kco) and np.array_equal(vc_t.cpu().numpy(), vco)
            want = O.decode_int8_batch(q.astype(np.float32).reshape(n, DH), qp.astype(np.float32).reshape(n, DH),
                                       kco.reshape(n, S_max, DH), vco.reshape(n, S_max, DH), ks_o.reshape(n),
                                       vs_o.reshape(n), np.full(n, pos + 1, np.int32), op).reshape(B, H, DH)
            assert_close(out, want, f"step {step} window={w}", 2e-5, 1e-5)
            qp = q


def test_bounded_wait_reports_instead_of_hanging(engine):
    """Mode 2 of the bring-up kernel never issues its tile load, so its wait on the load barrier
    runs out: the kernel returns, the context stays usable and the status channel reports it."""
    A = torch.zeros((128, 64), dtype=torch.bfloat16, device="cuda")
    D = torch.zeros((128, 128), device="cuda")
    rc = engine.lib.logos_selftest_umma(engine.h, 2, L.BF16, A.data_ptr(), A.data_ptr(), D.data_ptr())
    assert rc == L.OK
    with pytest.raises(L.LogosError) as e:
        engine.synchronize()
    assert e.value.status == L.ERR_KERNEL_TIMEOUT
    engine.synchronize()                       # the flag is cleared, the context still works
    x = torch.ones((1, 1, 16, 64), device="cuda")
    out = engine.attention(x, x, x, L.Params.make(0.125))
    assert torch.allclose(out, x)
