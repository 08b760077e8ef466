"""Attention backward (logos_attention_bwd) against the fp64 backward oracle for every switch, against the
reference's own backward kernels run on this GPU (causal mask, the GPU model's stencils), and the
reproducibility of its fixed-order sums."""
import ctypes as C
import os

import numpy as np
import pytest
import torch

import oracle as O
from logos_b200 import lib as L
from logos_b200 import synthetic as syn

pytestmark = pytest.mark.gpu


def _case(B, H, S, DH, seed):
    return [syn.normal((B, H, S, DH), seed, t) for t in range(1, 5)]


def _check(engine, B, H, S, DH, scale, causal, window, stride, eta, nu, alpha, mode, seed, tol=2e-5):
    Q, K, V, dO = _case(B, H, S, DH, seed)
    p = L.Params.make(scale, causal, window, stride, eta, nu, alpha, mode)
    op = O.attn_params(scale, causal, window, stride, eta, nu, alpha, mode)
    want = O.attention_bwd(Q, K, V, dO, op)
    dev = lambda a: torch.from_numpy(a).cuda()
    got = engine.attention_bwd(dev(Q), dev(K), dev(V), dev(dO), p)
    engine.synchronize()
    for name, g, w in zip(("dQ", "dK", "dV"), got, want):
        g = g.cpu().numpy()
        assert np.isfinite(g).all(), name
        err = np.abs(g - w).max()
        ref = np.abs(w).max()
        assert err <= tol * max(ref, 1.0), f"{name}: max-abs {err:.3e} against magnitude {ref:.3e}"


@pytest.mark.parametrize("DH", [32, 64, 128])
def test_bwd_causal_plain(engine, DH):
    _check(engine, 2, 2, 150, DH, 1.0 / np.sqrt(DH), True, 0, 0, 0.0, 0.0, 1.0, L.DIFFUSE_NONE, 300 + DH)


@pytest.mark.parametrize("mode", [L.DIFFUSE_NONE, L.DIFFUSE_CAUSAL, L.DIFFUSE_CENTRAL])
@pytest.mark.parametrize("alpha", [1.0, 0.3])
def test_bwd_navier_stokes_and_blend(engine, mode, alpha):
    _check(engine, 1, 3, 200, 64, 0.125, True, 0, 0, 0.1, 0.05, alpha, mode, 310 + mode)


@pytest.mark.parametrize("window,stride", [(8, 4), (64, 16), (64, 0), (16, 100), (300, 16)])
def test_bwd_honours_the_shunyam_mask(engine, window, stride):
    # 300 >= S: the rule is off (seq <= window) and the mask is plain causal
    _check(engine, 1, 2, 260, 64, 0.125, True, window, stride, 0.1, 0.05, 1.0, L.DIFFUSE_CAUSAL, 320 + window)


def test_bwd_not_causal_and_ragged_sizes(engine):
    _check(engine, 1, 2, 97, 64, 0.125, False, 0, 0, 0.1, 0.05, 1.0, L.DIFFUSE_CAUSAL, 330)
    for S in (1, 2, 63, 64, 65, 129):
        _check(engine, 1, 1, S, 64, 0.125, True, 0, 0, 0.1, 0.05, 0.5, L.DIFFUSE_CENTRAL, 331 + S)


def test_bwd_is_reproducible_bit_for_bit(engine):
    Q, K, V, dO = (torch.from_numpy(a).cuda() for a in _case(2, 4, 512, 64, 340))
    p = L.Params.make(0.125, True, 64, 16, 0.1, 0.05, 1.0, L.DIFFUSE_CAUSAL)
    a = [t.clone() for t in engine.attention_bwd(Q, K, V, dO, p)]
    b = engine.attention_bwd(Q, K, V, dO, p)
    engine.synchronize()
    for x, y in zip(a, b):
        assert torch.equal(x, y)


def test_bwd_leaves_the_decode_counters_alone(engine):
    """Backward and decode share the context's workspace: a split-K decode right after a backward must still find
    its arrival counters at zero."""
    Q, K, V, dO = (torch.from_numpy(a).cuda() for a in _case(1, 2, 256, 64, 345))
    engine.attention_bwd(Q, K, V, dO, L.Params.make(0.125, True, 0, 0, 0.1, 0.05, 1.0, L.DIFFUSE_CAUSAL))
    from test_decode_gpu import run_case
    run_case(engine, 2, 2, 4096, [4096, 1500], L.Params.make(0.125, True, 0, 0, 0.1, 0.05, 1.0, L.DIFFUSE_CAUSAL), seed=346)


def test_bwd_matches_autograd_of_the_forward_at_length(engine):
    """S = 1024, 8 heads: torch autograd through an fp64 restatement of the forward (advection, causal
    diffusion, masked softmax) as a third, independent witness at a size the C oracle takes long for."""
    B, H, S, DH = 1, 8, 1024, 64
    Q, K, V, dO = (torch.from_numpy(a).cuda() for a in _case(B, H, S, DH, 350))
    eta, nu, scale = 0.1, 0.05, 0.125
    p = L.Params.make(scale, True, 0, 0, eta, nu, 1.0, L.DIFFUSE_CAUSAL)
    got = engine.attention_bwd(Q, K, V, dO, p)
    q, k, v = (t.double().requires_grad_(True) for t in (Q, K, V))
    qp = torch.cat([q[:, :, :1], q[:, :, :-1]], dim=2)
    vp = torch.cat([v[:, :, :1], v[:, :, :-1]], dim=2)
    qa, vs = q + eta * (q - qp), (1 - nu) * v + nu * vp
    s = (qa @ k.transpose(-1, -2)) * scale
    s = s.masked_fill(torch.ones(S, S, dtype=torch.bool, device="cuda").triu(1), float("-inf"))
    out = torch.softmax(s, dim=-1) @ vs
    out.backward(dO.double())
    for name, g, w in zip(("dQ", "dK", "dV"), got, (q.grad, k.grad, v.grad)):
        err = float((g.double() - w).abs().max())
        assert err <= 2e-5 * max(float(w.abs().max()), 1.0), (name, err)


@pytest.mark.parametrize("S,all_rows", [(64, 0), (48, 1), (192, 1), (100, 1)])
def test_bwd_against_the_reference_kernels(engine, S, all_rows):
    """The reference's own backward chain (cuda/train_gpu.cu:657-748 through oracle/_ref/liblogos_refbwd.so)
    on one head: causal mask, Q_adv and V_s as its forward caches them.  The oracle and the engine must both
    agree with it: the oracle is pinned by it, the engine replaces it.  As launched by the reference the chain
    transposes all of K only when seq = DH (see oracle/ref_bwd_harness.cu), so it is taken as it is at
    seq = 64 and with the transpose launched over every row and column at the other lengths."""
    path = os.path.join(os.path.dirname(O.__file__), "_ref", "liblogos_refbwd.so")
    if not os.path.exists(path):
        pytest.skip("oracle/_ref/liblogos_refbwd.so was not built (needs the reference tree)")
    ref = C.CDLL(path)
    DH, eta, nu = 64, 0.1, 0.05
    Q, K, V, dO = _case(1, 1, S, DH, 360 + S)
    dev = lambda a: torch.from_numpy(a).cuda()
    Qd, Kd, Vd, dOd = dev(Q[0, 0]), dev(K[0, 0]), dev(V[0, 0]), dev(dO[0, 0])
    Qa = (Qd + eta * (Qd - torch.cat([Qd[:1], Qd[:-1]]))).contiguous()
    Vs = ((1.0 - nu) * Vd + nu * torch.cat([Vd[:1], Vd[:-1]])).contiguous()
    dQ, dK, dV = (torch.empty_like(Qd) for _ in range(3))
    scratch = torch.empty(3 * S * S + 3 * S * DH, dtype=torch.float32, device="cuda")
    vp = lambda t: C.c_void_p(t.data_ptr())
    ref.refbwd_attention_head.argtypes = [C.c_void_p] * 7 + [C.c_int, C.c_int, C.c_float, C.c_float, C.c_void_p, C.c_int]
    torch.cuda.synchronize()
    rc = ref.refbwd_attention_head(vp(Qa), vp(Kd), vp(Vs), vp(dOd), vp(dQ), vp(dK), vp(dV), S, DH, eta, nu,
                                   vp(scratch), all_rows)
    torch.cuda.synchronize()
    assert rc == 0
    p = L.Params.make(0.125, True, 0, 0, eta, nu, 1.0, L.DIFFUSE_CAUSAL)
    op = O.attn_params(0.125, True, 0, 0, eta, nu, 1.0, L.DIFFUSE_CAUSAL)
    want = O.attention_bwd(Q, K, V, dO, op)
    got = engine.attention_bwd(dev(Q), dev(K), dev(V), dev(dO), p)
    engine.synchronize()
    for name, r, w, g in zip(("dQ", "dK", "dV"), (dQ, dK, dV), want, got):
        r = r.cpu().numpy()
        mag = max(float(np.abs(r).max()), 1.0)
        assert np.abs(w[0, 0] - r).max() <= 2e-5 * mag, f"oracle vs reference kernels, {name}"
        assert np.abs(g[0, 0].cpu().numpy() - r).max() <= 2e-5 * mag, f"engine vs reference kernels, {name}"
