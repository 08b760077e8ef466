"""Attention backward on the tensor cores (logos_attention_bwd16) against the fp64 backward oracle on the same
16-bit-rounded operands, every switch, and against the exact fp32 backward at length.  The weights of a tile
(probabilities and their gradients) travel between the products as 16-bit operands, so the tolerance is that of the
operand type: 4e-3 of the largest gradient in FP16, 2e-2 in BF16."""
import numpy as np
import pytest
import torch

import oracle as O
from logos_b200 import lib as L
from logos_b200 import synthetic as syn

pytestmark = pytest.mark.gpu

TOL = {torch.float16: 4e-3, torch.bfloat16: 2e-2}


def _inputs(B, H, S, seed, dtype):
    return [torch.from_numpy(syn.normal((B, H, S, 64), seed, t)).cuda().to(dtype) for t in range(1, 5)]


def _check(engine, dtype, B, H, S, causal, window, stride, eta, nu, alpha, mode, seed):
    Q, K, V, dO = _inputs(B, H, S, seed, dtype)
    p = L.Params.make(0.125, causal, window, stride, eta, nu, alpha, mode)
    op = O.attn_params(0.125, causal, window, stride, eta, nu, alpha, mode)
    want = O.attention_bwd(*(t.float().cpu().numpy() for t in (Q, K, V, dO)), op)
    got = engine.attention_bwd16(Q, K, V, dO, p)
    engine.synchronize()
    for name, g, w in zip(("dQ", "dK", "dV"), got, want):
        g = g.cpu().numpy()
        assert np.isfinite(g).all(), name
        err, mag = np.abs(g - w).max(), max(np.abs(w).max(), 1.0)
        assert err <= TOL[dtype] * mag, f"{name}: max-abs {err:.3e} against magnitude {mag:.3e}"


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("mode", [L.DIFFUSE_NONE, L.DIFFUSE_CAUSAL, L.DIFFUSE_CENTRAL])
@pytest.mark.parametrize("alpha", [1.0, 0.3])
def test_bwd16_navier_stokes_and_blend(engine, dtype, mode, alpha):
    _check(engine, dtype, 1, 2, 300, True, 0, 0, 0.1, 0.05, alpha, mode, 600 + mode)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("window,stride", [(8, 4), (64, 16), (64, 0), (16, 100), (400, 16)])
def test_bwd16_honours_the_shunyam_mask(engine, dtype, window, stride):
    _check(engine, dtype, 1, 2, 390, True, window, stride, 0.1, 0.05, 1.0, L.DIFFUSE_CAUSAL, 610 + window)


@pytest.mark.parametrize("S", [1, 2, 127, 128, 129, 257])
def test_bwd16_ragged_sizes_and_not_causal(engine, S):
    _check(engine, torch.float16, 2, 1, S, True, 0, 0, 0.1, 0.05, 1.0, L.DIFFUSE_CAUSAL, 620 + S)
    _check(engine, torch.float16, 1, 1, S, False, 0, 0, 0.0, 0.0, 1.0, L.DIFFUSE_NONE, 630 + S)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_bwd16_against_the_fp32_backward_at_length(engine, dtype):
    """S = 4096 with the production mask and S = 2048 causal: the exact fp32 kernels on the same operands."""
    for S, w, st in ((4096, 64, 16), (2048, 0, 0)):
        Q, K, V, dO = _inputs(1, 4, S, 640 + S, dtype)
        p = L.Params.make(0.125, True, w, st, 0.1, 0.05, 1.0, L.DIFFUSE_CAUSAL)
        got = [t.clone() for t in engine.attention_bwd16(Q, K, V, dO, p)]
        want = engine.attention_bwd(Q.float(), K.float(), V.float(), dO.float(), p)
        engine.synchronize()
        for name, g, w_ in zip(("dQ", "dK", "dV"), got, want):
            err, mag = float((g - w_).abs().max()), max(float(w_.abs().max()), 1.0)
            assert err <= TOL[dtype] * mag, f"S={S} {name}: {err:.3e} against {mag:.3e}"


def test_bwd16_is_reproducible_and_checks_its_arguments(engine):
    Q, K, V, dO = _inputs(2, 2, 512, 650, torch.float16)
    p = L.Params.make(0.125, True, 64, 16, 0.1, 0.05, 1.0, L.DIFFUSE_CAUSAL)
    a = [t.clone() for t in engine.attention_bwd16(Q, K, V, dO, p)]
    b = engine.attention_bwd16(Q, K, V, dO, p)
    engine.synchronize()
    for x, y in zip(a, b):
        assert torch.equal(x, y)
    with pytest.raises(L.LogosError) as e:
        engine.attention_bwd16(Q[..., :32].contiguous(), K[..., :32].contiguous(), V[..., :32].contiguous(),
                               dO[..., :32].contiguous(), p)
    assert e.value.status == L.ERR_UNSUPPORTED
