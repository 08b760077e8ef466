"""logos_attention_fwd_strided: tensors that are not packed [B][H][S][DH] (token-major, padded rows, one head of a
larger tensor) give the same bits as the packed call on the same values, on the tensor-core kernels and on the
fp32 kernel, and agree with the oracle."""
import numpy as np
import pytest
import torch

import oracle as O
from logos_b200 import lib as L
from logos_b200 import synthetic as syn
from helpers import assert_close

pytestmark = pytest.mark.gpu


def _token_major(x):
    """[B, H, S, D] values stored as [B, S, H, D]; returned as a [B, H, S, D] view of that storage."""
    return x.permute(0, 2, 1, 3).contiguous().permute(0, 2, 1, 3)


def _padded(x, pad):
    """Rows of D values stored with a pitch of D + pad."""
    B, H, S, D = x.shape
    buf = torch.zeros((B, H, S, D + pad), dtype=x.dtype, device=x.device)
    buf[..., :D] = x
    return buf[..., :D]


CASES = [
    (L.Params.make(0.125, True, 0, 0, 0.1, 0.05, 1.0, L.DIFFUSE_CAUSAL), "causal, tensor cores"),
    (L.Params.make(0.125, True, 64, 16, 0.1, 0.05, 1.0, L.DIFFUSE_CAUSAL), "window + landmarks, tensor cores"),
    (L.Params.make(0.125, True, 64, 0, 0.1, 0.05, 1.0, L.DIFFUSE_NONE), "pure window, tensor cores"),
    (L.Params.make(0.125, True, 0, 0, 0.1, 0.05, 0.3, L.DIFFUSE_CENTRAL), "blend, fp32 kernel"),
]


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("B", [1, 3])
def test_strided_equals_packed(engine, dtype, B):
    H, S, D = 4, 700, 64
    g = torch.Generator(device="cuda").manual_seed(B + 11)
    Q, K, V = (torch.randn((B, H, S, D), device="cuda", generator=g).to(dtype) for _ in range(3))
    for p, what in CASES:
        want = engine.attention(Q, K, V, p)
        # token-major inputs and output (for B > 1 the slabs are not evenly spaced: one launch per sequence)
        out_tm = _token_major(torch.zeros_like(want))
        got = engine.attention_strided(_token_major(Q), _token_major(K), _token_major(V), p, out=out_tm)
        engine.synchronize()
        assert torch.equal(got, want), f"token-major, {what}"
        # padded rows in, packed fp32 out
        got = engine.attention_strided(_padded(Q, 8), _padded(K, 8), _padded(V, 8), p, out_dtype=torch.float32)
        want32 = engine.attention(Q, K, V, p, out_dtype=torch.float32)
        engine.synchronize()
        assert torch.equal(got, want32), f"padded rows, {what}"
        # two heads out of the middle of the packed tensor, written into the same place of a packed output
        full = torch.zeros_like(want)
        engine.attention_strided(Q[:, 1:3], K[:, 1:3], V[:, 1:3], p, out=full[:, 1:3])
        engine.synchronize()
        assert torch.equal(full[:, 1:3], want[:, 1:3]) and not bool(full[:, 0].any()) and not bool(full[:, 3].any()), what


def test_strided_against_the_oracle(engine):
    B, H, S, D = 2, 3, 333, 64
    q, k, v = (syn.normal((B, H, S, D), 500, t) for t in (1, 2, 3))
    p = L.Params.make(0.125, True, 64, 16, 0.1, 0.05, 1.0, L.DIFFUSE_CAUSAL)
    dev = lambda a: torch.from_numpy(a).cuda().bfloat16()
    Q, K, V = dev(q), dev(k), dev(v)
    got = engine.attention_strided(_token_major(Q), _token_major(K), _token_major(V), p, out_dtype=torch.float32)
    want = O.attention_batched(Q.float().cpu().numpy(), K.float().cpu().numpy(), V.float().cpu().numpy(),
                               O.attn_params(0.125, True, 64, 16, 0.1, 0.05, 1.0, L.DIFFUSE_CAUSAL))
    assert_close(got.cpu().numpy(), want, "token-major window + landmarks")


def test_strided_argument_checks(engine):
    B, H, S, D = 1, 2, 128, 64
    Q = torch.zeros((B, H, S, D), dtype=torch.bfloat16, device="cuda")
    p = L.Params.make(0.125, True, 0, 0, 0.0, 0.0, 1.0, L.DIFFUSE_NONE)
    bad = L.Strides(H * S * D, S * D, 32)                       # rows overlap
    import ctypes as C
    from logos_b200.engine import _ptr
    rc = engine.lib.logos_attention_fwd_strided(engine.h, L.BF16, L.BF16, _ptr(Q), _ptr(Q), _ptr(Q), _ptr(Q), B, H, S, D,
                                                C.byref(bad), None, C.byref(p))
    assert rc == L.ERR_INVALID_ARG
    odd = L.Strides(H * S * (D + 4), S * (D + 4), D + 4)        # 16-bit rows not 16-byte aligned: the tensor-core path refuses
    buf = torch.zeros((B, H, S, D + 4), dtype=torch.bfloat16, device="cuda")
    rc = engine.lib.logos_attention_fwd_strided(engine.h, L.BF16, L.BF16, _ptr(buf), _ptr(buf), _ptr(buf), _ptr(Q), B, H, S, D,
                                                C.byref(odd), None, C.byref(p))
    assert rc == L.ERR_ALIGNMENT
