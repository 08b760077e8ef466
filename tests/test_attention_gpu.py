"""Prefill / window attention on the GPU against the reference: the golden vectors made by
the reference's own CPU code, the CPU oracle on seeded inputs, and the reference's CUDA
kernel run live on the same GPU."""
import numpy as np
import pytest
import torch

import oracle as O
from logos_b200 import lib as L
from logos_b200 import synthetic as syn
from helpers import assert_close

pytestmark = pytest.mark.gpu


def dev(a, dtype=torch.float32):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda().to(dtype)


def oracle_params(p):
    return O.attn_params(p.scale, p.causal, p.window, p.stride, p.ns_eta, p.ns_nu, p.ns_alpha, p.diffuse_mode)


# ---- golden vectors produced by the reference's CPU path --------------------------------

def test_golden_full_cases(engine, golden):
    Q, K, V = (golden[k] for k in ("full_Q", "full_K", "full_V"))
    for n, (sp, w, s, use_ns, al) in enumerate(golden["full_cases"]):
        p = L.Params.make(0.25, True, int(w) if sp else 0, int(s), 0.1 if use_ns else 0.0, 0.05,
                          float(al) if use_ns else 0.0, L.DIFFUSE_CENTRAL if use_ns else L.DIFFUSE_NONE)
        out = engine.attention(dev(Q)[None, None], dev(K)[None, None], dev(V)[None, None], p)
        assert_close(out[0, 0].cpu().numpy(), golden[f"full_out{n}"], f"golden case {n}", 1e-5, 1e-5)


def test_golden_m12_m20(engine, golden):
    p = L.Params.make(0.25, True, 0, 0, 0.2, 0.1, 1.0, L.DIFFUSE_CENTRAL)
    Q, K, V = (dev(golden[k])[None, None] for k in ("m12_Q", "m12_K", "m12_V"))
    assert_close(engine.attention(Q, K, V, p)[0, 0].cpu().numpy(), golden["m12_ns"], "M12", 1e-6, 1e-5)
    p = L.Params.make(0.25, True, 0, 0, 1.0, 0.1, 1.0, L.DIFFUSE_CENTRAL)
    assert_close(engine.attention(Q, K, V, p)[0, 0].cpu().numpy(), golden["m12_ns_eta1"], "M12 eta=1", 1e-6, 1e-5)
    Q, K, V = (dev(golden[k])[None, None] for k in ("m20_Q", "m20_K", "m20_V"))
    p = L.Params.make(float(1 / np.sqrt(np.float32(2))), True, 0, 0, 1.0, 0.0, 1.0, L.DIFFUSE_CENTRAL)
    assert_close(engine.attention(Q, K, V, p)[0, 0].cpu().numpy(), golden["m20_ns"], "M20 hand case", 1e-5, 1e-5)


# ---- the fp32 single-head entry point that stands in for cuda_flash_attention_fwd --------

@pytest.mark.parametrize("seq", [1, 15, 16, 17, 63, 64, 65, 129, 512])
@pytest.mark.parametrize("DH", [64, 128, 24])
def test_flash_fwd_f32_vs_oracle_and_reference_kernel(engine, seq, DH):
    Q, K, V = (syn.normal((seq, DH), 1, t) for t in (1, 2, 3))
    K[syn.normal((seq, DH), 1, 9) > 2.3] *= 8          # outlier channels
    scale = float(1 / np.sqrt(DH))
    R = O.refgpu()
    Qd, Kd, Vd = dev(Q), dev(K), dev(V)
    for (shun, w, s) in [(False, 0, 0), (True, 32, 8), (True, 64, 16), (True, 8, 5)]:
        active = shun and seq > w
        got = engine.flash_attention_fwd_f32(Qd, Kd, Vd, scale, True, active, w, s).cpu().numpy()
        p = O.attn_params(scale, True, w if active else 0, s, 0.0, 0.0, 0.0, O.DIFFUSE_NONE)
        assert_close(got, O.attention_rows(Q, K, V, p), f"seq={seq} DH={DH} shunyam={(shun, w, s)}", 2e-5, 1e-5)
        if R is not None:
            ref = torch.empty((seq, DH), device="cuda")
            rc = R.refgpu_flash_attention_fwd(Qd.data_ptr(), Kd.data_ptr(), Vd.data_ptr(), ref.data_ptr(), seq, DH, scale, 1, int(active), max(w, 1), max(s, 1))
            torch.cuda.synchronize()
            assert rc == 0
            assert_close(got, ref.cpu().numpy(), "vs reference CUDA kernel", 2e-5, 1e-5)


def test_flash_fwd_f32_rejections(engine):
    x = torch.zeros((8, 130), device="cuda")
    with pytest.raises(L.LogosError) as e:
        engine.flash_attention_fwd_f32(x, x, x, 0.1)         # DH > 128, as the reference (VedicGEMM.cu:1074)
    assert e.value.status == L.ERR_UNSUPPORTED
    import ctypes as C
    y = torch.zeros((8, 64), device="cuda")
    rc = engine.lib.logos_flash_attention_fwd_f32(engine.h, y.data_ptr(), y.data_ptr(), y.data_ptr(), y.data_ptr(),
                                                  y.data_ptr(), 8, 64, 0.125, 1, 0, 0, 0)
    assert rc == L.ERR_UNSUPPORTED                            # attn_ptr must be NULL


# ---- batched entry point: every switch, 16-bit and fp32 inputs ---------------------------

CASES = [
    # (window, stride, eta, nu, alpha, mode)
    (0, 0, 0.0, 0.0, 1.0, L.DIFFUSE_NONE),
    (0, 0, 0.1, 0.05, 1.0, L.DIFFUSE_CAUSAL),      # the GPU model's setting
    (0, 0, 0.1, 0.05, 1.0, L.DIFFUSE_CENTRAL),     # the CPU model's stencil, pure NS
    (0, 0, 0.1, 0.05, 0.3, L.DIFFUSE_CENTRAL),     # the CPU model's default blend
    (64, 16, 0.1, 0.05, 1.0, L.DIFFUSE_CAUSAL),    # production Shunyam
    (8, 4, 0.1, 0.05, 0.3, L.DIFFUSE_CENTRAL),     # CPU defaults (PhysicsConfig.hpp:21-22)
    (32, 0, 0.1, 0.05, 1.0, L.DIFFUSE_CAUSAL),     # pure window
]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("S", [1, 33, 64, 65, 200])
def test_batched_all_switches(engine_general, dtype, S):
    engine = engine_general
    B, H, DH = 2, 3, 64
    Q, K, V = (syn.normal((B, H, S, DH), 2, t) for t in (1, 2, 3))
    K[syn.normal((B, H, S, DH), 2, 9) > 2.3] *= 8
    Qt, Kt, Vt = dev(Q, dtype), dev(K, dtype), dev(V, dtype)
    Qr, Kr, Vr = (t.float().cpu().numpy() for t in (Qt, Kt, Vt))   # inputs as the kernel sees them
    for (w, s, eta, nu, al, mode) in CASES:
        p = L.Params.make(0.125, True, w, s, eta, nu, al, mode)
        out = engine.attention(Qt, Kt, Vt, p, out_dtype=torch.float32).cpu().numpy()
        want = O.attention_batched(Qr, Kr, Vr, oracle_params(p))
        assert_close(out, want, f"S={S} {dtype} case={(w, s, eta, nu, al, mode)}", 5e-5, 2e-5)
        if dtype != torch.float32:
            out16 = engine.attention(Qt, Kt, Vt, p)
            assert out16.dtype == dtype
            assert torch.equal(out16, torch.from_numpy(out).cuda().to(dtype)), "16-bit output is not the rounded fp32 one"


def test_non_causal(engine):
    S, DH = 70, 64
    Q, K, V = (syn.normal((1, 1, S, DH), 3, t) for t in (1, 2, 3))
    p = L.Params.make(0.125, False, 0, 0, 0.1, 0.05, 1.0, L.DIFFUSE_CENTRAL)
    out = engine.attention(dev(Q), dev(K), dev(V), p).cpu().numpy()
    assert_close(out, O.attention_batched(Q, K, V, oracle_params(p)), "non-causal", 5e-5, 2e-5)


def test_prefill_equals_decode_last_row(engine):
    """The decode kernel on a quantized cache returns the last prefill row over the same
    dequantized K/V (causal diffusion: no look-ahead, so the two must agree)."""
    B, H, S, DH = 2, 2, 300, 64
    k = syn.normal_with_outliers((B, H, S, DH), 5, 1)
    v = syn.normal_with_outliers((B, H, S, DH), 5, 2)
    q = dev(syn.normal((B, H, S, DH), 5, 3), torch.float16)
    kq, ks = engine.nikhilam_compress(dev(k))
    vq, vs = engine.nikhilam_compress(dev(v))
    kd, vd = engine.nikhilam_decompress(kq, ks), engine.nikhilam_decompress(vq, vs)
    for (w, s) in [(0, 0), (64, 16)]:
        p = L.Params.make(0.125, True, w, s, 0.1, 0.05, 1.0, L.DIFFUSE_CAUSAL)
        full = engine.attention(q.float(), kd, vd, p)
        engine.reserve(engine.decode_workspace_bytes(B, H, S, DH))
        lens = torch.full((B,), S, dtype=torch.int32, device="cuda")
        last = engine.decode_int8(q[:, :, -1].contiguous(), q[:, :, -2].contiguous(), kq, vq, ks, vs, lens, p)
        assert_close(last.cpu().numpy(), full[:, :, -1].cpu().numpy(), f"decode vs prefill {(w, s)}", 2e-5, 1e-5)
