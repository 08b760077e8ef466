"""The CPU oracle against the reference: golden vectors produced by the reference's own
headers, the properties its unit tests assert, and (where oracle/_ref is present) the
reference code itself, live."""
import ctypes as C

import numpy as np
import pytest

import oracle as O

L = O.lib()


def causal(seq):
    m = np.empty((seq, seq), np.float32)
    L.lo_causal_mask(m, seq)
    return m


def ns(Q, K, V, mask, T, eta, nu):
    o = np.empty((Q.shape[0], V.shape[1]), np.float32)
    L.lo_ns_attention(Q, K, V, mask, T, eta, nu, o, Q.shape[0], Q.shape[1], V.shape[1])
    return o


# ---- golden vectors from the reference -------------------------------------------------

def test_m12_golden(golden):
    Q, K, V = golden["m12_Q"], golden["m12_K"], golden["m12_V"]
    assert np.array_equal(ns(Q, K, V, causal(8), 4.0, 0.2, 0.1), golden["m12_ns"])
    assert np.array_equal(ns(Q, K, V, causal(8), 4.0, 1.0, 0.1), golden["m12_ns_eta1"])
    # and the fp64 general routine within fp32 rounding
    p = O.attn_params(0.25, True, 0, 0, 0.2, 0.1, 1.0, O.DIFFUSE_CENTRAL)
    assert np.abs(O.attention_rows(Q, K, V, p) - golden["m12_ns"]).max() < 1e-6


def test_m20_golden(golden):
    Q, K, V = golden["m20_Q"], golden["m20_K"], golden["m20_V"]
    T = np.sqrt(np.float32(2))
    assert np.array_equal(ns(Q, K, V, causal(2), T, 1.0, 0.0), golden["m20_ns"])
    assert np.array_equal(ns(Q, K, V, causal(2), T, 0.0, 0.0), golden["m20_std"])
    # the property M20 asserts: advection changes the output
    assert np.abs(golden["m20_ns"] - golden["m20_std"]).sum() > 1e-5
    Q, K, V = golden["m20d_Q"], golden["m20d_K"], golden["m20d_V"]
    assert np.array_equal(ns(Q, K, V, causal(3), 1.0, 0.0, 1.0), golden["m20d_nu1"])
    assert np.array_equal(ns(Q, K, V, causal(3), 1.0, 0.0, 0.0), golden["m20d_nu0"])


def test_full_attention_golden(golden):
    Q, K, V = golden["full_Q"], golden["full_K"], golden["full_V"]
    for n, (sp, w, s, use_ns, al) in enumerate(golden["full_cases"]):
        p = O.attn_params(0.25, True, int(w) if sp else 0, int(s), 0.1 if use_ns else 0.0, 0.05,
                          float(al) if use_ns else 0.0, O.DIFFUSE_CENTRAL if use_ns else O.DIFFUSE_NONE)
        got = O.attention_rows(Q, K, V, p)
        assert np.abs(got - golden[f"full_out{n}"]).max() < 2e-6, n


def test_shunyam_masks_golden(golden):
    for key in golden.files:
        if not key.startswith("mask_"):
            continue
        seq, w, s = (int(x) for x in key.split("_")[1:])
        m = np.empty((seq, seq), np.float32)
        L.lo_shunyam_mask(m, seq, w, s)
        assert np.array_equal((m == 0).astype(np.uint8), golden[key])
        # the index predicate used by the kernels opens the same set whenever the rule is on
        if seq > w:
            p = O.attn_params(1.0, True, w, s)
            al = np.array([[L.lo_allowed(i, j, seq, C.byref(p)) for j in range(seq)] for i in range(seq)])
            assert np.array_equal(al.astype(np.uint8), golden[key])


def test_mha_golden(golden):
    X = golden["mha_X"]
    seq, d_model = X.shape
    H = golden["mha_WQ"].shape[0]
    cfg = O.HeadCfg(1, 8, 4, 1, 0.3, 0.1, 0.05, 0, 1)
    out = np.empty((seq, d_model), np.float32)
    L.lo_mha_forward(X, golden["mha_WQ"], golden["mha_WK"], golden["mha_WV"], golden["mha_WO"],
                     golden["mha_Wp"], seq, d_model, H, C.byref(cfg), out)
    assert np.array_equal(out, golden["mha_out"])
    cfg.threads = 4
    out2 = np.empty_like(out)
    L.lo_mha_forward(X, golden["mha_WQ"], golden["mha_WK"], golden["mha_WV"], golden["mha_WO"],
                     golden["mha_Wp"], seq, d_model, H, C.byref(cfg), out2)
    assert np.array_equal(out, out2)


# ---- properties the reference's tests assert --------------------------------------------

def test_softmax_properties_m5_m20():
    # tests/test_math_unit.cpp:2190-2250: rows sum to 1, extremes stay finite, T flattens
    s = np.array([[-10, -5, 0, 5], [10, 1, 0, -5], [0, 0, 0, 0]], np.float32)
    p = np.empty_like(s)
    L.lo_boltzmann_softmax(s, p, 3, 4, 1.0)
    assert p[0, 3] > 0.9 and p[1, 0] > p[1, 1]
    assert np.allclose(p.sum(1), 1.0, atol=1e-4)
    s = np.array([[1000, 999, 0], [-1000, 1000, 1000]], np.float32)
    p = np.empty_like(s)
    L.lo_boltzmann_softmax(s, p, 2, 3, 1.0)
    assert np.isfinite(p).all() and p[0, 0] > p[0, 1]
    s = np.array([[4, 0, 0, 0]], np.float32)
    p1, p2 = np.empty_like(s), np.empty_like(s)
    L.lo_boltzmann_softmax(s, p1, 1, 4, 1.0)
    L.lo_boltzmann_softmax(s, p2, 1, 4, 2.0)
    assert p2[0, 0] < p1[0, 0]
    s = np.array([[0, -1e30, -1e30, -1e30, -1e30]], np.float32)
    p = np.empty_like(s)
    L.lo_boltzmann_softmax(s, p, 1, 5, 1.0)
    assert np.isfinite(p).all() and p[0, 0] > 0.99 and abs(p.sum() - 1) < 1e-3


def test_ns_nu0_equals_standard_m27():
    rng = np.random.default_rng(7)
    Q, K, V = (rng.uniform(-0.5, 0.5, (8, 16)).astype(np.float32) for _ in range(3))
    a = ns(Q, K, V, causal(8), 4.0, 0.0, 0.0)
    b = np.empty_like(a)
    L.lo_std_attention(Q, K, V, causal(8), 4.0, b, 8, 16, 16)
    assert np.abs(a - b).max() < 1e-3
    assert np.abs(a).max() <= np.abs(V).max() + 1e-5  # outputs are convex combinations of V


def test_diffusion_formula_m12f():
    V = np.array([[2.0], [4.0], [6.0]], np.float32)
    Vs = np.empty_like(V)
    L.lo_ns_diffuse_central(V, Vs, 3, 1, 0.1)
    assert abs(Vs[1, 0] - 4.0) < 1e-5
    L.lo_ns_diffuse_central(V, Vs, 3, 1, 1.0)
    assert abs(Vs[1, 0] - 4.0) < 1e-5
    L.lo_ns_diffuse_central(V, Vs, 3, 1, 0.0)
    assert np.array_equal(Vs, V)


def test_ns_kernels_adjoint_k7_k8():
    # tests/test_cuda_kernels.cu:437-535 checks <A x, y> == <x, A^T y>; here with explicit A
    seq, d = 16, 32
    i = np.arange(seq * d, dtype=np.float32).reshape(seq, d)
    Q = np.sin(0.1 * i).astype(np.float32)
    Qa = np.empty_like(Q)
    L.lo_ns_advect(Q, Qa, seq, d, 0.1)
    A = np.eye(seq) * 1.1 - np.eye(seq, k=-1) * 0.1
    A[0, 0] = 1.0
    assert np.abs(Qa - (A @ Q.astype(np.float64))).max() < 1e-6
    Vs = np.empty_like(Q)
    L.lo_ns_diffuse_causal(Q, Vs, seq, d, 0.05)
    D = np.eye(seq) * 0.95 + np.eye(seq, k=-1) * 0.05
    D[0, 0] = 1.0
    assert np.abs(Vs - (D @ Q.astype(np.float64))).max() < 1e-6


# ---- Nikhilam INT8: fixtures of the reference's tests ------------------------------------

def test_nikhilam_s13_roundtrip():
    # tests/test_syntax_build.cu:487-540: 32x64 ramp 5.0 .. 9.84, abs err < 0.1, rel < 1 %
    x = (5.0 + np.arange(32 * 64, dtype=np.float32) * (4.84 / (32 * 64 - 1))).astype(np.float32)
    q, s = O.nikhilam_compress(x)
    xd = O.nikhilam_dequantize(q, s)
    assert np.abs(xd - x).max() < 0.1
    assert (np.abs(xd - x) / np.abs(x)).max() < 0.01
    assert s == np.float32((np.float32(x.max()) + np.float32(1e-8)) / np.float32(127.5))


def test_nikhilam_m5_snr():
    # tests/test_math_units.cu:377-446: 4096-sample sine, amplitude 7.5, SNR >= 40 dB
    x = (7.5 * np.sin(np.arange(4096) * 0.01)).astype(np.float32)
    q, s = O.nikhilam_compress(x)
    xd = O.nikhilam_dequantize(q, s)
    snr = 10 * np.log10((x.astype(np.float64) ** 2).sum() / ((x - xd).astype(np.float64) ** 2).sum())
    assert snr >= 40.0
    assert abs(L.lo_absmax(x, x.size) - 7.5) < 0.01


def test_nikhilam_mem3_and_identities():
    # tests/test_memory_stress.cu:177-243: (i % 201) - 100 over 1 M values, error < 1.0
    x = ((np.arange(1 << 20) % 201) - 100).astype(np.float32)
    q, s = O.nikhilam_compress(x)
    assert np.abs(O.nikhilam_dequantize(q, s) - x).max() < 1.0
    assert q.min() >= -127 and q.max() <= 127
    # zero tensor: scale is the epsilon floor, bytes are zero
    q0, s0 = O.nikhilam_compress(np.zeros(64, np.float32))
    assert s0 == np.float32(np.float32(1e-8) / np.float32(127.5)) and not q0.any()
    # round-half-even, not half-away (tests/test_math_unit.cpp:697 uses std::round; production does not)
    scale = np.float32(1.0) - np.float32(1e-8)
    assert list(O.nikhilam_quantize(np.array([0.5, 1.5, 2.5, -0.5, -1.5], np.float32), scale)) == [0, 2, 2, 0, -2]
    # saturation of values beyond the scale's range (the append contract)
    assert list(O.nikhilam_quantize(np.array([1e6, -1e6], np.float32), 1.0)) == [127, -127]


# ---- live comparison with the reference when it is built ---------------------------------

@pytest.mark.skipif(O.ref() is None, reason="oracle/_ref not built (no reference tree)")
def test_live_reference_agreement():
    R = O.ref()
    rng = np.random.default_rng(11)
    for seq, dk in [(5, 2), (17, 3), (64, 16), (130, 64)]:
        Q, K, V = (rng.standard_normal((seq, dk)).astype(np.float32) for _ in range(3))
        a = ns(Q, K, V, causal(seq), np.sqrt(np.float32(dk)), 0.1, 0.05)
        b = np.empty_like(a)
        R.ref_ns_attention(Q, K, V, causal(seq), np.sqrt(np.float32(dk)), 0.1, 0.05, b, seq, dk, dk)
        assert np.array_equal(a, b)
        for (sp, w, s, use_ns, al) in [(1, 8, 4, 1, 0.3), (1, 32, 8, 1, 1.0), (0, 8, 4, 0, 0.0)]:
            R.ref_attention_full(Q, K, V, seq, dk, sp, w, s, use_ns, al, 0.1, 0.05, b)
            p = O.attn_params(1 / np.sqrt(dk), True, w if sp else 0, s, 0.1 if use_ns else 0, 0.05,
                              al if use_ns else 0.0, O.DIFFUSE_CENTRAL if use_ns else 0)
            assert np.abs(O.attention_rows(Q, K, V, p) - b).max() < 5e-6


def test_decode_composition_matches_last_row():
    """lo_decode_int8 == last row of the full attention over dequantized K/V."""
    rng = np.random.default_rng(5)
    for mode in (O.DIFFUSE_NONE, O.DIFFUSE_CAUSAL, O.DIFFUSE_CENTRAL):
        for (w, s, al) in [(0, 0, 1.0), (8, 4, 1.0), (8, 4, 0.3)]:
            n, d = 37, 64
            Q = rng.standard_normal((n, d)).astype(np.float32)
            Kq, ks = O.nikhilam_compress(rng.standard_normal((n, d)).astype(np.float32))
            Vq, vs = O.nikhilam_compress(rng.standard_normal((n, d)).astype(np.float32))
            p = O.attn_params(0.125, True, w, s, 0.1, 0.05, al, mode)
            full = O.attention_rows(Q, O.nikhilam_dequantize(Kq, ks), O.nikhilam_dequantize(Vq, vs), p)
            got = O.decode_int8_batch(Q[-1:], Q[-2:-1], Kq[None], Vq[None], [ks], [vs], [n], p)
            assert np.abs(got[0] - full[-1]).max() < 1e-6


def test_backward_oracle_is_the_gradient_of_the_forward_oracle():
    """lo_attention_bwd_f64 pinned by central differences of the (reference-pinned) forward oracle: every
    diffusion stencil, the blend, the Shunyam mask with and without landmarks, and no causal mask."""
    rng = np.random.default_rng(7)
    S, d = 20, 8
    cases = [(0, 0, 0.0, 0.0, 1.0, 0, True), (0, 0, 0.1, 0.05, 1.0, 1, True), (0, 0, 0.1, 0.05, 1.0, 2, True),
             (6, 4, 0.1, 0.05, 0.3, 1, True), (6, 0, 0.2, 0.1, 0.6, 2, True), (0, 0, 0.1, 0.05, 1.0, 1, False)]
    for (w, st, eta, nu, alpha, mode, causal) in cases:
        p = O.attn_params(0.35, causal, w, st, eta, nu, alpha, mode)
        Q, K, V, dO = (rng.standard_normal((1, 1, S, d)).astype(np.float32) for _ in range(4))
        dQ, dK, dV = O.attention_bwd(Q, K, V, dO, p)
        f = lambda: float((O.attention_batched(Q, K, V, p).astype(np.float64) * dO).sum())
        for X, G in ((Q, dQ), (K, dK), (V, dV)):
            for _ in range(8):
                i = tuple(int(rng.integers(0, n)) for n in X.shape)
                old, h = X[i], 1e-2
                X[i] = old + h; fp = f()
                X[i] = old - h; fm = f()
                X[i] = old
                num = (fp - fm) / (2 * h)
                assert abs(num - G[i]) <= 2e-3 * (abs(num) + 1e-2), (w, st, mode, alpha, i, num, G[i])
