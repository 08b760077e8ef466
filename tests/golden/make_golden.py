"""Generates tests/golden/attention_golden.npz from the reference's own CPU code.

Run where the reference tree is present and oracle/_ref has been built
(`make -C oracle ref`):   python tests/golden/make_golden.py

Every output array below is produced by the unmodified LOGOS headers
(include/Attention.hpp) through oracle/_ref/liblogos_ref.so; the inputs follow the
reference's unit tests M12, M20 and M27 (tests/test_math_unit.cpp:1178-1325,
2186-2345, 3191-3304) plus seeded cases for the paths its tests never exercise
(Shunyam mask, alpha blend, multi-head forward).
"""
import ctypes as C
import os
import sys

import numpy as np

ROOT = os.path.abspath(os.path.join(os.path.dirname(__file__), "..", ".."))
sys.path.insert(0, ROOT)
import oracle as O  # noqa: E402

R = O.ref()
assert R is not None, "build oracle/_ref first"
out = {}


def causal(seq):
    m = np.empty((seq, seq), np.float32)
    R.ref_causal_mask(m, seq)
    return m


def ns(Q, K, V, mask, T, eta, nu):
    o = np.empty((Q.shape[0], V.shape[1]), np.float32)
    R.ref_ns_attention(Q, K, V, mask, T, eta, nu, o, Q.shape[0], Q.shape[1], V.shape[1])
    return o


# M12: seed 42, uniform(-0.5, 0.5), seq 8, d 16, eta 0.2, nu 0.1
# M12 draws four values in (-1, 1) after its last set_global_seed(42), then Q, K and V
R.ref_seed(42)
t = np.empty((1, 4), np.float32)
R.ref_fill_random(t, 1, 4, -1.0, 1.0)
Q = np.empty((8, 16), np.float32); K = Q.copy(); V = Q.copy()
R.ref_fill_random(Q, 8, 16, -0.5, 0.5); R.ref_fill_random(K, 8, 16, -0.5, 0.5); R.ref_fill_random(V, 8, 16, -0.5, 0.5)
out.update(m12_Q=Q, m12_K=K, m12_V=V, m12_ns=ns(Q, K, V, causal(8), 4.0, 0.2, 0.1),
           m12_ns_eta1=ns(Q, K, V, causal(8), 4.0, 1.0, 0.1))

# M20 hand case: eta = 1, nu = 0, T = sqrt(2)
Q = np.array([[1, 2], [3, 4]], np.float32); K = np.array([[2, 0], [0, 1]], np.float32)
V = np.array([[10, 0], [0, 10]], np.float32)
out.update(m20_Q=Q, m20_K=K, m20_V=V, m20_ns=ns(Q, K, V, causal(2), np.sqrt(np.float32(2)), 1.0, 0.0),
           m20_std=ns(Q, K, V, causal(2), np.sqrt(np.float32(2)), 0.0, 0.0))
# M20 diffusion case: constant 0.1 Q/K, V with one spike, nu = 1 and nu = 0
Q = np.full((3, 3), 0.1, np.float32); K = Q.copy(); V = np.zeros((3, 2), np.float32); V[1, 0] = 10
out.update(m20d_Q=Q, m20d_K=K, m20d_V=V, m20d_nu1=ns(Q, K, V, causal(3), 1.0, 0.0, 1.0),
           m20d_nu0=ns(Q, K, V, causal(3), 1.0, 0.0, 0.0))

# seeded cases through the whole per-head attention (mask choice, blend)
rng = np.random.default_rng(2024)
seq, dk = 48, 16
Q, K, V = (rng.standard_normal((seq, dk)).astype(np.float32) for _ in range(3))
out.update(full_Q=Q, full_K=K, full_V=V)
cases = [(1, 8, 4, 1, 0.3), (0, 8, 4, 1, 1.0), (1, 8, 4, 0, 0.3), (1, 16, 5, 1, 0.7), (1, 64, 16, 1, 1.0)]
out["full_cases"] = np.array(cases, np.float32)
for n, (sp, w, s, use_ns, al) in enumerate(cases):
    o = np.empty((seq, dk), np.float32)
    R.ref_attention_full(Q, K, V, seq, dk, sp, w, s, use_ns, al, 0.1, 0.05, o)
    out[f"full_out{n}"] = o

# Shunyam masks
for (s_, w_, st_) in [(20, 8, 4), (33, 8, 5), (9, 8, 4), (70, 64, 16)]:
    m = np.empty((s_, s_), np.float32)
    R.ref_shunyam_mask(m, s_, w_, st_)
    out[f"mask_{s_}_{w_}_{st_}"] = (m == 0).astype(np.uint8)

# multi-head forward, d_model 64, 4 heads, seq 40, reference defaults (sparse 8/4, NS alpha 0.3)
d_model, H, dk, seq = 64, 4, 16, 40
X = rng.standard_normal((seq, d_model)).astype(np.float32)
W = {k: (rng.standard_normal(shp) * 0.1).astype(np.float32) for k, shp in
     dict(WQ=(H, d_model, dk), WK=(H, d_model, dk), WV=(H, d_model, dk), WO=(H, dk, d_model),
          Wp=(d_model, d_model)).items()}
cfg = O.HeadCfg(1, 8, 4, 1, 0.3, 0.1, 0.05, 0, 1)
o = np.empty((seq, d_model), np.float32)
R.ref_mha_forward(X, W["WQ"], W["WK"], W["WV"], W["WO"], W["Wp"], seq, d_model, H, C.byref(cfg), o)
out.update(mha_X=X, mha_out=o, **{f"mha_{k}": v for k, v in W.items()})

path = os.path.join(os.path.dirname(__file__), "attention_golden.npz")
np.savez_compressed(path, **out)
print(path, os.path.getsize(path), "bytes,", len(out), "arrays")
