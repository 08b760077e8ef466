"""ctypes access to the test-only checkers in this folder.

TEST INFRASTRUCTURE ONLY: imported by tests/, by the smoke check and by the
CPU-baseline leg of the benchmark.  The product package never imports it.

`lib()`     -> the C restatement (liblogos_oracle.so), built on demand with gcc.
`ref()`     -> the reference's own CPU headers behind C entry points
               (oracle/_ref/liblogos_ref.so), or None when it was not built.
`refgpu()`  -> the reference's own CUDA kernels for sm_100a
               (oracle/_ref/liblogos_refgpu.so), or None.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from functools import lru_cache

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))

f32p = np.ctypeslib.ndpointer(dtype=np.float32, flags="C_CONTIGUOUS")
i8p = np.ctypeslib.ndpointer(dtype=np.int8, flags="C_CONTIGUOUS")
i32p = np.ctypeslib.ndpointer(dtype=np.int32, flags="C_CONTIGUOUS")

DIFFUSE_NONE, DIFFUSE_CAUSAL, DIFFUSE_CENTRAL = 0, 1, 2


class HeadCfg(C.Structure):
    _fields_ = [("use_sparse", C.c_int), ("sparse_window", C.c_int), ("sparse_stride", C.c_int),
                ("use_navier_stokes", C.c_int), ("ns_alpha", C.c_float), ("ns_eta", C.c_float),
                ("ns_nu", C.c_float), ("kv_int8_roundtrip", C.c_int), ("threads", C.c_int)]


class AttnParams(C.Structure):
    _fields_ = [("scale", C.c_float), ("causal", C.c_int), ("window", C.c_int),
                ("stride", C.c_int), ("ns_eta", C.c_float), ("ns_nu", C.c_float),
                ("ns_alpha", C.c_float), ("diffuse_mode", C.c_int)]


def build(force: bool = False) -> None:
    """Compile the C restatement (and, when the reference tree is present, oracle/_ref)."""
    so = os.path.join(HERE, "liblogos_oracle.so")
    src = os.path.join(HERE, "logos_oracle.c")
    if force or not os.path.exists(so) or os.path.getmtime(so) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", HERE, "oracle"], stdout=subprocess.DEVNULL)
    ref_tree = os.path.abspath(os.path.join(HERE, "..", "..", "reference"))
    if os.path.isdir(os.path.join(ref_tree, "include")):
        subprocess.check_call(["make", "-C", HERE, "ref", "refgpu", "refbwd"], stdout=subprocess.DEVNULL)
        if os.path.exists(os.path.join(HERE, "..", "logos_b200", "liblogos_attn_shim.so")):
            subprocess.check_call(["make", "-C", HERE, "refmodel"], stdout=subprocess.DEVNULL)


@lru_cache(maxsize=None)
def lib() -> C.CDLL:
    build()
    L = C.CDLL(os.path.join(HERE, "liblogos_oracle.so"))
    L.lo_gemm.argtypes = [f32p, f32p, f32p, C.c_int, C.c_int, C.c_int]
    L.lo_boltzmann_softmax.argtypes = [f32p, f32p, C.c_int, C.c_int, C.c_float]
    L.lo_causal_mask.argtypes = [f32p, C.c_int]
    L.lo_shunyam_mask.argtypes = [f32p, C.c_int, C.c_int, C.c_int]
    L.lo_ns_attention.argtypes = [f32p, f32p, f32p, f32p, C.c_float, C.c_float, C.c_float, f32p,
                                  C.c_int, C.c_int, C.c_int]
    L.lo_std_attention.argtypes = [f32p, f32p, f32p, f32p, C.c_float, f32p, C.c_int, C.c_int,
                                   C.c_int]
    L.lo_head_forward.argtypes = [f32p, f32p, f32p, f32p, f32p, C.c_int, C.c_int, C.c_int,
                                  C.POINTER(HeadCfg), f32p, C.c_void_p]
    L.lo_mha_forward.argtypes = [f32p, f32p, f32p, f32p, f32p, f32p, C.c_int, C.c_int, C.c_int,
                                 C.POINTER(HeadCfg), f32p]
    for name in ("lo_ns_advect", "lo_ns_diffuse_causal", "lo_ns_diffuse_central"):
        getattr(L, name).argtypes = [f32p, f32p, C.c_int, C.c_int, C.c_float]
    L.lo_allowed.argtypes = [C.c_int, C.c_int, C.c_int, C.POINTER(AttnParams)]
    L.lo_allowed.restype = C.c_int
    L.lo_attention_rows_f64.argtypes = [f32p, f32p, f32p, f32p, C.c_int, C.c_int, C.c_int,
                                        C.c_int, C.POINTER(AttnParams)]
    L.lo_attention_bwd_f64.argtypes = [f32p, f32p, f32p, f32p, C.c_int, C.c_int, C.POINTER(AttnParams), f32p, f32p,
                                       f32p]
    L.lo_absmax.argtypes = [f32p, C.c_long]
    L.lo_absmax.restype = C.c_float
    L.lo_nikhilam_scale.argtypes = [C.c_float]
    L.lo_nikhilam_scale.restype = C.c_float
    L.lo_nikhilam_quantize.argtypes = [f32p, i8p, C.c_float, C.c_long]
    L.lo_nikhilam_dequantize.argtypes = [i8p, f32p, C.c_float, C.c_long]
    L.lo_nikhilam_compress.argtypes = [f32p, i8p, C.c_long]
    L.lo_nikhilam_compress.restype = C.c_float
    L.lo_decode_int8.argtypes = [f32p, C.c_void_p, i8p, i8p, C.c_float, C.c_float, C.c_int,
                                 C.c_int, C.POINTER(AttnParams), f32p]
    L.lo_decode_int8_batch.argtypes = [f32p, C.c_void_p, i8p, i8p, f32p, f32p, i32p, C.c_int,
                                       C.c_int, C.c_int, C.POINTER(AttnParams), f32p, C.c_int]
    L.lo_max_threads.restype = C.c_int
    return L


def _cpu_has_avx2_fma() -> bool:
    try:
        with open("/proc/cpuinfo") as f:
            flags = next((ln for ln in f if ln.startswith("flags")), "")
        return " avx2" in flags and " fma" in flags and " bmi2" in flags
    except OSError:
        return False


@lru_cache(maxsize=None)
def ref_v3():
    """The reference CPU headers built for x86-64-v3, or None (not built / this CPU lacks AVX2+FMA)."""
    if not _cpu_has_avx2_fma():
        return None
    return _load_ref(os.path.join(HERE, "_ref", "liblogos_ref_v3.so"))


@lru_cache(maxsize=None)
def ref():
    return _load_ref(os.path.join(HERE, "_ref", "liblogos_ref.so"))


def _load_ref(path):
    if not os.path.exists(path):
        return None
    L = C.CDLL(path)
    L.ref_gemm.argtypes = [f32p, f32p, f32p, C.c_int, C.c_int, C.c_int]
    L.ref_boltzmann_softmax.argtypes = [f32p, f32p, C.c_int, C.c_int, C.c_float]
    L.ref_causal_mask.argtypes = [f32p, C.c_int]
    L.ref_shunyam_mask.argtypes = [f32p, C.c_int, C.c_int, C.c_int]
    L.ref_ns_attention.argtypes = [f32p, f32p, f32p, f32p, C.c_float, C.c_float, C.c_float, f32p,
                                   C.c_int, C.c_int, C.c_int]
    L.ref_attention_full.argtypes = [f32p, f32p, f32p, C.c_int, C.c_int, C.c_int, C.c_int,
                                     C.c_int, C.c_int, C.c_float, C.c_float, C.c_float, f32p]
    L.ref_head_forward.argtypes = [f32p, f32p, f32p, f32p, f32p, C.c_int, C.c_int, C.c_int,
                                   C.POINTER(HeadCfg), f32p]
    L.ref_mha_forward.argtypes = [f32p, f32p, f32p, f32p, f32p, f32p, C.c_int, C.c_int, C.c_int,
                                  C.POINTER(HeadCfg), f32p]
    L.ref_attention_full_batch.argtypes = [f32p, f32p, f32p, C.c_int, C.c_int, C.c_int, C.c_int,
                                           C.c_int, C.c_int, C.c_int, C.c_float, C.c_float,
                                           C.c_float, f32p, C.c_int]
    L.ref_hardware_threads.restype = C.c_int
    L.ref_seed.argtypes = [C.c_uint]
    L.ref_fill_random.argtypes = [f32p, C.c_int, C.c_int, C.c_float, C.c_float]
    return L


@lru_cache(maxsize=None)
def refgpu():
    path = os.path.join(HERE, "_ref", "liblogos_refgpu.so")
    if not os.path.exists(path):
        return None
    L = C.CDLL(path)
    vp = C.c_void_p
    L.refgpu_absmax.argtypes = [vp, vp, C.c_int]
    L.refgpu_quantize.argtypes = [vp, vp, C.c_float, C.c_int]
    L.refgpu_dequantize.argtypes = [vp, vp, C.c_float, C.c_int]
    L.refgpu_ns_advect.argtypes = [vp, vp, C.c_int, C.c_int, C.c_float]
    L.refgpu_ns_diffuse.argtypes = [vp, vp, C.c_int, C.c_int, C.c_float]
    L.refgpu_flash_attention_fwd.argtypes = [vp, vp, vp, vp, C.c_int, C.c_int, C.c_float, C.c_int,
                                             C.c_int, C.c_int, C.c_int]
    return L


def refmodel(kind: str):
    """Path of oracle/_ref/refmodel_stock or refmodel_dropin (the reference's ModelGPU::forward as a
    program), or None when it was not built."""
    path = os.path.join(HERE, "_ref", f"refmodel_{kind}")
    return path if os.path.exists(path) else None


# ---------------------------------------------------------------- numpy front ends

def _f(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def attn_params(scale, causal=True, window=0, stride=0, ns_eta=0.0, ns_nu=0.0, ns_alpha=1.0,
                diffuse_mode=DIFFUSE_NONE) -> AttnParams:
    return AttnParams(float(scale), int(causal), int(window), int(stride), float(ns_eta),
                      float(ns_nu), float(ns_alpha), int(diffuse_mode))


def attention_rows(Q, K, V, p: AttnParams, row0=0, row1=None):
    """fp64-accumulated attention rows [row0,row1) of one head; Q,K,V are [seq, d]."""
    Q, K, V = _f(Q), _f(K), _f(V)
    seq, d = Q.shape
    row1 = seq if row1 is None else row1
    out = np.empty((row1 - row0, d), np.float32)
    lib().lo_attention_rows_f64(Q, K, V, out, seq, d, row0, row1, C.byref(p))
    return out


def attention_batched(Q, K, V, p: AttnParams):
    """[..., seq, d] -> [..., seq, d], every leading index an independent head."""
    Q, K, V = _f(Q), _f(K), _f(V)
    lead = Q.shape[:-2]
    Qf, Kf, Vf = (x.reshape((-1,) + x.shape[-2:]) for x in (Q, K, V))
    out = np.stack([attention_rows(Qf[i], Kf[i], Vf[i], p) for i in range(Qf.shape[0])])
    return out.reshape(lead + out.shape[-2:])


def nikhilam_compress(x):
    """-> (int8 array of x.shape, fp32 scale); one scale for the whole tensor."""
    x = _f(x)
    q = np.empty(x.shape, np.int8)
    s = lib().lo_nikhilam_compress(x.reshape(-1), q.reshape(-1), x.size)
    return q, np.float32(s)


def nikhilam_quantize(x, scale):
    x = _f(x)
    q = np.empty(x.shape, np.int8)
    lib().lo_nikhilam_quantize(x.reshape(-1), q.reshape(-1), float(scale), x.size)
    return q


def nikhilam_dequantize(q, scale):
    q = np.ascontiguousarray(q, dtype=np.int8)
    x = np.empty(q.shape, np.float32)
    lib().lo_nikhilam_dequantize(q.reshape(-1), x.reshape(-1), float(scale), q.size)
    return x


def decode_int8_batch(q, q_prev, Kq, Vq, k_scale, v_scale, lens, p: AttnParams, threads=0):
    """q,q_prev: [n,d]; Kq,Vq: [n,s_max,d] int8; scales,lens: [n] -> out [n,d]."""
    q = _f(q)
    n, d = q.shape
    s_max = Kq.shape[1]
    out = np.empty((n, d), np.float32)
    qp = None
    if q_prev is not None:
        qp_arr = _f(q_prev)
        qp = qp_arr.ctypes.data_as(C.c_void_p)
    lib().lo_decode_int8_batch(q, qp, np.ascontiguousarray(Kq, np.int8),
                               np.ascontiguousarray(Vq, np.int8), _f(k_scale), _f(v_scale),
                               np.ascontiguousarray(lens, np.int32), n, s_max, d, C.byref(p), out,
                               threads or lib().lo_max_threads())
    return out


def attention_bwd(Q, K, V, dO, p: AttnParams):
    """Gradients (dQ, dK, dV) of attention_batched's output with respect to Q, K, V ([B, H, S, d] fp32) for
    a given dO, fp64 inside (lo_attention_bwd_f64)."""
    Q, K, V, dO = (_f(a) for a in (Q, K, V, dO))
    B, H, S, d = Q.shape
    dQ, dK, dV = (np.empty_like(Q) for _ in range(3))
    fn = lib().lo_attention_bwd_f64
    for b in range(B):
        for h in range(H):
            fn(Q[b, h], K[b, h], V[b, h], dO[b, h], S, d, C.byref(p), dQ[b, h], dK[b, h], dV[b, h])
    return dQ, dK, dV
