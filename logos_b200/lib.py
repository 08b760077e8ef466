"""ctypes binding of the C ABI in include/logos_attn.h.

Loading fails loudly: there is no CPU fallback, so a missing or unloadable
`liblogos_attn.so` raises instead of degrading.
"""
from __future__ import annotations

import ctypes as C
import os
from functools import lru_cache

PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(PKG, "liblogos_attn.so")

OK, ERR_INVALID_ARG, ERR_UNSUPPORTED, ERR_WORKSPACE, ERR_CUDA, ERR_NO_DEVICE, ERR_ALIGNMENT = range(7)
ERR_SCRATCH_LIMIT = 7
ERR_KERNEL_TIMEOUT = 8
F32, BF16, F16 = 0, 1, 2
DIFFUSE_NONE, DIFFUSE_CAUSAL, DIFFUSE_CENTRAL = 0, 1, 2
class Strides(C.Structure):
    """logos_strides: elements between two sequences, two heads, two rows."""
    _fields_ = [("batch", C.c_int64), ("head", C.c_int64), ("row", C.c_int64)]


MHA_ATTEND_DEQUANTIZED = 1
OPT_FORCE_GENERAL, OPT_DECODE_CHUNK, OPT_PEER_WAIT_MS, OPT_WORKSPACE_LOCK, OPT_GEMM_NARROW, OPT_DECODE_DEPTH = 0, 1, 2, 3, 4, 5
OPT_QKV_OUT_F16, OPT_PROJECT_OVERLAP = 6, 7
COMM_HANDLE_BYTES = 80


ALLOC_FN = C.CFUNCTYPE(C.c_int, C.POINTER(C.c_void_p), C.c_size_t, C.c_void_p)   # logos_alloc_fn
FREE_FN = C.CFUNCTYPE(None, C.c_void_p, C.c_void_p)                                 # logos_free_fn


class LogosError(RuntimeError):
    def __init__(self, status: int, message: str):
        super().__init__(f"logos_attn status {status}: {message}")
        self.status = status


class Params(C.Structure):
    """logos_attn_params."""
    _fields_ = [("scale", C.c_float), ("causal", C.c_int), ("window", C.c_int),
                ("stride", C.c_int), ("ns_eta", C.c_float), ("ns_nu", C.c_float),
                ("ns_alpha", C.c_float), ("diffuse_mode", C.c_int)]

    @classmethod
    def make(cls, scale, causal=True, window=0, stride=0, ns_eta=0.0, ns_nu=0.0, ns_alpha=1.0,
             diffuse_mode=DIFFUSE_NONE) -> "Params":
        return cls(float(scale), int(causal), int(window), int(stride), float(ns_eta),
                   float(ns_nu), float(ns_alpha), int(diffuse_mode))


# name -> (restype, argtypes); every symbol include/logos_attn.h declares
_vp, _i, _f, _i64, _sz = C.c_void_p, C.c_int, C.c_float, C.c_int64, C.c_size_t
_PP = C.POINTER(Params)
SIGNATURES = {
    "logos_abi_version": (_i, []),
    "logos_status_string": (C.c_char_p, [_i]),
    "logos_ctx_create": (_i, [_i, C.POINTER(_vp)]),
    "logos_ctx_destroy": (_i, [_vp]),
    "logos_ctx_set_stream": (_i, [_vp, _vp]),
    "logos_ctx_reserve": (_i, [_vp, _sz]),
    "logos_ctx_set_workspace": (_i, [_vp, _vp, _sz]),
    "logos_ctx_set_allocator": (_i, [_vp, _vp, _vp, _vp]),
    "logos_ctx_synchronize": (_i, [_vp]),
    "logos_last_error": (C.c_char_p, [_vp]),
    "logos_ctx_set_option": (_i, [_vp, _i, _i]),
    "logos_comm_create": (_i, [_vp, _i, _i, _sz, C.POINTER(_vp)]),
    "logos_comm_handle": (_i, [_vp, _vp]),
    "logos_comm_connect": (_i, [_vp, _vp]),
    "logos_comm_connect_local": (_i, [C.POINTER(_vp), _i]),
    "logos_comm_destroy": (_i, [_vp]),
    "logos_decode_int8_push": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _PP]),
    "logos_decode_int8_collect": (_i, [_vp, _vp, _vp, _i, _i, _i]),
    "logos_decode_int8_gather": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _PP, _vp]),
    "logos_decode_step_int8": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _PP, _vp]),
    "logos_decode_step_int8_to": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _PP, _i, _vp]),
    "logos_layer_norm": (_i, [_vp, _i, _vp, _vp, _vp, _vp, _i, _i, C.c_float]),
    "logos_decode_step_int8_gather": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i,
                                          _PP, _vp]),
    "logos_comm_push": (_i, [_vp, _vp, _vp, _i, _i, _sz]),
    "logos_comm_wait": (_i, [_vp, _vp, _vp, _sz]),
    "logos_comm_all_gather_heads": (_i, [_vp, _vp, _vp, _vp, _i, _i, _sz]),
    "logos_flash_attention_fwd_f32": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _f, _i, _i, _i, _i]),
    "logos_attention_fwd": (_i, [_vp, _i, _i, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _PP]),
    "logos_prefill_fwd": (_i, [_vp, _i, _i, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _PP, _vp, _vp, _vp, _vp, _i]),
    "logos_selftest_umma": (_i, [_vp, _i, _i, _vp, _vp, _vp]),
    "logos_attention_workspace_bytes": (_sz, [_i, _i, _i, _i]),
    "logos_kv_quantize": (_i, [_vp, _i, _vp, _i64, _vp, _i64, _vp, _i, _i64]),
    "logos_kv_quantize_absmax": (_i, [_vp, _i, _vp, _i64, _vp, _i64, _vp, _vp, _i, _i64]),
    "logos_project": (_i, [_vp, _i, _i, _vp, _vp, _vp, _vp, _i, _i, _i]),
    "logos_qkv_project": (_i, [_vp, _i, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _vp, _vp]),
    "logos_project_heads": (_i, [_vp, _i, _i, _vp, _vp, _vp, _vp, _i, _i, _i, _i]),
    "logos_kv_dequantize16": (_i, [_vp, _i, _vp, _i64, _vp, _vp, _i64, _i, _i64]),
    "logos_attention_fwd_strided": (_i, [_vp, _i, _i, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _vp, _vp, _PP]),
    "logos_attention_bwd16_workspace_bytes": (_sz, [_i, _i, _i, _i]),
    "logos_attention_bwd16": (_i, [_vp, _i, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _PP]),
    "logos_attention_bwd_workspace_bytes": (_sz, [_i, _i, _i, _i]),
    "logos_attention_bwd": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _PP]),
    "logos_mha_workspace_bytes": (_sz, [_i, _i, _i, _i]),
    "logos_mha_f32_workspace_bytes": (_sz, [_i, _i, _i]),
    "logos_mha_forward_f32": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _PP, _i, _vp, _sz]),
    "logos_gemm_f32": (_i, [_vp, _vp, _i, _i64, _vp, _i, _i64, _vp, _i, _i64, _i, _i, _i, _i]),
    "logos_mha_forward": (_i, [_vp, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _PP, _vp, _vp, _vp, _vp,
                               _i, _i, _vp, _sz]),
    "logos_kv_dequantize": (_i, [_vp, _vp, _i64, _vp, _vp, _i64, _i, _i64]),
    "logos_kv_append": (_i, [_vp, _i, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i]),
    "logos_decode_int8": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _PP, _vp]),
    "logos_decode_workspace_bytes": (_sz, [_i, _i, _i, _i]),
    "logos_decode_int8_noalloc": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _PP, _vp]),
    "logos_decode_step_int8_host": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i,
                                        _i, _i, _PP, _vp]),
}


@lru_cache(maxsize=None)
def load_library() -> C.CDLL:
    if not os.path.exists(LIB_PATH):
        raise LogosError(ERR_NO_DEVICE,
                         f"{LIB_PATH} is missing: build it with `python -m logos_b200.build` "
                         "(nvcc, sm_100a); there is no CPU fallback")
    lib = C.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError if the library lacks a declared symbol
        fn.restype = res
        fn.argtypes = args
    return lib
