"""The C-ABI library: it loads without a GPU, exports every function include/logos_attn.h
declares, and refuses to hand out a context when there is no device (no CPU fallback)."""
import ctypes as C
import os
import re

import pytest

from logos_b200 import lib as L

ROOT = os.path.abspath(os.path.join(os.path.dirname(__file__), ".."))


def declared_functions():
    names = set()
    for fn in os.listdir(os.path.join(ROOT, "include")):
        if fn.endswith(".h"):
            text = open(os.path.join(ROOT, "include", fn)).read()
            text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
            names |= set(re.findall(r"\b(logos_[a-z0-9_]+)\s*\(", text))
    return names


def test_library_exports_every_declared_symbol():
    lib = L.load_library()
    declared = declared_functions()
    assert declared, "header parse found nothing"
    for name in declared:
        assert hasattr(lib, name), f"{name} declared in include/ but not exported"
    assert declared == set(L.SIGNATURES), "python binding and header disagree"


def test_version_and_status_strings():
    lib = L.load_library()
    assert lib.logos_abi_version() == 1
    seen = {lib.logos_status_string(i) for i in range(7)}
    assert len(seen) == 7 and b"ok" in seen
    assert lib.logos_status_string(99) == b"unknown status"


def test_no_device_means_no_context():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    lib = L.load_library()
    h = C.c_void_p()
    assert lib.logos_ctx_create(0, C.byref(h)) == L.ERR_NO_DEVICE
    assert not h.value
    from logos_b200.engine import Engine
    with pytest.raises(L.LogosError):
        Engine(0)


def test_null_context_is_rejected_without_touching_a_device():
    lib = L.load_library()
    p = L.Params.make(0.125)
    assert lib.logos_attention_fwd(None, 0, 0, None, None, None, None, 1, 1, 1, 64, C.byref(p)) == L.ERR_INVALID_ARG
    assert lib.logos_decode_int8(None, None, None, None, None, None, None, None, 1, 1, 1, 64, C.byref(p), None) == L.ERR_INVALID_ARG
    assert lib.logos_kv_quantize(None, 0, None, 0, None, 0, None, 1, 16) == L.ERR_INVALID_ARG
    assert lib.logos_ctx_destroy(None) == L.OK
    assert lib.logos_decode_workspace_bytes(64, 16, 8192, 64) > 64 * 1024


def test_shim_exports_the_reference_symbol():
    """liblogos_attn_shim.so defines cuda_flash_attention_fwd with the C++ signature the reference
    declares (cuda/VedicGEMM.cuh:236-243): (const float*, const float*, const float*, float*, float*,
    int, int, float, bool, bool, int, int)."""
    import subprocess
    from logos_b200.build import SHIM, build
    build()
    out = subprocess.run(["nm", "-D", "--defined-only", SHIM], capture_output=True, text=True, check=True).stdout
    assert "_Z24cuda_flash_attention_fwdPKfS0_S0_PfS1_iifbbii" in out
