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


def test_weight_shadow_index_maps():
    """The K-major shadows that logos_mha_forward takes, as include/logos_attn.h states them:
    Wt_qkv[(which H + h) 64 + c][k] = W_which[h][k][c]; for the CPU classes Wt_o is block diagonal with
    Wt_o[h 64 + j][h 64 + c] = W_O[h][c][j]; Wt_proj[n][k] = W_proj[k][n]."""
    import torch
    from logos_b200.attention import MultiHeadAttention
    H, d, dk = 3, 192, 64
    g = torch.Generator().manual_seed(0)
    WQ, WK, WV = (torch.randn((H, d, dk), generator=g) for _ in range(3))
    WO = torch.randn((H, dk, d), generator=g)
    Wp = torch.randn((d, d), generator=g)
    mha = MultiHeadAttention(None, WQ, WK, WV, WO, Wp)
    Wt_qkv, Wt_o, Wt_proj = mha.shadows(torch.float32)
    assert Wt_qkv.shape == (3 * H * dk, d) and Wt_o.shape == (d, H * dk) and Wt_proj.shape == (d, d)
    for which, W in enumerate((WQ, WK, WV)):
        for h in range(H):
            assert torch.equal(Wt_qkv[(which * H + h) * dk:(which * H + h + 1) * dk], W[h].t())
    for h in range(H):
        assert torch.equal(Wt_o[h * dk:(h + 1) * dk, h * dk:(h + 1) * dk], WO[h][:, :dk].t())
    off = Wt_o.clone()
    for h in range(H):
        off[h * dk:(h + 1) * dk, h * dk:(h + 1) * dk] = 0
    assert not bool(off.any())
    assert torch.equal(Wt_proj, Wp.t())
    # what the shadows compute is the class's forward after the attention: concat = first dk columns of head_out W_O[h]
    head_out = torch.randn((H, 5, dk), generator=g)
    concat = torch.cat([(head_out[h] @ WO[h])[:, :dk] for h in range(H)], dim=1)
    tokens = head_out.permute(1, 0, 2).reshape(5, H * dk)
    assert torch.allclose(tokens @ Wt_o.t(), concat, atol=1e-5)
