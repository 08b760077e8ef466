"""Bring-up check of the tcgen05 / TMA / TMEM building blocks on one tile, through the C ABI.
Each case runs in the order a bring-up needs: the K-major x K-major product first, then the
K-major x MN-major one."""
import pytest
import torch

from logos_b200 import lib as L

pytestmark = pytest.mark.gpu


def _run(engine, mode, dtype):
    g = torch.Generator(device="cuda").manual_seed(7 + mode)
    code = L.BF16 if dtype == torch.bfloat16 else L.F16
    if mode == 0:
        A = torch.randn((128, 64), device="cuda", generator=g).to(dtype)
        B = torch.randn((128, 64), device="cuda", generator=g).to(dtype)
        want = A.float() @ B.float().T
    else:
        A = torch.rand((128, 128), device="cuda", generator=g).to(dtype)
        B = torch.randn((128, 64), device="cuda", generator=g).to(dtype)
        want = A.float() @ B.float()
    D = torch.full(want.shape, float("nan"), device="cuda")
    rc = engine.lib.logos_selftest_umma(engine.h, mode, code, A.data_ptr(), B.data_ptr(), D.data_ptr())
    assert rc == L.OK, engine.lib.logos_last_error(engine.h)
    engine.synchronize()
    err = (D - want).abs().max().item()
    assert err < 1e-3, f"mode {mode} {dtype}: max-abs {err}"


def test_qk_shape_bf16(engine):
    _run(engine, 0, torch.bfloat16)


def test_pv_shape_bf16(engine):
    _run(engine, 1, torch.bfloat16)


def test_qk_shape_f16(engine):
    _run(engine, 0, torch.float16)


def test_pv_shape_f16(engine):
    _run(engine, 1, torch.float16)


def test_pv_shape_weights_in_tmem_bf16(engine):
    _run(engine, 3, torch.bfloat16)


def test_pv_shape_weights_in_tmem_f16(engine):
    _run(engine, 3, torch.float16)


def test_timing_modes_report_a_plausible_cost(engine):
    """mode 16 + m: 32 x the MMAs of mode m back to back, D[0] = clock cycles.  An MMA of these shapes cannot take
    less than its flops at the tensor pipe's rate (32 or 64 cycles) and should stay within a few times that."""
    for mode, n, floor in ((0, 4, 64.0), (1, 8, 32.0), (3, 8, 32.0)):
        A = torch.zeros((128, 64 if mode == 0 else 128), device="cuda", dtype=torch.bfloat16)
        B = torch.zeros((128, 64), device="cuda", dtype=torch.bfloat16)
        D = torch.zeros((128, 128 if mode == 0 else 64), device="cuda")
        rc = engine.lib.logos_selftest_umma(engine.h, 16 + mode, L.BF16, A.data_ptr(), B.data_ptr(), D.data_ptr())
        assert rc == L.OK, engine.lib.logos_last_error(engine.h)
        engine.synchronize()
        per_mma = float(D[0, 0]) / (32 * n)
        assert 0.9 * floor <= per_mma <= 8 * floor, (mode, per_mma)
    with pytest.raises(L.LogosError):
        engine._check(engine.lib.logos_selftest_umma(engine.h, 18, L.BF16, A.data_ptr(), B.data_ptr(), D.data_ptr()))
