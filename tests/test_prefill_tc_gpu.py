"""The tensor-core (tcgen05) prefill kernel against the CPU oracle and against the engine's own
exact fp32 kernel, on the shapes it takes: DH 64, BF16 / FP16 inputs, causal, optional pure
sliding window, optional Navier-Stokes prologue (advection + causal diffusion)."""
import numpy as np
import pytest
import torch

import oracle as O
from logos_b200 import lib as L
from logos_b200 import synthetic as syn
from helpers import assert_close

pytestmark = pytest.mark.gpu

CASES = [
    # (window, eta, nu, mode)
    (0, 0.0, 0.0, L.DIFFUSE_NONE),
    (0, 0.1, 0.05, L.DIFFUSE_CAUSAL),
    (0, 0.1, 0.0, L.DIFFUSE_NONE),
    (64, 0.1, 0.05, L.DIFFUSE_CAUSAL),
    (32, 0.0, 0.0, L.DIFFUSE_NONE),
]


def run(engine, engine_general, B, H, S, dtype, case, seed, outliers=False):
    w, eta, nu, mode = case[:4]
    stride = case[4] if len(case) > 4 else 0
    Q, K, V = (syn.normal((B, H, S, 64), seed, t) for t in (1, 2, 3))
    if outliers:
        K[syn.normal((B, H, S, 64), seed, 9) > 2.3] *= 8
    dev = lambda a: torch.from_numpy(a).cuda().to(dtype)
    Qt, Kt, Vt = dev(Q), dev(K), dev(V)
    p = L.Params.make(0.125, True, w, stride, eta, nu, 1.0, mode)
    got = engine.attention(Qt, Kt, Vt, p, out_dtype=torch.float32)
    engine.synchronize()
    got = got.cpu().numpy()
    Qr, Kr, Vr = (t.float().cpu().numpy() for t in (Qt, Kt, Vt))
    op = O.attn_params(0.125, True, w, stride, eta, nu, 1.0, mode)
    want = O.attention_batched(Qr, Kr, Vr, op)
    assert_close(got, want, f"S={S} {dtype} case={case} vs oracle")
    ref = engine_general.attention(Qt, Kt, Vt, p, out_dtype=torch.float32).cpu().numpy()
    assert_close(got, ref, f"S={S} {dtype} case={case} vs fp32 kernel")
    return got


def test_smallest_case_first(engine, engine_general):
    run(engine, engine_general, 1, 1, 128, torch.bfloat16, CASES[0], 31)


@pytest.mark.parametrize("S", [1, 64, 127, 128, 129, 200, 256, 300, 512])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_shapes_and_switches(engine, engine_general, S, dtype):
    for n, case in enumerate(CASES):
        run(engine, engine_general, 2, 2, S, dtype, case, 40 + n)


# Shunyam with landmarks: (window, eta, nu, mode, stride); 64/16 is the reference's production setting
LANDMARK_CASES = [
    (64, 0.1, 0.05, L.DIFFUSE_CAUSAL, 16),
    (64, 0.0, 0.0, L.DIFFUSE_NONE, 16),
    (8, 0.1, 0.05, L.DIFFUSE_CAUSAL, 5),      # stride does not divide the tile size
    (32, 0.0, 0.05, L.DIFFUSE_CAUSAL, 8),
    (16, 0.1, 0.0, L.DIFFUSE_NONE, 1),        # every key is a landmark: equals full causal attention
]


@pytest.mark.parametrize("S", [65, 127, 200, 513, 1100])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_window_with_landmarks(engine, engine_general, S, dtype):
    for n, case in enumerate(LANDMARK_CASES):
        run(engine, engine_general, 1, 2, S, dtype, case, 70 + n, outliers=(n == 0))


def test_gather_kernel_keeps_the_shapes_the_tensor_core_kernel_declines(engine, engine_general):
    """Viscosity above 1/2 is outside the tcgen05 kernel's FP16 weight range: Shunyam shapes then run on the
    mma.sync gather kernel (window + landmark tiles), everything else on the fp32 kernel."""
    run(engine, engine_general, 1, 2, 700, torch.bfloat16, (64, 0.1, 0.6, L.DIFFUSE_CAUSAL, 16), 90)
    run(engine, engine_general, 1, 2, 300, torch.float16, (16, 0.1, 0.7, L.DIFFUSE_CAUSAL, 0), 91)


@pytest.mark.parametrize("S,stride", [(2500, 16), (2500, 3), (4096, 64), (1500, 1)])
def test_landmarks_over_many_tiles(engine, engine_general, S, stride):
    """Several landmark tiles per work item (more than 128 landmarks), strides that do and do not divide the
    tile size, stride 1 (every key a landmark: full causal attention)."""
    run(engine, engine_general, 1, 2, S, torch.bfloat16, (64, 0.1, 0.05, L.DIFFUSE_CAUSAL, stride), 95, outliers=True)
    run(engine, engine_general, 1, 1, S, torch.float16, (32, 0.0, 0.0, L.DIFFUSE_NONE, stride), 96)


def test_outlier_keys_long_sequence(engine, engine_general):
    # 1 % of K entries x8: large score spread, the lazy re-scaling of O must still be exact enough
    run(engine, engine_general, 1, 2, 1024, torch.bfloat16, CASES[1], 50, outliers=True)
    run(engine, engine_general, 1, 2, 1024, torch.bfloat16, CASES[3], 51, outliers=True)


def test_sixteen_bit_output_is_rounded_fp32(engine):
    Q, K, V = (torch.from_numpy(syn.normal((1, 2, 256, 64), 52, t)).cuda().bfloat16() for t in (1, 2, 3))
    p = L.Params.make(0.125, True, 0, 0, 0.1, 0.05, 1.0, L.DIFFUSE_CAUSAL)
    a = engine.attention(Q, K, V, p, out_dtype=torch.float32)
    b = engine.attention(Q, K, V, p)
    engine.synchronize()
    assert b.dtype == torch.bfloat16 and torch.equal(b, a.bfloat16())


def test_full_size_sampled(engine):
    """Causal prefill at B=4, H=16, S=4096 (benchmark configuration 2): sampled heads and rows
    against the oracle, plus a property -- rows of the output are convex combinations of V_s
    rows, so every output lies inside the per-channel range of V."""
    B, H, S = 4, 16, 4096
    g = torch.Generator(device="cuda").manual_seed(60)
    Q, K, V = (torch.randn((B, H, S, 64), device="cuda", generator=g).bfloat16() for _ in range(3))
    p = L.Params.make(0.125, True, 0, 0, 0.1, 0.05, 1.0, L.DIFFUSE_CAUSAL)
    out = engine.attention(Q, K, V, p, out_dtype=torch.float32)
    engine.synchronize()
    assert bool(torch.isfinite(out).all())
    vmax = V.float().amax(dim=2, keepdim=True) + 1e-2
    vmin = V.float().amin(dim=2, keepdim=True) - 1e-2
    assert bool(((out <= vmax) & (out >= vmin)).all())
    op = O.attn_params(0.125, True, 0, 0, 0.1, 0.05, 1.0, O.DIFFUSE_CAUSAL)
    for (b, h) in [(0, 0), (3, 15)]:
        q, k, v = (t[b, h].float().cpu().numpy() for t in (Q, K, V))
        for (r0, r1) in [(0, 130), (2040, 2060), (4090, 4096)]:
            want = O.attention_rows(q, k, v, op, r0, r1)
            assert_close(out[b, h, r0:r1].cpu().numpy(), want, f"head {(b, h)} rows {r0}:{r1}")


@pytest.mark.parametrize("case", [CASES[1], CASES[3]])
def test_many_ragged_items_per_cta(engine, engine_general, case):
    """600 work items of five different lengths on the persistent CTAs, the last block of every
    head with its second query tile beyond the sequence: the whole output against the engine's fp32
    kernel, sampled heads against the oracle."""
    B, H, S = 3, 40, 1100
    w, eta, nu, mode = case
    g = torch.Generator(device="cuda").manual_seed(61)
    Q, K, V = (torch.randn((B, H, S, 64), device="cuda", generator=g).bfloat16() for _ in range(3))
    p = L.Params.make(0.125, True, w, 0, eta, nu, 1.0, mode)
    got = engine.attention(Q, K, V, p, out_dtype=torch.float32)
    engine.synchronize()
    ref = engine_general.attention(Q, K, V, p, out_dtype=torch.float32)
    assert_close(got.cpu().numpy(), ref.cpu().numpy(), f"case={case} vs fp32 kernel")
    op = O.attn_params(0.125, True, w, 0, eta, nu, 1.0, mode)
    for (b, h) in [(0, 0), (1, 17), (2, 39)]:
        q, k, v = (t[b, h].float().cpu().numpy() for t in (Q, K, V))
        assert_close(got[b, h].cpu().numpy(), O.attention_rows(q, k, v, op), f"case={case} head {(b, h)} vs oracle")


@pytest.mark.parametrize("stride", [0, 16])
def test_window_configuration_full_size_sampled(engine, stride):
    """Shunyam window attention at the benchmark's own size (B=8, H=16, S=8192, window 64, 1 % of the K
    entries x8), with the reference's landmark stride 16 (cuda/train_gpu.cu:1172-1173) and without:
    sampled heads and row ranges against the oracle -- the first block, rows around the window length,
    block boundaries of both kernels' tilings, and the last rows (about 508 landmarks per row there)."""
    B, H, S, W = 8, 16, 8192, 64
    g = torch.Generator(device="cuda").manual_seed(62 + stride)
    Q, K, V = (torch.randn((B, H, S, 64), device="cuda", generator=g) for _ in range(3))
    K[torch.rand(K.shape, device="cuda", generator=g) < 0.01] *= 8
    Q, K, V = Q.bfloat16(), K.bfloat16(), V.bfloat16()
    p = L.Params.make(0.125, True, W, stride, 0.1, 0.05, 1.0, L.DIFFUSE_CAUSAL)
    out = engine.attention(Q, K, V, p, out_dtype=torch.float32)
    engine.synchronize()
    assert bool(torch.isfinite(out).all())
    op = O.attn_params(0.125, True, W, stride, 0.1, 0.05, 1.0, O.DIFFUSE_CAUSAL)
    for (b, h) in [(0, 0), (5, 9), (7, 15)]:
        q, k, v = (t[b, h].float().cpu().numpy() for t in (Q, K, V))
        for (r0, r1) in [(0, 140), (250, 262), (1020, 1030), (4090, 4102), (8120, 8192)]:
            want = O.attention_rows(q, k, v, op, r0, r1)
            assert_close(out[b, h, r0:r1].cpu().numpy(), want, f"stride {stride} head {(b, h)} rows {r0}:{r1}")
