"""The tensor-core projection GEMMs (logos_project, logos_qkv_project) against fp64 products of the
same 16-bit-rounded operands, the Q/K/V scatter into the attention layout, and the epilogue's per-tensor
max|x| against the quantiser's own first pass (bytes and scales must come out identical)."""
import numpy as np
import pytest
import torch

from logos_b200 import lib as L

pytestmark = pytest.mark.gpu


def _ref(A, W):
    return (A.double() @ W.double()).float()


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("M,N,K", [(128, 128, 64), (256, 192, 1024), (300, 1024, 1024), (32, 3072, 1024), (1, 64, 72), (7, 1024, 4096), (33, 128, 256)])
def test_project_matches_fp64_product(engine, dtype, M, N, K):
    g = torch.Generator(device="cuda").manual_seed(M * 7 + N)
    A = (torch.randn((M, K), device="cuda", generator=g)).to(dtype)
    W = (torch.randn((K, N), device="cuda", generator=g) * 0.02).to(dtype)
    Wt = W.t().contiguous()
    want = _ref(A, W)
    got = engine.project(A, Wt, out_dtype=torch.float32)
    engine.synchronize()
    tol = 2e-5 * K ** 0.5 + 1e-6                         # fp32 accumulation of K products of magnitude ~0.02
    assert float((got - want).abs().max()) <= tol
    # 16-bit output with a residual: the rounding of (product + residual)
    R = torch.randn((M, N), device="cuda", generator=g).to(dtype)
    got16 = engine.project(A, Wt, residual=R)
    engine.synchronize()
    ref16 = (want + R.float()).to(dtype)
    # the accumulation order differs from the fp64 product, so allow the last bit of the 16-bit result
    ulp = (ref16.float().abs() * (2.0 ** -7 if dtype == torch.bfloat16 else 2.0 ** -10)).clamp_min(1e-3)
    assert bool(((got16.float() - ref16.float()).abs() <= ulp).all())
    R32 = R.float()
    got32 = engine.project(A, Wt, residual=R32, out_dtype=torch.float32)
    engine.synchronize()
    assert float((got32 - (want + R32)).abs().max()) <= tol + 1e-6


@pytest.mark.parametrize("B,S,H,D", [(2, 128, 2, 256), (3, 200, 4, 512), (1, 77, 1, 64), (2, 256, 16, 1024)])
def test_qkv_project_scatter_and_absmax(engine, B, S, H, D):
    g = torch.Generator(device="cuda").manual_seed(B * 100 + S)
    X = torch.randn((B * S, D), device="cuda", generator=g).bfloat16()
    Wq, Wk, Wv = (torch.randn((H, D, 64), device="cuda", generator=g) * 0.05 for _ in range(3))
    Wq, Wk, Wv = Wq.bfloat16(), Wk.bfloat16(), Wv.bfloat16()
    # K-major shadow of the stacked weight: row (which * H + h) * 64 + c = column c of W_which[h]
    Wt = torch.cat([W.transpose(1, 2).reshape(H * 64, D) for W in (Wq, Wk, Wv)], dim=0).contiguous()
    Q, K, V, ka, va = engine.qkv_project(X, Wt, B, S, H, absmax=True)
    engine.synchronize()
    Xf = X.double().view(B, S, D)
    for got, W in ((Q, Wq), (K, Wk), (V, Wv)):
        want = torch.einsum("bsd,hdc->bhsc", Xf, W.double()).float()
        assert got.shape == (B, H, S, 64)
        err = (got.float() - want).abs()
        assert bool((err <= want.abs() * 2.0 ** -7 + 1e-3).all()), float(err.max())
    # the epilogue's max|x| is the maximum of exactly the stored values
    assert torch.equal(ka, K.float().abs().amax(dim=(2, 3)))
    assert torch.equal(va, V.float().abs().amax(dim=(2, 3)))
    # ... so the cache quantised from it is the one the two-pass quantiser makes
    S_max = S + 5
    kc1 = torch.zeros((B, H, S_max, 64), dtype=torch.int8, device="cuda")
    kc2 = torch.zeros_like(kc1)
    s1 = engine.nikhilam_compress_absmax(K, ka, kc1.view(B * H, S_max, 64))
    _, s2 = engine.nikhilam_compress(K, cache=kc2.view(B * H, S_max, 64))
    engine.synchronize()
    assert torch.equal(s1, s2) and torch.equal(kc1, kc2)


@pytest.mark.parametrize("B,S,H,D", [(32, 1, 16, 1024), (2, 130, 2, 256)])
def test_qkv_project_fp16_output_of_bf16_operands(engine, B, S, H, D):
    """LOGOS_OPT_QKV_OUT_F16: the same accumulators stored as FP16 (what the decode entry points take), the max|x|
    tables those of the stored values; the option does not outlast the call that asked for it."""
    g = torch.Generator(device="cuda").manual_seed(B * 7 + S)
    X = torch.randn((B * S, D), device="cuda", generator=g).bfloat16()
    Wt = (torch.randn((3 * H * 64, D), device="cuda", generator=g) * 0.05).bfloat16()
    Q, K, V, ka, va = engine.qkv_project(X, Wt, B, S, H, absmax=True, out_f16=True)
    Qb, Kb, Vb = engine.qkv_project(X, Wt, B, S, H)
    engine.synchronize()
    assert Q.dtype == torch.float16 and Qb.dtype == torch.bfloat16
    want = (X.double() @ Wt.double().t()).view(B, S, 3, H, 64).permute(2, 0, 3, 1, 4).float()
    for i, (got, gotb) in enumerate(((Q, Qb), (K, Kb), (V, Vb))):
        err = (got.float() - want[i]).abs()
        assert bool((err <= want[i].abs() * 2.0 ** -10 + 1e-3).all()), float(err.max())      # FP16 keeps three more bits
        assert bool(((gotb.float() - want[i]).abs() <= want[i].abs() * 2.0 ** -7 + 1e-3).all())
    assert torch.equal(ka, K.float().abs().amax(dim=(2, 3))) and torch.equal(va, V.float().abs().amax(dim=(2, 3)))


def test_small_projections_launched_to_overlap_the_kernel_before(engine):
    """LOGOS_OPT_PROJECT_OVERLAP: a chain of M <= 32 projections, each reading what the one before wrote, gives the
    same bits as the ordinary launches (the weights are fetched early, the activations after the wait)."""
    g = torch.Generator(device="cuda").manual_seed(77)
    X = torch.randn((32, 1024), device="cuda", generator=g).bfloat16()
    Ws = [(torch.randn((1024, 1024), device="cuda", generator=g) * 0.03).bfloat16() for _ in range(6)]

    def chain():
        y = X
        for W in Ws:
            y = engine.project(y, W, residual=y)
        engine.synchronize()
        return y

    want = chain()
    engine.set_option(L.OPT_PROJECT_OVERLAP, 1)
    try:
        for _ in range(3):
            assert torch.equal(chain(), want)
    finally:
        engine.set_option(L.OPT_PROJECT_OVERLAP, 0)


def test_projection_argument_checks(engine):
    A = torch.zeros((4, 60), device="cuda", dtype=torch.bfloat16)       # K not a multiple of 8
    Wt = torch.zeros((64, 60), device="cuda", dtype=torch.bfloat16)
    with pytest.raises(L.LogosError):
        engine.project(A, Wt)
    A32 = torch.zeros((4, 64), device="cuda")
    with pytest.raises(KeyError if False else L.LogosError):
        engine.project(A32, torch.zeros((64, 64), device="cuda"))       # fp32 operands are not taken


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("B,S,H,N", [(1, 128, 1, 64), (2, 256, 4, 256), (3, 200, 4, 512), (2, 77, 16, 1024), (1, 1, 2, 128)])
def test_project_heads_reads_the_attention_layout(engine, dtype, B, S, H, N):
    """C = sum over heads of head_out[b, h] · W_O[h] with head_out still [B, H, S, 64]: equal to the same
    product on the per-token concatenation, sequences that are no multiple of the tile included."""
    g = torch.Generator(device="cuda").manual_seed(B * 1000 + S + H)
    O_ = torch.randn((B, H, S, 64), device="cuda", generator=g).to(dtype)
    Wo = (torch.randn((H, 64, N), device="cuda", generator=g) * 0.05).to(dtype)
    Wt_o = Wo.reshape(H * 64, N).t().contiguous()                      # [N][H*64]
    want = torch.einsum("bhsc,hcn->bsn", O_.double(), Wo.double()).reshape(B * S, N).float()
    got = engine.project_heads(O_, Wt_o, out_dtype=torch.float32)
    engine.synchronize()
    tol = 2e-5 * (H * 64) ** 0.5 * 3 + 1e-6
    assert float((got - want).abs().max()) <= tol
    # and bit-identical to the row-major GEMM on the concatenated operand (same tiles, same order of k)
    A = O_.permute(0, 2, 1, 3).reshape(B * S, H * 64).contiguous()
    same = engine.project(A, Wt_o, out_dtype=torch.float32)
    engine.synchronize()
    assert torch.equal(got, same)
    R = torch.randn((B * S, N), device="cuda", generator=g).to(dtype)
    got_r = engine.project_heads(O_, Wt_o, residual=R)
    same_r = engine.project(A, Wt_o, residual=R)
    engine.synchronize()
    assert torch.equal(got_r, same_r)


@pytest.mark.parametrize("M,N,K,batch", [(64, 64, 16, 1), (70, 33, 19, 3), (512, 64, 1024, 4), (1, 5, 7, 2), (130, 257, 64, 1)])
def test_gemm_f32_strided_batched(engine, M, N, K, batch):
    g = torch.Generator(device="cuda").manual_seed(M + 3 * N + 7 * K)
    lda, ldb, ldc = K + 3, N + 2, N + 5
    A = torch.randn((batch, M, lda), device="cuda", generator=g)
    Bm = torch.randn((batch, K, ldb), device="cuda", generator=g)
    Cm = torch.full((batch, M, ldc), -7.0, device="cuda")
    from logos_b200.engine import _ptr
    engine._check(engine.lib.logos_gemm_f32(engine.h, _ptr(A), lda, M * lda, _ptr(Bm), ldb, K * ldb, _ptr(Cm), ldc,
                                            M * ldc, M, N, K, batch))
    engine.synchronize()
    want = (A[:, :, :K].double() @ Bm[:, :, :N].double()).float()
    assert float((Cm[:, :, :N] - want).abs().max()) <= 1e-5 * K ** 0.5 + 1e-6
    assert bool((Cm[:, :, N:] == -7.0).all())                     # the padding of C is not touched
    # stride 0: one A for the whole batch
    engine._check(engine.lib.logos_gemm_f32(engine.h, _ptr(A), lda, 0, _ptr(Bm), ldb, K * ldb, _ptr(Cm), ldc,
                                            M * ldc, M, N, K, batch))
    engine.synchronize()
    want0 = (A[0:1, :, :K].double() @ Bm[:, :, :N].double()).float()
    assert float((Cm[:, :, :N] - want0).abs().max()) <= 1e-5 * K ** 0.5 + 1e-6


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_kv_dequantize16_is_the_rounded_fp32_product(engine, dtype):
    g = torch.Generator(device="cuda").manual_seed(5)
    n, S_max, rows = 6, 96, 80
    q = torch.randint(-127, 128, (n, S_max, 64), device="cuda", generator=g, dtype=torch.int8)
    scales = torch.rand((n,), device="cuda", generator=g) * 0.05 + 1e-3
    got = engine.nikhilam_decompress16(q, scales, dtype, rows=rows)
    want32 = engine.nikhilam_decompress(q, scales, rows=rows)
    engine.synchronize()
    assert torch.equal(got, want32.to(dtype))


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("M,N,K", [(148 * 128, 256, 64), (20000, 320, 136), (9000, 3072, 1024), (65536, 1024, 1024)])
def test_wide_kernel_equals_the_narrow_one(engine, dtype, M, N, K):
    """Problems that fill the device take the persistent 128 x 256-tile kernel: bit-identical to the 128 x 128
    kernel (same products in the same order), ragged M, N no multiple of 256, several tiles per CTA, and the
    fp64 product as the outside witness."""
    g = torch.Generator(device="cuda").manual_seed(M + N + K)
    A = torch.randn((M, K), device="cuda", generator=g).to(dtype)
    W = (torch.randn((K, N), device="cuda", generator=g) * 0.02).to(dtype)
    Wt = W.t().contiguous()
    R = torch.randn((M, N), device="cuda", generator=g).to(dtype)
    wide32 = engine.project(A, Wt, out_dtype=torch.float32)
    wide16 = engine.project(A, Wt, residual=R)
    engine.set_option(L.OPT_GEMM_NARROW, 1)
    try:
        narrow32 = engine.project(A, Wt, out_dtype=torch.float32)
        narrow16 = engine.project(A, Wt, residual=R)
    finally:
        engine.set_option(L.OPT_GEMM_NARROW, 0)
    engine.synchronize()
    assert torch.equal(wide32, narrow32) and torch.equal(wide16, narrow16)
    rows = torch.randint(0, M, (64,), device="cuda", generator=g)
    want = (A[rows].double() @ W.double()).float()
    assert float((wide32[rows] - want).abs().max()) <= 2e-5 * K ** 0.5 + 1e-6


def test_wide_kernel_qkv_scatter_and_heads(engine):
    """The wide kernel's other two forms: the Q/K/V scatter with max|x| (four head slices per tile) and the
    head-major A operand, both against the narrow kernel."""
    B, S, H, D = 16, 1280, 4, 512            # 160 m tiles x 3 n tiles: wide; S no multiple of 128 x anything special
    g = torch.Generator(device="cuda").manual_seed(99)
    X = torch.randn((B * S, D), device="cuda", generator=g).bfloat16()
    Wt = (torch.randn((3 * H * 64, D), device="cuda", generator=g) * 0.05).bfloat16()
    outs = engine.qkv_project(X, Wt, B, S, H, absmax=True)
    O_ = torch.randn((B, H, S, 64), device="cuda", generator=g).bfloat16()
    Wt_o = (torch.randn((512, H * 64), device="cuda", generator=g) * 0.05).bfloat16()
    y = engine.project_heads(O_, Wt_o)
    engine.set_option(L.OPT_GEMM_NARROW, 1)
    try:
        outs_n = engine.qkv_project(X, Wt, B, S, H, absmax=True)
        y_n = engine.project_heads(O_, Wt_o)
    finally:
        engine.set_option(L.OPT_GEMM_NARROW, 0)
    engine.synchronize()
    for a_, b_ in zip(outs, outs_n):
        assert torch.equal(a_, b_)
    assert torch.equal(y, y_n)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("rows,D", [(32, 1024), (5, 264), (300, 2048), (1, 8)])
def test_layer_norm_matches_the_fp32_formula(engine, dtype, rows, D):
    """logos_layer_norm: biased variance in a second pass, fp32 arithmetic, one rounding to the 16-bit type
    (layernorm_kernel, cuda/VedicGEMM.cu:157-199)."""
    g = torch.Generator(device="cuda").manual_seed(rows * 3 + D)
    X = (torch.randn((rows, D), device="cuda", generator=g) * 3.0 + 0.5).to(dtype)
    gamma = torch.randn((D,), device="cuda", generator=g)
    beta = torch.randn((D,), device="cuda", generator=g)
    for overlap in (0, 1):
        engine.set_option(L.OPT_PROJECT_OVERLAP, overlap)
        try:
            Y = engine.layer_norm(X, gamma, beta, 1e-5)
        finally:
            engine.set_option(L.OPT_PROJECT_OVERLAP, 0)
        engine.synchronize()
        x = X.double()
        mean = x.mean(dim=1, keepdim=True)
        var = ((x - mean) ** 2).mean(dim=1, keepdim=True)
        want = (gamma.double() * ((x - mean) / torch.sqrt(var + 1e-5)) + beta.double()).float()
        ulp = want.abs() * (2.0 ** -8 if dtype == torch.bfloat16 else 2.0 ** -11) + 1e-4
        assert bool(((Y.float() - want).abs() <= ulp).all()), float((Y.float() - want).abs().max())
