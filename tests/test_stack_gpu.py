"""The attention stack (logos_b200/stack.py): layers made of the engine's projection, quantisation and
attention calls against a numpy / oracle composition of the same steps, the incremental decode step
against the oracle's decode over the same INT8 cache, and the generate loop's bookkeeping."""
import math

import numpy as np
import pytest
import torch

import oracle as O
from logos_b200 import lib as L
from logos_b200 import synthetic as syn
from logos_b200.stack import AttentionStack, StackConfig, generate_feynman, make_weights
from helpers import assert_close

pytestmark = pytest.mark.gpu

CFG = StackConfig(vocab_size=192, d_model=128, num_heads=2, num_layers=2, max_seq_len=160, window=16, stride=4)
bf = syn.bf16_round


def _ln(x):
    x = x.astype(np.float64)
    return ((x - x.mean(-1, keepdims=True)) / np.sqrt(x.var(-1, keepdims=True) + 1e-5)).astype(np.float32)


def _oracle_prefill(w, ids, cfg):
    """The same layer steps in numpy, with a BF16 rounding wherever the device stores BF16."""
    B, S = ids.shape
    H, D = cfg.num_heads, cfg.d_model
    f = lambda t: bf(t.float().cpu().numpy())
    X = f(w["embed"])[ids.reshape(-1)]
    op = O.attn_params(0.125, True, cfg.window, cfg.stride, cfg.ns_eta, cfg.ns_nu, 1.0, O.DIFFUSE_CAUSAL)
    caches = []
    for l in range(cfg.num_layers):
        Xn = bf(_ln(X))
        proj = lambda W: bf(np.einsum("md,hdc->hmc", Xn.astype(np.float64), f(W[l]).astype(np.float64)).astype(np.float32))
        Q, K, V = (proj(w[k]).reshape(H, B, S, 64).transpose(1, 0, 2, 3) for k in ("W_Q", "W_K", "W_V"))
        caches.append((K.copy(), V.copy(), Q[:, :, S - 1].copy()))
        Oa = bf(O.attention_batched(Q, K, V, op))                                     # [B, H, S, 64]
        A = Oa.transpose(0, 2, 1, 3).reshape(B * S, H * 64)
        Y = bf((A.astype(np.float64) @ f(w["W_O"][l]).reshape(H * 64, D).astype(np.float64)).astype(np.float32))
        X = bf((Y.astype(np.float64) @ f(w["W_proj"][l]).astype(np.float64)).astype(np.float32) + X)
    last = X.reshape(B, S, D)[:, S - 1]
    return (last.astype(np.float64) @ f(w["lm_head"]).astype(np.float64)).astype(np.float32), X, caches


def test_prefill_layers_match_the_oracle_composition(engine):
    w = make_weights(CFG, seed=3, std=0.08)
    B, S = 2, 96
    ids = torch.from_numpy(np.random.default_rng(1).integers(0, CFG.vocab_size, (B, S))).cuda()
    st = AttentionStack(engine, CFG, w, batch=B)
    logits = st.prefill(ids)
    engine.synchronize()
    want, _, caches = _oracle_prefill(w, ids.cpu().numpy(), CFG)
    # BF16 storage between the steps: every stored tensor is within one BF16 rounding of the oracle's
    assert_close(logits.cpu().numpy(), want, "prefill logits", max_abs=3e-2, rel_l2=1e-2)
    # the cache holds the Nikhilam quantisation of the raw K and V of every layer
    for l, (K, V, _) in enumerate(caches):
        kc, vc, ks, vs = st.cache.layer(l)
        for b in range(B):
            for h in range(CFG.num_heads):
                q_o, s_o = O.nikhilam_compress(K[b, h])
                got = kc[b, h, :S].cpu().numpy().astype(np.int32)
                # K on the device may differ from the oracle's by one BF16 step in a few entries; the
                # quantised bytes then differ by at most one level there
                assert np.abs(got - q_o.astype(np.int32)).max() <= 1
                assert abs(float(ks[b, h]) - float(s_o)) <= 1e-2 * float(s_o)


def test_decode_step_matches_oracle_over_the_same_cache(engine):
    w = make_weights(CFG, seed=4, std=0.08)
    B, S = 3, 70
    rng = np.random.default_rng(2)
    ids = torch.from_numpy(rng.integers(0, CFG.vocab_size, (B, S))).cuda()
    st = AttentionStack(engine, CFG, w, batch=B)
    st.prefill(ids)
    new = torch.from_numpy(rng.integers(0, CFG.vocab_size, (B,))).cuda()
    # what the device holds before the step: caches, scales, previous queries
    before = [(st.cache.k[l].cpu().numpy().copy(), st.cache.v[l].cpu().numpy().copy(), st.cache.ks[l].cpu().numpy().copy(),
               st.cache.vs[l].cpu().numpy().copy(), st.q_prev[l].float().cpu().numpy().copy()) for l in range(CFG.num_layers)]
    logits = st.decode(new)
    engine.synchronize()
    H, D = CFG.num_heads, CFG.d_model
    f = lambda t: bf(t.float().cpu().numpy())
    f16 = lambda a: a.astype(np.float16).astype(np.float32)
    x = f(w["embed"])[new.cpu().numpy()]
    op = O.attn_params(0.125, True, CFG.window, CFG.stride, CFG.ns_eta, CFG.ns_nu, 1.0, O.DIFFUSE_CAUSAL)
    for l in range(CFG.num_layers):
        kc, vc, ks, vs, qp = before[l]
        xn = bf(_ln(x))
        proj = lambda W: f16(bf(np.einsum("md,hdc->mhc", xn.astype(np.float64), f(W[l]).astype(np.float64)).astype(np.float32)))
        q, k, v = proj(w["W_Q"]), proj(w["W_K"]), proj(w["W_V"])                    # [B, H, 64]
        for b in range(B):
            for h in range(H):
                kc[b, h, S] = O.nikhilam_quantize(k[b, h], ks[b, h])
                vc[b, h, S] = O.nikhilam_quantize(v[b, h], vs[b, h])
        n = B * H
        o = O.decode_int8_batch(q.reshape(n, 64), qp.reshape(n, 64), kc.reshape(n, -1, 64), vc.reshape(n, -1, 64),
                                ks.reshape(n), vs.reshape(n), np.full(n, S + 1, np.int32), op).reshape(B, H * 64)
        y = bf((bf(o).astype(np.float64) @ f(w["W_O"][l]).reshape(H * 64, D).astype(np.float64)).astype(np.float32))
        x = bf((y.astype(np.float64) @ f(w["W_proj"][l]).astype(np.float64)).astype(np.float32) + x)
        # the appended rows are in the device cache, bit for bit (same FP16 values, same scales)
        got_k = st.cache.k[l][:, :, S].cpu().numpy().astype(np.int32)
        assert np.abs(got_k - kc[:, :, S].astype(np.int32)).max() <= 1
    want = (x.astype(np.float64) @ f(w["lm_head"]).astype(np.float64)).astype(np.float32)
    assert_close(logits.cpu().numpy(), want, "decode logits", max_abs=3e-2, rel_l2=1e-2)
    assert int(st.cache.lens[0]) == S + 1


def test_generate_loop_bookkeeping(engine):
    w = make_weights(CFG, seed=6, std=0.08)
    prompt = list(np.random.default_rng(3).integers(2, CFG.vocab_size, 40))
    # greedy: one beam, one expansion -> the tokens of a hand-written prefill + argmax + decode loop
    st = AttentionStack(engine, CFG, w, batch=1)
    out = generate_feynman(st, prompt, max_new=6, beam_width=1, top_k_expand=1, eos_token=-1)
    st2 = AttentionStack(engine, CFG, w, batch=1)
    logits = st2.prefill(torch.tensor([prompt], device="cuda"))
    toks = []
    for _ in range(6):
        t = int(logits[0].argmax())
        toks.append(t)
        logits = st2.decode(torch.tensor([t], device="cuda"))
    assert out[0].tokens == prompt + toks
    # four beams: sorted by amplitude, consistent action, all beams extend the prompt
    st4 = AttentionStack(engine, CFG, w, batch=4)
    beams = generate_feynman(st4, prompt, max_new=5, beam_width=4, hbar=0.7, top_k_expand=8, eos_token=-1)
    assert len(beams) == 4 and all(b.tokens[:len(prompt)] == prompt and len(b.tokens) == len(prompt) + 5 for b in beams)
    amps = [b.log_amplitude for b in beams]
    assert amps == sorted(amps, reverse=True)
    assert all(math.isclose(b.log_amplitude, -b.action / 0.7, rel_tol=1e-5, abs_tol=1e-6) for b in beams)
    assert len({tuple(b.tokens) for b in beams}) == 4


def test_captured_decode_step_replays_the_eager_steps(engine):
    """capture_decode: the whole step as one CUDA graph gives the eager step's logits, step after step; with
    greedy=True the graph feeds its own arg-max tokens back and reproduces the eager greedy loop."""
    w = make_weights(CFG, seed=9, std=0.3)
    g = torch.Generator(device="cuda").manual_seed(9)
    ids = torch.randint(0, CFG.vocab_size, (3, 40), device="cuda", generator=g)
    eager = AttentionStack(engine, CFG, w, batch=3)
    first = eager.prefill(ids).argmax(dim=1)
    tok, want_logits, want_tokens = first.clone(), [], []
    for _ in range(5):
        lg = eager.decode(tok)
        tok = lg.argmax(dim=1)
        want_logits.append(lg.clone())
        want_tokens.append(tok.clone())
    st = AttentionStack(engine, CFG, w, batch=3)
    st.prefill(ids)
    graph, gids, glogits = st.capture_decode(greedy=True)
    try:
        gids.copy_(first)
        for k in range(5):
            graph.replay()
            torch.cuda.synchronize()
            assert torch.equal(glogits, want_logits[k])
            assert torch.equal(gids, want_tokens[k])
    finally:
        graph.reset()
        engine.set_option(L.OPT_WORKSPACE_LOCK, 0)
