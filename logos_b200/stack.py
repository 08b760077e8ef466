"""The attention stack of the LOGOS model over the engine, with an incremental generate loop.

What the reference does per layer (ModelGPU::forward, cuda/ModelGPU.cu:876-1061): LayerNorm, then per
head Q/K/V projections, Nikhilam quantisation of the raw K and V (:908), the Navier-Stokes prologue,
attention (Shunyam whenever seq > window, :966), head_out·W_O[h] summed over heads, W_proj and the
residual add.  Generation (generate_feynman, cuda/train_gpu.cu:2020-2084) re-runs that whole forward
over the whole context for every beam and every new token.

Here the same layer is five calls into the engine -- one fused Q/K/V GEMM whose epilogue also leaves the
per-tensor max|x| for the quantiser, the two cache quantisations, the attention, and two projection
GEMMs -- and generation is prefill once, then per token one append + decode step per layer straight
from the INT8 cache; beams share the prompt's cache rows.  With several GPUs each rank projects and
attends over its own heads and the per-head outputs are gathered through the engine's peer exchange.

Out of scope, as in the rest of this package: the feed-forward half of the block, training, the
tokenizer.  LayerNorm, the embedding lookup and the host-side beam bookkeeping are plain torch / numpy.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import numpy as np
import torch
import torch.nn.functional as F

from . import lib as L
from .engine import Comm, Engine
from .kvcache import KVCache
from .sharding import head_range


@dataclass
class StackConfig:
    """Field names follow GPUModelConfig / GPUPhysicsConfig (cuda/ModelGPU.cuh:52-82)."""
    vocab_size: int = 8192
    d_model: int = 1024
    num_heads: int = 16
    num_layers: int = 16
    max_seq_len: int = 2176
    shunyam: bool = True
    window: int = 64
    stride: int = 16
    navier_stokes: bool = True
    ns_eta: float = 0.1
    ns_nu: float = 0.05


def make_weights(cfg: StackConfig, seed: int = 5, std: float = 0.02, device="cuda") -> dict:
    """Random-init weights ~ N(0, std) in the reference's shapes: per layer and head W_Q, W_K, W_V
    [d, 64] and W_O [64, d]; per layer W_proj [d, d]; embedding and lm_head [V, d] / [d, V]."""
    g = torch.Generator(device="cpu").manual_seed(seed)
    Lr, H, D, V = cfg.num_layers, cfg.num_heads, cfg.d_model, cfg.vocab_size
    r = lambda *shape: (torch.randn(shape, generator=g) * std).to(device)
    return {"embed": r(V, D), "W_Q": r(Lr, H, D, 64), "W_K": r(Lr, H, D, 64), "W_V": r(Lr, H, D, 64),
            "W_O": r(Lr, H, 64, D), "W_proj": r(Lr, D, D), "lm_head": r(D, V),
            "ln_gamma": torch.ones((Lr, D), device=device), "ln_beta": torch.zeros((Lr, D), device=device)}


class AttentionStack:
    def __init__(self, engine: Engine, cfg: StackConfig, weights: dict, batch: int, rank: int = 0, world: int = 1,
                 comm: Comm | None = None, dtype=torch.bfloat16):
        self.eng, self.cfg, self.rank, self.world, self.comm, self.dtype = engine, cfg, rank, world, comm, dtype
        if world > 1 and comm is None:
            raise ValueError("several ranks need a connected Comm")
        H, D = cfg.num_heads, cfg.d_model
        self.lo, self.hi = head_range(H, rank, world)
        self.Hl = self.hi - self.lo
        w = weights
        sh = lambda t: t.to(dtype).contiguous()
        # K-major 16-bit shadows (the reference keeps an FP16 shadow of every weight, cuda/MixedPrecision.cuh:149-161)
        self.Wt_qkv = [sh(torch.cat([w[k][l, self.lo:self.hi].transpose(1, 2).reshape(self.Hl * 64, D)
                                     for k in ("W_Q", "W_K", "W_V")], dim=0)) for l in range(cfg.num_layers)]
        self.Wt_o = [sh(w["W_O"][l].reshape(H * 64, D).t()) for l in range(cfg.num_layers)]       # [D, H*64]
        self.Wt_proj = [sh(w["W_proj"][l].t()) for l in range(cfg.num_layers)]
        self.Wt_lm = sh(w["lm_head"].t())                                                          # [V, D]
        self.embed = w["embed"].to(dtype)
        self.ln_g, self.ln_b = w["ln_gamma"].float(), w["ln_beta"].float()
        self.ln_g16, self.ln_b16 = self.ln_g.to(dtype), self.ln_b.to(dtype)
        self.cache = KVCache(cfg.num_layers, batch, self.Hl, cfg.max_seq_len, 64, device=self.embed.device)
        self.q_prev = torch.zeros((cfg.num_layers, batch, self.Hl, 64), dtype=torch.float16, device=self.embed.device)
        # a decode step's Q, K, V of every layer: the queries become q_prev in one copy at the end of the step
        self.qkv_step = torch.empty((cfg.num_layers, 3, batch, self.Hl, 1, 64), dtype=torch.float16, device=self.embed.device)
        self.batch = batch
        engine.reserve(engine.decode_workspace_bytes(batch, self.Hl, cfg.max_seq_len, 64))
        ns = cfg.navier_stokes
        self.params = L.Params.make(1.0 / math.sqrt(64.0), True, cfg.window if cfg.shunyam else 0, cfg.stride,
                                    cfg.ns_eta if ns else 0.0, cfg.ns_nu if ns else 0.0, 1.0 if ns else 0.0,
                                    L.DIFFUSE_CAUSAL if ns else L.DIFFUSE_NONE)
        self.times = {}

    # ---- pieces ------------------------------------------------------------------------------
    def _norm(self, X, l):
        # one kernel: 16-bit in and out, fp32 statistics inside
        if self.cfg.d_model <= 2048 and self.cfg.d_model % 8 == 0:
            return self.eng.layer_norm(X, self.ln_g[l], self.ln_b[l], 1e-5)
        return F.layer_norm(X, (self.cfg.d_model,), self.ln_g16[l], self.ln_b16[l], 1e-5)

    def _gather(self, local, shape_tail):
        """[B, H_loc, ...] -> [B, H, ...] on every rank."""
        if self.world == 1:
            return local
        out = torch.empty((local.shape[0], self.cfg.num_heads) + tuple(shape_tail), dtype=local.dtype, device=local.device)
        return self.comm.all_gather_heads(local.contiguous(), out)

    # ---- prefill -----------------------------------------------------------------------------
    def prefill(self, ids: torch.Tensor) -> torch.Tensor:
        """ids [B, S] -> logits of the last position [B, V]; fills cache slots [0, B) of every layer
        (B may be smaller than the cache's batch: beams then copy a slot with KVCache.share_prompt)."""
        B, S = ids.shape
        cfg, eng = self.cfg, self.eng
        assert B <= self.batch and S <= cfg.max_seq_len
        X = self.embed[ids.reshape(-1)]                                    # [B*S, D]
        for l in range(cfg.num_layers):
            Xn = self._norm(X, l)
            Q, K, V, ka, va = eng.qkv_project(Xn, self.Wt_qkv[l], B, S, self.Hl, absmax=True)
            kc, vc, ks, vs = self.cache.layer(l)
            ks[:B].copy_(eng.nikhilam_compress_absmax(K, ka, kc[:B].view(B * self.Hl, cfg.max_seq_len, 64)))
            vs[:B].copy_(eng.nikhilam_compress_absmax(V, va, vc[:B].view(B * self.Hl, cfg.max_seq_len, 64)))
            O = eng.attention(Q, K, V, self.params)                        # [B, H_loc, S, 64]
            self.q_prev[l, :B].copy_(Q[:, :, S - 1].half())
            O = self._gather(O, (S, 64))
            Y = eng.project_heads(O.contiguous(), self.Wt_o[l])           # head-major operand: nothing is permuted
            X = eng.project(Y, self.Wt_proj[l], residual=X)
        self.cache.set_lens(S)
        last = X.view(B, S, cfg.d_model)[:, S - 1]
        return eng.project(last.contiguous(), self.Wt_lm, out_dtype=torch.float32)

    # ---- one generated token -------------------------------------------------------------------
    def decode(self, ids: torch.Tensor) -> torch.Tensor:
        """ids [B] (the newest token of every sequence) -> logits [B, V]; the cache grows by one row."""
        cfg, eng, B = self.cfg, self.eng, self.batch
        x = self.embed[ids]                                                # [B, D]
        self.cache.advance(1)                                              # lens = length after the append
        lens = self.cache.lens
        # the weights are never written during generation: the small projections may fetch them while the kernel
        # before them still runs
        eng.set_option(L.OPT_PROJECT_OVERLAP, 1)
        try:
            return self._decode_layers(x, lens)
        finally:
            eng.set_option(L.OPT_PROJECT_OVERLAP, 0)

    def _decode_layers(self, x, lens):
        cfg, eng, B = self.cfg, self.eng, self.batch
        for l in range(cfg.num_layers):
            xn = self._norm(x, l)
            # the decode entry points take FP16: the projection's epilogue stores Q, K, V in that type
            q, k, v = eng.qkv_project(xn, self.Wt_qkv[l], B, 1, self.Hl, as_block=True, out_f16=True,
                                      out=self.qkv_step[l]).view(3, B, self.Hl, 64).unbind(0)
            kc, vc, ks, vs = self.cache.layer(l)
            if self.world == 1:      # the rows come out in the projections' type
                o = eng.decode_step(q, self.q_prev[l], k, v, kc, vc, ks, vs, lens, self.params, out_dtype=self.dtype)
            else:
                o = eng.decode_step(q, self.q_prev[l], k, v, kc, vc, ks, vs, lens, self.params, comm=self.comm)
            a = o.view(B, cfg.num_heads * 64).to(self.dtype)
            y = eng.project(a, self.Wt_o[l])
            x = eng.project(y, self.Wt_proj[l], residual=x)
        logits = eng.project(x, self.Wt_lm, out_dtype=torch.float32)
        self.q_prev.copy_(self.qkv_step[:, 0, :, :, 0])
        return logits


    def capture_decode(self, greedy: bool = False):
        """Record one decode step (all layers) into a CUDA graph.  Returns (graph, ids, logits): fill `ids`
        ([B] int64) in place, replay, read `logits`.  With `greedy` the graph ends by writing the arg-max token of
        every sequence back into `ids`, so a greedy loop is replay after replay with nothing between them.  No library
        collective is captured: with several ranks the gather inside the step is the engine's own peer exchange."""
        ids = torch.zeros((self.batch,), dtype=torch.long, device=self.embed.device)
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        self.eng.use_stream(side)
        try:
            with torch.cuda.stream(side):
                lens0 = self.cache.lens.clone()
                qp0 = self.q_prev.clone()
                self.decode(ids)                      # warm-up: every lazy set-up happens before the capture
                side.synchronize()
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph, stream=side, capture_error_mode="thread_local"):
                    logits = self.decode(ids)
                    if greedy:
                        ids.copy_(logits.argmax(dim=1))
                self.cache.lens.copy_(lens0)          # the warm-up step is taken back
                self.q_prev.copy_(qp0)
        finally:
            self.eng.use_stream(torch.cuda.current_stream())
        torch.cuda.current_stream().wait_stream(side)
        self.eng.set_option(L.OPT_WORKSPACE_LOCK, 1)
        return graph, ids, logits


# ---- generation: the reference's beam search on top of prefill + decode ------------------------------

@dataclass
class FeynmanBeam:
    """cuda/train_gpu.cu:2013-2017."""
    tokens: list
    log_amplitude: float = 0.0
    action: float = 0.0


def _expand(logits_row: np.ndarray, top_k: int):
    """Host softmax and top-k of one beam's logits, as at cuda/train_gpu.cu:2050-2065."""
    p = np.exp(logits_row - logits_row.max())
    p = p / (p.sum() + 1e-9)
    idx = np.argsort(-p, kind="stable")[:top_k]
    return [(int(t), float(p[t])) for t in idx if p[t] >= 1e-10]


def generate_feynman(stack: AttentionStack, prompt_ids, max_new=64, beam_width=4, hbar=1.0, top_k_expand=50,
                     eos_token=1):
    """generate_feynman (cuda/train_gpu.cu:2020-2084) with incremental decode: the prompt is prefilled once,
    its cache rows are shared by all beams, and every new token costs one decode step per layer instead of
    a forward over the whole context.  The stack's batch must be `beam_width`.  Returns the beams sorted by
    log amplitude."""
    V = stack.cfg.vocab_size
    beam_width = max(1, min(beam_width, 32))
    top_k_expand = max(1, min(top_k_expand, V))
    hbar = max(0.01, hbar)
    assert stack.batch == beam_width, "one cache slot per beam"
    dev = stack.embed.device
    prompt = list(prompt_ids)
    logits = stack.prefill(torch.tensor([prompt], dtype=torch.long, device=dev))  # once, into slot 0 ...
    if beam_width > 1:                                                             # ... which every beam shares
        stack.cache.share_prompt(0, range(1, beam_width))
        stack.q_prev[:, 1:] = stack.q_prev[:, :1]
    logits = logits.expand(beam_width, V)
    beams = [FeynmanBeam(list(prompt))]
    slots = [0]                                     # cache slot of each live beam
    for s in range(max_new):
        host = logits.float().cpu().numpy()
        cands = []                                  # (beam, parent slot)
        for beam, slot in zip(beams, slots):
            if beam.tokens and beam.tokens[-1] == eos_token and s > 0:
                cands.append((beam, slot))
                continue
            for tok, p in _expand(host[slot], top_k_expand):
                dS = -math.log(p + 1e-10)
                cands.append((FeynmanBeam(beam.tokens + [tok], beam.log_amplitude - dS / hbar, beam.action + dS), slot))
        cands.sort(key=lambda c: -c[0].log_amplitude)
        cands = cands[:beam_width]
        beams = [c[0] for c in cands]
        parents = [c[1] for c in cands] + [0] * (beam_width - len(cands))
        if all(b.tokens and b.tokens[-1] == eos_token for b in beams) or s == max_new - 1:
            break
        # every surviving beam takes a cache slot; a slot whose parent is another slot gets its rows
        if parents != list(range(beam_width)):
            idx = torch.tensor(parents, dtype=torch.long, device=dev)
            n = int(stack.cache.lens.max())
            stack.cache.k[:, :, :, :n] = stack.cache.k[:, idx][:, :, :, :n]
            stack.cache.v[:, :, :, :n] = stack.cache.v[:, idx][:, :, :, :n]
            stack.cache.ks.copy_(stack.cache.ks[:, idx])
            stack.cache.vs.copy_(stack.cache.vs[:, idx])
            stack.q_prev.copy_(stack.q_prev[:, idx])
        slots = list(range(len(beams)))
        newest = [b.tokens[-1] for b in beams] + [0] * (beam_width - len(beams))
        logits = stack.decode(torch.tensor(newest, dtype=torch.long, device=dev))
    return sorted(beams, key=lambda b: -b.log_amplitude)
