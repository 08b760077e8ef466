"""Host-side mirror of the reference's attention classes over the engine.

`MultiHeadAttention.forward(X)` is `Tensor MultiHeadAttention::forward(const Tensor&)` of LOGOS
(include/Attention.hpp:290-300; per head AttentionHead::forward, :218-267): per-head projections,
the attention with its Navier-Stokes prologue, masks, softmax and blend, W_O, the first d_k columns
of each head side by side, W_proj -- optionally with K and V passed through the Nikhilam INT8
quantiser (cuda/ModelGPU.cu:908).  Every step runs in the engine: `forward` is the fp32 form
(logos_mha_forward_f32: fp32 FMA GEMMs and the fp32 attention kernel), `forward16` the BF16 / FP16
form on the tensor cores (logos_mha_forward; d_k = 64).  torch only owns the memory.
"""
from __future__ import annotations

import ctypes as C
import math

import torch

from . import lib as L
from .engine import Engine, _ptr


class MultiHeadAttention:
    """Field names follow AttentionHead / MultiHeadAttention (include/Attention.hpp:190-288)."""

    def __init__(self, engine: Engine, W_Q, W_K, W_V, W_O, W_proj, *, use_sparse=True, sparse_window=8,
                 sparse_stride=4, use_navier_stokes=False, ns_alpha=0.3, ns_eta=0.1, ns_nu=0.05,
                 diffuse_mode=L.DIFFUSE_CENTRAL, kv_int8=False):
        self.eng = engine
        # [H, d, dk] x3, [H, dk, d], [d, d]: fp32, row-major, as Tensor stores them
        self.W_Q, self.W_K, self.W_V, self.W_O, self.W_proj = (w.contiguous().float() for w in (W_Q, W_K, W_V, W_O, W_proj))
        self.num_heads, self.d_model, self.d_k = W_Q.shape[0], W_Q.shape[1], W_Q.shape[2]
        self.use_sparse, self.sparse_window, self.sparse_stride = use_sparse, sparse_window, sparse_stride
        self.use_navier_stokes, self.ns_alpha, self.ns_eta, self.ns_nu = use_navier_stokes, ns_alpha, ns_eta, ns_nu
        self.diffuse_mode, self.kv_int8 = diffuse_mode, kv_int8
        self._shadows = {}

    def params(self) -> L.Params:
        ns = self.use_navier_stokes and self.ns_alpha > 0.0
        return L.Params.make(1.0 / math.sqrt(self.d_k), True, self.sparse_window if self.use_sparse else 0,
                             self.sparse_stride, self.ns_eta if ns else 0.0, self.ns_nu if ns else 0.0,
                             self.ns_alpha if ns else 0.0, self.diffuse_mode if ns else L.DIFFUSE_NONE)

    def forward(self, X: torch.Tensor) -> torch.Tensor:
        """X: [seq, d_model] fp32 on the GPU -> [seq, d_model] fp32."""
        eng, seq = self.eng, X.shape[0]
        X = X.contiguous().float()
        out = torch.empty((seq, self.d_model), dtype=torch.float32, device=X.device)
        need = eng.lib.logos_mha_f32_workspace_bytes(seq, self.d_model, self.num_heads)
        scratch = torch.empty(need, dtype=torch.uint8, device=X.device)
        p = self.params()
        eng._check(eng.lib.logos_mha_forward_f32(eng.h, _ptr(X), _ptr(self.W_Q), _ptr(self.W_K), _ptr(self.W_V),
                                                 _ptr(self.W_O), _ptr(self.W_proj), _ptr(out), seq, self.d_model,
                                                 self.num_heads, C.byref(p), int(self.kv_int8), _ptr(scratch), need))
        return out

    # ---- 16-bit form ---------------------------------------------------------------------------
    def shadows(self, dtype):
        """K-major 16-bit shadows of the weights, made once (the reference keeps an FP16 shadow of every
        parameter, cuda/MixedPrecision.cuh:149-161): Wt_qkv[(which H + h) 64 + c][k] = W_which[h][k][c];
        Wt_o[h 64 + j][h 64 + c] = W_O[h][c][j] for j < 64 (block diagonal: the columns the class keeps);
        Wt_proj[n][k] = W_proj[k][n]."""
        if dtype not in self._shadows:
            H, d, dk = self.num_heads, self.d_model, self.d_k
            assert dk == 64, "the tensor-core projections take d_k = 64"
            qkv = torch.stack([self.W_Q, self.W_K, self.W_V])                         # [3, H, d, dk]
            Wt_qkv = qkv.permute(0, 1, 3, 2).reshape(3 * H * dk, d)
            Wt_o = torch.zeros((d, H * dk), dtype=torch.float32, device=self.W_O.device)
            for h in range(H):
                Wt_o[h * dk:(h + 1) * dk, h * dk:(h + 1) * dk] = self.W_O[h][:, :dk].t()
            Wt_proj = self.W_proj.t()
            self._shadows[dtype] = tuple(w.contiguous().to(dtype) for w in (Wt_qkv, Wt_o, Wt_proj))
        return self._shadows[dtype]

    def forward16(self, X: torch.Tensor, dtype=torch.bfloat16) -> torch.Tensor:
        """X: [seq, d_model] -> [seq, d_model] fp32, operands and intermediates in `dtype`, fp32 accumulation."""
        seq = X.shape[0]
        Wt_qkv, Wt_o, Wt_proj = self.shadows(dtype)
        caches = None
        if self.kv_int8:
            H = self.num_heads
            caches = (torch.empty((1, H, seq, 64), dtype=torch.int8, device=X.device),
                      torch.empty((1, H, seq, 64), dtype=torch.int8, device=X.device),
                      torch.empty((1, H), dtype=torch.float32, device=X.device),
                      torch.empty((1, H), dtype=torch.float32, device=X.device))
        return self.eng.mha_forward(X.contiguous().to(dtype), Wt_qkv, Wt_o, Wt_proj, 1, seq, self.num_heads,
                                    self.params(), out_dtype=torch.float32, caches=caches,
                                    attend_dequantized=self.kv_int8)
