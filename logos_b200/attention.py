"""Host-side mirror of the reference's attention classes over the engine.

`MultiHeadAttention.forward(X)` follows include/Attention.hpp:290-300 of LOGOS (per-head
projections, attention, W_O, keep the first d_k columns of each head, W_proj) with the
attention itself -- Navier-Stokes prologue, masks, softmax, PV, and optionally the Nikhilam
INT8 round trip of K and V (cuda/ModelGPU.cu:908) -- done by the engine's kernels.  The
projections are plain fp32 library GEMMs (torch.matmul); they are not part of the engine.
"""
from __future__ import annotations

import math

import torch

from . import lib as L
from .engine import Engine


class MultiHeadAttention:
    """Field names follow AttentionHead / MultiHeadAttention (include/Attention.hpp:190-288)."""

    def __init__(self, engine: Engine, W_Q, W_K, W_V, W_O, W_proj, *, use_sparse=True, sparse_window=8,
                 sparse_stride=4, use_navier_stokes=False, ns_alpha=0.3, ns_eta=0.1, ns_nu=0.05,
                 diffuse_mode=L.DIFFUSE_CENTRAL, kv_int8=False):
        self.eng = engine
        self.W_Q, self.W_K, self.W_V, self.W_O, self.W_proj = W_Q, W_K, W_V, W_O, W_proj   # [H,d,dk] x3, [H,dk,d], [d,d]
        self.num_heads, self.d_model, self.d_k = W_Q.shape[0], W_Q.shape[1], W_Q.shape[2]
        self.use_sparse, self.sparse_window, self.sparse_stride = use_sparse, sparse_window, sparse_stride
        self.use_navier_stokes, self.ns_alpha, self.ns_eta, self.ns_nu = use_navier_stokes, ns_alpha, ns_eta, ns_nu
        self.diffuse_mode, self.kv_int8 = diffuse_mode, kv_int8

    def params(self) -> L.Params:
        ns = self.use_navier_stokes and self.ns_alpha > 0.0
        return L.Params.make(1.0 / math.sqrt(self.d_k), True, self.sparse_window if self.use_sparse else 0,
                             self.sparse_stride, self.ns_eta if ns else 0.0, self.ns_nu if ns else 0.0,
                             self.ns_alpha if ns else 0.0, self.diffuse_mode if ns else L.DIFFUSE_NONE)

    def forward(self, X: torch.Tensor) -> torch.Tensor:
        """X: [seq, d_model] fp32 on the GPU -> [seq, d_model]."""
        seq = X.shape[0]
        Q = torch.matmul(X, self.W_Q)          # [H, seq, dk]
        K = torch.matmul(X, self.W_K)
        V = torch.matmul(X, self.W_V)
        if self.kv_int8:                       # raw K and V through the INT8 cache, as at ModelGPU.cu:908
            kq, ks = self.eng.nikhilam_compress(K)
            vq, vs = self.eng.nikhilam_compress(V)
            K, V = self.eng.nikhilam_decompress(kq, ks), self.eng.nikhilam_decompress(vq, vs)
        head_out = self.eng.attention(Q[None].contiguous(), K[None].contiguous(), V[None].contiguous(),
                                      self.params())[0]                      # [H, seq, dk]
        proj = torch.matmul(head_out, self.W_O)                               # [H, seq, d_model]
        concat = proj[:, :, :self.d_k].permute(1, 0, 2).reshape(seq, self.d_model)   # first dk columns of each head
        return torch.matmul(concat, self.W_proj)
