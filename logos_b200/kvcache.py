"""Nikhilam INT8 KV cache of a whole model as one arena per kind.

The reference keeps one `NikhilamTensor {int8* data; float scale; int size}` per head and layer,
each with its own cudaMalloc (`HeadCache`, cuda/ModelGPU.cuh:15-49; filled at cuda/ModelGPU.cu:908,
freed and re-made every forward).  Here all layers, sequences and heads share two arenas

    k, v      int8    [L][B][H][S_max][DH]      a (layer, sequence, head) tensor is contiguous
    ks, vs    float32 [L][B][H]                 NikhilamTensor::scale of that tensor
    lens      int32   [B]                       tokens held per sequence (the same in every layer)

so a layer's slice is exactly the `[B][H][S_max][DH]` + `[B][H]` layout the engine's kernels take,
nothing is allocated after construction, and the whole cache goes to disk and back as one file.
At 16 layers x 32 sequences x 16 heads x 2176 tokens x 64 channels the arenas hold 2.28 GB.

File format (little endian): 8 bytes magic "LOGOSKV1", 8 x int64 {L, B, H, S_max, DH, S_used, 0, 0},
lens int32 [B], ks, vs float32 [L][B][H], then k and v as int8 [L][B][H][S_used][DH] -- only the rows
in use travel, S_used = max(lens).
"""
from __future__ import annotations

import struct

import numpy as np
import torch

MAGIC = b"LOGOSKV1"


class KVCache:
    def __init__(self, layers: int, batch: int, heads: int, s_max: int, dh: int, device="cuda"):
        if min(layers, batch, heads, s_max, dh) <= 0:
            raise ValueError("KVCache: every extent must be positive")
        if dh % 16 != 0:
            raise ValueError("KVCache: DH must be a multiple of 16 (rows are 16-byte vectors)")
        self.shape = (layers, batch, heads, s_max, dh)
        self.k = torch.zeros(self.shape, dtype=torch.int8, device=device)
        self.v = torch.zeros(self.shape, dtype=torch.int8, device=device)
        self.ks = torch.zeros((layers, batch, heads), dtype=torch.float32, device=device)
        self.vs = torch.zeros((layers, batch, heads), dtype=torch.float32, device=device)
        self.lens = torch.zeros((batch,), dtype=torch.int32, device=device)

    # ---- views --------------------------------------------------------------------
    def layer(self, l: int):
        """(k, v, ks, vs) of layer l: [B][H][S_max][DH] int8 x2 and [B][H] float32 x2, no copies."""
        return self.k[l], self.v[l], self.ks[l], self.vs[l]

    def nbytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in (self.k, self.v, self.ks, self.vs, self.lens))

    # ---- filling (through the engine's kernels) --------------------------------------
    def fill(self, engine, l: int, K: torch.Tensor, V: torch.Tensor):
        """Quantise a prompt's raw K and V ([B][H][S][DH], before diffusion, as at ModelGPU.cu:908)
        into rows [0, S) of layer l and set that layer's scales.  Call set_lens(S) once per prompt."""
        L_, B, H, S_max, DH = self.shape
        if K.shape != V.shape or tuple(K.shape[:2]) != (B, H) or K.shape[3] != DH or K.shape[2] > S_max:
            raise ValueError(f"KVCache.fill: K/V {tuple(K.shape)} do not fit {self.shape}")
        kc, vc, ks, vs = self.layer(l)
        _, s = engine.nikhilam_compress(K, cache=kc.view(B * H, S_max, DH))
        ks.copy_(s)
        _, s = engine.nikhilam_compress(V, cache=vc.view(B * H, S_max, DH))
        vs.copy_(s)

    def set_lens(self, n):
        if isinstance(n, int):
            self.lens.fill_(n)
        else:
            self.lens.copy_(torch.as_tensor(n, dtype=torch.int32))

    def append(self, engine, l: int, k_new: torch.Tensor, v_new: torch.Tensor):
        """One new token's K and V rows ([B][H][DH]) at position lens[b] of layer l, with the stored
        scales (saturating).  Call advance() after the last layer."""
        kc, vc, ks, vs = self.layer(l)
        engine.kv_append(k_new, v_new, kc, vc, ks, vs, self.lens)

    def advance(self, n: int = 1):
        self.lens.add_(n)

    def share_prompt(self, src: int, dst):
        """Copy sequence `src` (all layers, its rows in use and its scales) to the sequences in
        `dst`: beams that start from one prompt (cuda/train_gpu.cu:2020-2084 re-runs the prompt
        for each of them)."""
        n = int(self.lens[src])
        for d in dst:
            self.k[:, d, :, :n].copy_(self.k[:, src, :, :n])
            self.v[:, d, :, :n].copy_(self.v[:, src, :, :n])
            self.ks[:, d].copy_(self.ks[:, src])
            self.vs[:, d].copy_(self.vs[:, src])
            self.lens[d] = n

    # ---- disk -----------------------------------------------------------------------
    def dump(self, path: str):
        L_, B, H, S_max, DH = self.shape
        lens = self.lens.cpu().numpy().astype("<i4")
        s_used = int(lens.max()) if B else 0
        with open(path, "wb") as f:
            f.write(MAGIC)
            f.write(struct.pack("<8q", L_, B, H, S_max, DH, s_used, 0, 0))
            f.write(lens.tobytes())
            f.write(self.ks.cpu().numpy().astype("<f4").tobytes())
            f.write(self.vs.cpu().numpy().astype("<f4").tobytes())
            f.write(self.k[:, :, :, :s_used].contiguous().cpu().numpy().tobytes())
            f.write(self.v[:, :, :, :s_used].contiguous().cpu().numpy().tobytes())

    @classmethod
    def load(cls, path: str, device="cuda", s_max: int | None = None) -> "KVCache":
        with open(path, "rb") as f:
            if f.read(8) != MAGIC:
                raise ValueError(f"{path}: not a LOGOS KV cache file")
            L_, B, H, S_file, DH, s_used, _, _ = struct.unpack("<8q", f.read(64))
            S_max = S_file if s_max is None else s_max
            if s_used > S_max:
                raise ValueError(f"{path}: holds {s_used} rows per tensor, the cache only {S_max}")
            c = cls(L_, B, H, S_max, DH, device=device)
            c.lens.copy_(torch.from_numpy(np.frombuffer(f.read(4 * B), dtype="<i4").copy()))
            n = L_ * B * H
            c.ks.copy_(torch.from_numpy(np.frombuffer(f.read(4 * n), dtype="<f4").copy()).view(L_, B, H))
            c.vs.copy_(torch.from_numpy(np.frombuffer(f.read(4 * n), dtype="<f4").copy()).view(L_, B, H))
            rows = n * s_used * DH
            for arena in (c.k, c.v):
                buf = f.read(rows)
                if len(buf) != rows:
                    raise ValueError(f"{path}: truncated")
                arena[:, :, :, :s_used].copy_(torch.from_numpy(np.frombuffer(buf, dtype=np.int8).copy())
                                              .view(L_, B, H, s_used, DH))
        return c
