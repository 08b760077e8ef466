"""Torch-tensor front ends over the C ABI.

Torch is plumbing here: it owns device memory and streams; every operation below
is one call into liblogos_attn.so.  Names follow the reference: `MultiHeadAttention`
-style forward on [B,H,S,DH] tensors, `nikhilam_compress` / `nikhilam_decompress`,
`kv_append`, `decode_int8`.
"""
from __future__ import annotations

import ctypes as C

import torch

from . import lib as L

_DT = {torch.float32: L.F32, torch.bfloat16: L.BF16, torch.float16: L.F16}


def _ptr(t):
    return C.c_void_p(t.data_ptr()) if t is not None else C.c_void_p(0)


class Engine:
    """One context per process and GPU (logos_ctx)."""

    def __init__(self, device: int | None = None):
        self.lib = L.load_library()
        if not torch.cuda.is_available():
            raise L.LogosError(L.ERR_NO_DEVICE, "no CUDA device: the engine has no CPU path")
        self.device = torch.cuda.current_device() if device is None else int(device)
        h = C.c_void_p()
        self._check(self.lib.logos_ctx_create(self.device, C.byref(h)), None)
        self.h = h
        self.use_stream(torch.cuda.current_stream(self.device))

    def close(self):
        if getattr(self, "h", None):
            self.lib.logos_ctx_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def _check(self, rc, h="self"):
        if rc != L.OK:
            msg = self.lib.logos_status_string(rc).decode()
            if h == "self" and getattr(self, "h", None):
                msg += ": " + self.lib.logos_last_error(self.h).decode()
            raise L.LogosError(rc, msg)

    def use_stream(self, stream: torch.cuda.Stream):
        self._check(self.lib.logos_ctx_set_stream(self.h, C.c_void_p(stream.cuda_stream)))

    def synchronize(self):
        """Waits for the stream; raises if a kernel reported that one of its internal waits ran out."""
        self._check(self.lib.logos_ctx_synchronize(self.h))

    def reserve(self, nbytes: int):
        self._check(self.lib.logos_ctx_reserve(self.h, int(nbytes)))

    def set_workspace(self, buf: torch.Tensor):
        """Caller-owned scratch (a uint8 tensor the caller keeps alive) instead of the context's own block:
        what a captured CUDA graph must use, because logos_ctx_reserve may free and replace its block."""
        self._check(self.lib.logos_ctx_set_workspace(self.h, _ptr(buf), buf.numel() * buf.element_size()))

    def set_option(self, option: int, value: int):
        self._check(self.lib.logos_ctx_set_option(self.h, int(option), int(value)))

    # ---- attention ---------------------------------------------------------
    def flash_attention_fwd_f32(self, Q, K, V, scale, causal=True, shunyam=False, window=0, stride=0):
        """cuda_flash_attention_fwd: one head, fp32 [seq, DH]."""
        seq, DH = Q.shape
        out = torch.empty_like(Q)
        self._check(self.lib.logos_flash_attention_fwd_f32(
            self.h, _ptr(Q), _ptr(K), _ptr(V), _ptr(out), None, seq, DH, float(scale), int(causal),
            int(shunyam), int(window), int(stride)))
        return out

    def attention(self, Q, K, V, params: L.Params, out_dtype=None, out=None):
        """Q,K,V: [B,H,S,DH] contiguous -> O [B,H,S,DH]."""
        B, H, S, DH = Q.shape
        assert Q.is_contiguous() and K.is_contiguous() and V.is_contiguous()
        out_dtype = out_dtype or Q.dtype
        if out is None:
            out = torch.empty((B, H, S, DH), dtype=out_dtype, device=Q.device)
        self._check(self.lib.logos_attention_fwd(self.h, _DT[Q.dtype], _DT[out.dtype], _ptr(Q), _ptr(K),
                                                _ptr(V), _ptr(out), B, H, S, DH, C.byref(params)))
        return out

    def attention_strided(self, Q, K, V, params: L.Params, out=None, out_dtype=None):
        """Q, K, V: views of shape [B, H, S, DH] with any batch / head / row strides (the last dimension
        contiguous, one layout for the three); `out`: such a view too, or None for a packed tensor."""
        B, H, S, DH = Q.shape
        assert Q.stride() == K.stride() == V.stride() and Q.stride(3) == 1
        if out is None:
            out = torch.empty((B, H, S, DH), dtype=out_dtype or Q.dtype, device=Q.device)
        assert out.shape == Q.shape and out.stride(3) == 1
        si = L.Strides(Q.stride(0), Q.stride(1), Q.stride(2))
        so = L.Strides(out.stride(0), out.stride(1), out.stride(2))
        self._check(self.lib.logos_attention_fwd_strided(self.h, _DT[Q.dtype], _DT[out.dtype], _ptr(Q), _ptr(K), _ptr(V),
                                                        _ptr(out), B, H, S, DH, C.byref(si), C.byref(so),
                                                        C.byref(params)))
        return out

    # ---- projections -----------------------------------------------------------
    def qkv_project(self, X, Wt_qkv, B, S, H, absmax=False, as_block=False, out_f16=False, out=None):
        """X: [B*S, D] 16-bit; Wt_qkv: [3*H*64, D] (K-major shadow of the stacked W_Q | W_K | W_V) ->
        Q, K, V [B, H, S, 64] (three slices of one block, so that they can be converted or moved as one) and,
        with absmax, the tables max|K|, max|V| [B, H] for the quantiser.  out_f16: Q, K, V come out as FP16
        whatever X is (LOGOS_OPT_QKV_OUT_F16: what the decode entry points take)."""
        D = X.shape[1]
        assert X.is_contiguous() and Wt_qkv.is_contiguous() and Wt_qkv.shape == (3 * H * 64, D) and X.shape[0] == B * S
        want = torch.float16 if out_f16 else X.dtype
        block = out if out is not None else torch.empty((3, B, H, S, 64), dtype=want, device=X.device)
        assert block.shape == (3, B, H, S, 64) and block.dtype == want and block.is_contiguous()
        Q, K, V = block.unbind(0)
        ka = torch.empty((B, H), dtype=torch.float32, device=X.device) if absmax else None
        va = torch.empty((B, H), dtype=torch.float32, device=X.device) if absmax else None
        if out_f16:
            self.set_option(L.OPT_QKV_OUT_F16, 1)
        try:
            self._check(self.lib.logos_qkv_project(self.h, _DT[X.dtype], _ptr(X), _ptr(Wt_qkv), _ptr(Q), _ptr(K), _ptr(V),
                                                  B, S, H, D, _ptr(ka), _ptr(va)))
        finally:
            if out_f16:
                self.set_option(L.OPT_QKV_OUT_F16, 0)
        if as_block:
            return (block, ka, va) if absmax else block
        return (Q, K, V, ka, va) if absmax else (Q, K, V)

    def layer_norm(self, X, gamma, beta, eps=1e-5):
        """X [rows, D] 16-bit, gamma / beta fp32 [D] -> LayerNorm(X) in X's dtype (logos_layer_norm)."""
        rows, D = X.shape
        assert X.is_contiguous() and gamma.dtype == torch.float32 and beta.dtype == torch.float32
        Y = torch.empty_like(X)
        self._check(self.lib.logos_layer_norm(self.h, _DT[X.dtype], _ptr(X), _ptr(gamma), _ptr(beta), _ptr(Y), rows, D,
                                             float(eps)))
        return Y

    def project(self, A, Wt, residual=None, out_dtype=None, out=None):
        """A: [M, K] 16-bit, Wt: [N, K] (K-major shadow of W [K, N]) -> A·W (+ residual) [M, N]."""
        M, K = A.shape
        N = Wt.shape[0]
        assert A.is_contiguous() and Wt.is_contiguous() and Wt.shape[1] == K
        out_dtype = out_dtype or A.dtype
        if out is None:
            out = torch.empty((M, N), dtype=out_dtype, device=A.device)
        if residual is not None:
            assert residual.dtype == out.dtype and residual.shape == out.shape and residual.is_contiguous()
        self._check(self.lib.logos_project(self.h, _DT[A.dtype], _DT[out.dtype], _ptr(A), _ptr(Wt), _ptr(residual),
                                          _ptr(out), M, N, K))
        return out

    def attention_bwd16(self, Q, K, V, dO, params: L.Params):
        """The gradients on the tensor cores: Q, K, V, dO BF16 or FP16 [B, H, S, 64] -> fp32 (dQ, dK, dV)."""
        B, H, S, DH = Q.shape
        for t in (Q, K, V, dO):
            assert t.dtype == Q.dtype and t.is_contiguous() and t.shape == Q.shape
        self.reserve(self.lib.logos_attention_bwd16_workspace_bytes(B, H, S, DH))
        dQ, dK, dV = (torch.empty(Q.shape, dtype=torch.float32, device=Q.device) for _ in range(3))
        self._check(self.lib.logos_attention_bwd16(self.h, _DT[Q.dtype], _ptr(Q), _ptr(K), _ptr(V), _ptr(dO), _ptr(dQ),
                                                  _ptr(dK), _ptr(dV), B, H, S, DH, C.byref(params)))
        return dQ, dK, dV

    def attention_bwd(self, Q, K, V, dO, params: L.Params):
        """Gradients (dQ, dK, dV) of attention(Q, K, V, params) for the output gradient dO; fp32 [B, H, S, DH]."""
        B, H, S, DH = Q.shape
        for t in (Q, K, V, dO):
            assert t.dtype == torch.float32 and t.is_contiguous() and t.shape == Q.shape
        self.reserve(self.lib.logos_attention_bwd_workspace_bytes(B, H, S, DH))
        dQ, dK, dV = (torch.empty_like(Q) for _ in range(3))
        self._check(self.lib.logos_attention_bwd(self.h, _ptr(Q), _ptr(K), _ptr(V), _ptr(dO), _ptr(dQ), _ptr(dK),
                                                _ptr(dV), B, H, S, DH, C.byref(params)))
        return dQ, dK, dV

    def project_heads(self, head_out, Wt_o, residual=None, out_dtype=None, out=None):
        """head_out: [B, H, S, 64] as the attention wrote it; Wt_o: [N, H*64] -> sum over heads of
        head_out[b, h] · W_O[h] (+ residual), [B*S, N].  No per-token concatenation is made."""
        B, H, S, DH = head_out.shape
        N = Wt_o.shape[0]
        assert DH == 64 and head_out.is_contiguous() and Wt_o.is_contiguous() and Wt_o.shape[1] == H * 64
        out_dtype = out_dtype or head_out.dtype
        if out is None:
            out = torch.empty((B * S, N), dtype=out_dtype, device=head_out.device)
        if residual is not None:
            assert residual.dtype == out.dtype and residual.shape == out.shape and residual.is_contiguous()
        self._check(self.lib.logos_project_heads(self.h, _DT[head_out.dtype], _DT[out.dtype], _ptr(head_out), _ptr(Wt_o),
                                                _ptr(residual), _ptr(out), B, S, H, N))
        return out

    def mha_forward(self, X, Wt_qkv, Wt_o, Wt_proj, B, S, H, params: L.Params, residual=None, out_dtype=None,
                    caches=None, attend_dequantized=False, scratch=None):
        """MultiHeadAttention::forward for all heads and sequences in one call (logos_mha_forward).
        X: [B*S, D] 16-bit; caches: (k_cache, v_cache, k_scale, v_scale) or None -> [B*S, D]."""
        D = X.shape[1]
        assert X.is_contiguous() and X.shape[0] == B * S and Wt_qkv.shape == (3 * H * 64, D)
        assert Wt_o.shape == (D, H * 64) and Wt_proj.shape == (D, D)
        assert Wt_qkv.is_contiguous() and Wt_o.is_contiguous() and Wt_proj.is_contiguous()
        out = torch.empty((B * S, D), dtype=out_dtype or X.dtype, device=X.device)
        if residual is not None:
            assert residual.dtype == out.dtype and residual.shape == out.shape and residual.is_contiguous()
        need = self.lib.logos_mha_workspace_bytes(B, S, H, D)
        if scratch is None:
            scratch = torch.empty(need, dtype=torch.uint8, device=X.device)
        kc, vc, ks, vs = caches if caches is not None else (None, None, None, None)
        S_max = kc.shape[-2] if kc is not None else 0
        self._check(self.lib.logos_mha_forward(self.h, _DT[X.dtype], _DT[out.dtype], _ptr(X), _ptr(Wt_qkv), _ptr(Wt_o),
                                              _ptr(Wt_proj), _ptr(residual), _ptr(out), B, S, H, D, C.byref(params),
                                              _ptr(kc), _ptr(vc), _ptr(ks), _ptr(vs), S_max,
                                              L.MHA_ATTEND_DEQUANTIZED if attend_dequantized else 0, _ptr(scratch),
                                              scratch.numel()))
        return out

    def nikhilam_decompress16(self, q, scales, dtype, rows=None):
        """q: [..., S_max, DH] int8, scales [...] -> BF16 / FP16 of rows [0, rows)."""
        S_max, DH = q.shape[-2:]
        rows = S_max if rows is None else rows
        n = q.numel() // (S_max * DH)
        out = torch.empty(q.shape[:-2] + (rows, DH), dtype=dtype, device=q.device)
        self._check(self.lib.logos_kv_dequantize16(self.h, _DT[dtype], _ptr(q), S_max * DH, _ptr(scales), _ptr(out),
                                                  rows * DH, n, rows * DH))
        return out

    def nikhilam_compress_absmax(self, x, absmax, cache):
        """nikhilam_compress of x ([n..., S, DH]) into `cache` ([n, S_max, DH]) when max|x| per tensor is known."""
        S, DH = x.shape[-2:]
        n = x.numel() // (S * DH)
        scales = torch.empty(x.shape[:-2], dtype=torch.float32, device=x.device)
        self._check(self.lib.logos_kv_quantize_absmax(self.h, _DT[x.dtype], _ptr(x), S * DH, _ptr(cache),
                                                     cache.shape[-2] * cache.shape[-1], _ptr(absmax), _ptr(scales), n,
                                                     S * DH))
        return scales

    # ---- Nikhilam INT8 KV ----------------------------------------------------
    def prefill(self, Q, K, V, params: L.Params, k_cache, v_cache, k_scale, v_scale, out_dtype=None, out=None):
        """One layer's prefill in one call: the raw K, V ([B,H,S,DH]) quantised into rows [0, S) of the
        INT8 caches ([B,H,S_max,DH]) with their scales ([B,H]), then the attention -> O [B,H,S,DH]."""
        B, H, S, DH = Q.shape
        assert Q.is_contiguous() and K.is_contiguous() and V.is_contiguous()
        assert k_cache.is_contiguous() and v_cache.is_contiguous() and tuple(k_cache.shape[:2]) == (B, H)
        out_dtype = out_dtype or Q.dtype
        if out is None:
            out = torch.empty((B, H, S, DH), dtype=out_dtype, device=Q.device)
        self._check(self.lib.logos_prefill_fwd(self.h, _DT[Q.dtype], _DT[out.dtype], _ptr(Q), _ptr(K), _ptr(V),
                                              _ptr(out), B, H, S, DH, C.byref(params), _ptr(k_cache), _ptr(v_cache),
                                              _ptr(k_scale), _ptr(v_scale), k_cache.shape[2]))
        return out

    def nikhilam_compress(self, x, cache=None, rows=None):
        """x: [..., S, DH] (any leading dims = independent tensors) -> (int8 like x, scales[...]).

        With `cache` ([n, S_max, DH] int8) the bytes go to rows [0, S) of each cache tensor."""
        S, DH = x.shape[-2:]
        n = x.numel() // (S * DH)
        x = x.contiguous()
        scales = torch.empty(x.shape[:-2], dtype=torch.float32, device=x.device)
        if cache is None:
            q = torch.empty(x.shape, dtype=torch.int8, device=x.device)
            dst_stride = S * DH
        else:
            q = cache
            dst_stride = cache.shape[-2] * cache.shape[-1]
        self._check(self.lib.logos_kv_quantize(self.h, _DT[x.dtype], _ptr(x), S * DH, _ptr(q), dst_stride,
                                              _ptr(scales), n, S * DH))
        return q, scales

    def nikhilam_decompress(self, q, scales, rows=None):
        """q: [..., S_max, DH] int8, scales [...] -> fp32 of rows [0, rows)."""
        S_max, DH = q.shape[-2:]
        rows = S_max if rows is None else rows
        n = q.numel() // (S_max * DH)
        out = torch.empty(q.shape[:-2] + (rows, DH), dtype=torch.float32, device=q.device)
        self._check(self.lib.logos_kv_dequantize(self.h, _ptr(q), S_max * DH, _ptr(scales), _ptr(out),
                                                rows * DH, n, rows * DH))
        return out

    def kv_append(self, k_new, v_new, k_cache, v_cache, k_scale, v_scale, pos):
        B, H, S_max, DH = k_cache.shape
        self._check(self.lib.logos_kv_append(self.h, _DT[k_new.dtype], _ptr(k_new), _ptr(v_new), _ptr(k_cache),
                                            _ptr(v_cache), _ptr(k_scale), _ptr(v_scale), _ptr(pos), B, H,
                                            S_max, DH))

    def decode_workspace_bytes(self, B, H, S_max, DH):
        return self.lib.logos_decode_workspace_bytes(B, H, S_max, DH)

    def decode_int8(self, q, q_prev, k_cache, v_cache, k_scale, v_scale, lens, params: L.Params, out=None):
        B, H, S_max, DH = k_cache.shape
        if out is None:
            out = torch.empty((B, H, DH), dtype=torch.float32, device=q.device)
        self._check(self.lib.logos_decode_int8(self.h, _ptr(q), _ptr(q_prev), _ptr(k_cache), _ptr(v_cache),
                                              _ptr(k_scale), _ptr(v_scale), _ptr(lens), B, H, S_max, DH,
                                              C.byref(params), _ptr(out)))
        return out

    def decode_step(self, q, q_prev, k_new, v_new, k_cache, v_cache, k_scale, v_scale, lens, params: L.Params,
                    out=None, comm: "Comm | None" = None, out_dtype=torch.float32):
        """Append the new token at row lens-1 and decode, device tensors throughout.  With `comm` the
        heads are this rank's share and `out` is the gathered [B, H_local * world, DH] tensor.  Without it the
        rows may be stored in a 16-bit out_dtype (the A operand of the projection that follows)."""
        B, H, S_max, DH = k_cache.shape
        if comm is None:
            if out is None:
                out = torch.empty((B, H, DH), dtype=out_dtype, device=q.device)
            if out.dtype == torch.float32:
                self._check(self.lib.logos_decode_step_int8(
                    self.h, _ptr(q), _ptr(q_prev), _ptr(k_new), _ptr(v_new), _ptr(k_cache), _ptr(v_cache), _ptr(k_scale),
                    _ptr(v_scale), _ptr(lens), B, H, S_max, DH, C.byref(params), _ptr(out)))
            else:
                self._check(self.lib.logos_decode_step_int8_to(
                    self.h, _ptr(q), _ptr(q_prev), _ptr(k_new), _ptr(v_new), _ptr(k_cache), _ptr(v_cache), _ptr(k_scale),
                    _ptr(v_scale), _ptr(lens), B, H, S_max, DH, C.byref(params), _DT[out.dtype], _ptr(out)))
        else:
            if out is None:
                out = torch.empty((B, H * comm.world, DH), dtype=torch.float32, device=q.device)
            self._check(self.lib.logos_decode_step_int8_gather(
                self.h, comm.h, _ptr(q), _ptr(q_prev), _ptr(k_new), _ptr(v_new), _ptr(k_cache), _ptr(v_cache),
                _ptr(k_scale), _ptr(v_scale), _ptr(lens), B, H, S_max, DH, C.byref(params), _ptr(out)))
        return out

    def decode_int8_push(self, comm: "Comm", q, q_prev, k_cache, v_cache, k_scale, v_scale, lens, params: L.Params):
        """Decode over this rank's heads; the rows go into every rank's staging slot (see Comm)."""
        B, H, S_max, DH = k_cache.shape
        self._check(self.lib.logos_decode_int8_push(self.h, comm.h, _ptr(q), _ptr(q_prev), _ptr(k_cache),
                                                   _ptr(v_cache), _ptr(k_scale), _ptr(v_scale), _ptr(lens), B, H,
                                                   S_max, DH, C.byref(params)))

    def decode_int8_collect(self, comm: "Comm", gathered: torch.Tensor):
        """Wait for every rank's rows of the step and write them to gathered ([B, H, DH] fp32)."""
        B, H, DH = gathered.shape
        self._check(self.lib.logos_decode_int8_collect(self.h, comm.h, _ptr(gathered), B, H, DH))

    def decode_step_host(self, q, q_prev, k_new, v_new, k_cache, v_cache, k_scale, v_scale, lens, params,
                         out):
        """All of q, q_prev, k_new, v_new, lens, out are HOST (ideally pinned) tensors."""
        B, H, S_max, DH = k_cache.shape
        self._check(self.lib.logos_decode_step_int8_host(
            self.h, _ptr(q), _ptr(q_prev), _ptr(k_new), _ptr(v_new), _ptr(k_cache), _ptr(v_cache),
            _ptr(k_scale), _ptr(v_scale), _ptr(lens), B, H, S_max, DH, C.byref(params), _ptr(out)))
        return out


class Comm:
    """One rank's end of the head all-gather over peer-mapped memory (logos_comm)."""

    def __init__(self, engine: Engine, rank: int, world: int, gathered_bytes: int):
        self.eng, self.rank, self.world = engine, rank, world
        h = C.c_void_p()
        engine._check(engine.lib.logos_comm_create(engine.h, rank, world, int(gathered_bytes), C.byref(h)))
        self.h = h

    def handle(self) -> bytes:
        buf = C.create_string_buffer(L.COMM_HANDLE_BYTES)
        self.eng._check(self.eng.lib.logos_comm_handle(self.h, buf))
        return buf.raw

    def connect(self, handles: list[bytes]):
        """handles[r] = rank r's handle() (one process per GPU; the entry of this rank is ignored)."""
        blob = b"".join(handles)
        assert len(blob) == self.world * L.COMM_HANDLE_BYTES
        self.eng._check(self.eng.lib.logos_comm_connect(self.h, blob))

    @staticmethod
    def connect_local(comms: list["Comm"]):
        """All ranks live in this process (several contexts, on one or on several GPUs)."""
        arr = (C.c_void_p * len(comms))(*[c.h for c in comms])
        rc = comms[0].eng.lib.logos_comm_connect_local(arr, len(comms))
        comms[0].eng._check(rc)

    def push(self, local: torch.Tensor):
        """local: [B, H_local, ...] contiguous, bytes per (b, h) row a multiple of 16."""
        B, Hl = local.shape[:2]
        row = local[0, 0].numel() * local.element_size()
        self.eng._check(self.eng.lib.logos_comm_push(self.eng.h, self.h, _ptr(local), B, Hl, row))

    def wait(self, gathered: torch.Tensor):
        self.eng._check(self.eng.lib.logos_comm_wait(self.eng.h, self.h, _ptr(gathered),
                                                     gathered.numel() * gathered.element_size()))

    def all_gather_heads(self, local: torch.Tensor, gathered: torch.Tensor):
        self.push(local)
        self.wait(gathered)
        return gathered

    def close(self):
        if getattr(self, "h", None):
            self.eng.lib.logos_comm_destroy(self.h)
            self.h = None
