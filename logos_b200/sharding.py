"""(batch x head) partition of the attention path over the GPUs of one node.

Every (sequence, head) pair is independent in all kernels and the INT8 cache is per
(sequence, head), so the H heads are cut into contiguous blocks, one block per rank;
each rank owns its heads' cache and scales for all sequences.  The only exchange is an
all-gather of the attention outputs along the head axis (NCCL over NVLink/NVSwitch on
GPUs, gloo in CPU tests).  The single-GPU result is the parity reference: the N-GPU
result must be bit-identical per head.
"""
from __future__ import annotations

import torch
import torch.distributed as dist


def head_range(H: int, rank: int, world: int) -> tuple[int, int]:
    """Contiguous block of heads owned by `rank`; world must divide H (H=16: 16/8/4/2)."""
    if world <= 0 or rank < 0 or rank >= world:
        raise ValueError(f"bad rank {rank} of {world}")
    if H % world != 0:
        raise ValueError(f"{world} ranks do not divide {H} heads")
    per = H // world
    return rank * per, (rank + 1) * per


def shard_heads(x: torch.Tensor, rank: int, world: int, head_dim: int = 1) -> torch.Tensor:
    """The slice of a [B, H, ...] tensor that `rank` owns (a contiguous copy)."""
    lo, hi = head_range(x.shape[head_dim], rank, world)
    return x.narrow(head_dim, lo, hi - lo).contiguous()


def all_gather_heads(local: torch.Tensor, world: int, group=None) -> torch.Tensor:
    """[B, H_loc, ...] on every rank -> [B, H, ...] on every rank (head axis = 1)."""
    if world == 1:
        return local
    local = local.contiguous()
    flat = torch.empty((world * local.shape[0],) + tuple(local.shape[1:]), dtype=local.dtype,
                       device=local.device)
    dist.all_gather_into_tensor(flat, local, group=group)
    # rows [r*B, (r+1)*B) are rank r's [B, H_loc, ...]; interleave back along the head axis
    parts = flat.view((world,) + tuple(local.shape))
    return parts.movedim(0, 1).reshape(local.shape[0], world * local.shape[1], *local.shape[2:])


class ShardedDecoder:
    """Decode steps over this rank's heads of an INT8 KV cache, outputs all-gathered.

    The cache tensors ([B, H_loc, S_max, DH] int8) and scales ([B, H_loc]) live on the
    device for the lifetime of the object, like HeadCache in the reference
    (cuda/ModelGPU.cuh:42-49)."""

    def __init__(self, engine, k_cache, v_cache, k_scale, v_scale, params, rank=0, world=1, group=None):
        self.eng, self.params = engine, params
        self.kc, self.vc, self.ks, self.vs = k_cache, v_cache, k_scale, v_scale
        self.rank, self.world, self.group = rank, world, group
        B, Hl, S_max, DH = k_cache.shape
        self.shape = (B, Hl, S_max, DH)
        engine.reserve(engine.decode_workspace_bytes(B, Hl, S_max, DH))
        dev = k_cache.device
        self.out_local = torch.empty((B, Hl, DH), dtype=torch.float32, device=dev)
        self.pos = torch.empty((B,), dtype=torch.int32, device=dev)
        if world > 1:
            self._stage = [torch.empty((B, Hl, DH), dtype=torch.float16, device=dev) for _ in range(4)]
            self._lens = torch.empty((B,), dtype=torch.int32, device=dev)

    def step(self, q, q_prev, k_new, v_new, lens):
        """Device tensors in (this rank's heads), gathered [B, H, DH] fp32 out.
        lens[b] = context length after the append."""
        torch.sub(lens, 1, out=self.pos)
        self.eng.kv_append(k_new, v_new, self.kc, self.vc, self.ks, self.vs, self.pos)
        self.eng.decode_int8(q, q_prev, self.kc, self.vc, self.ks, self.vs, lens, self.params, out=self.out_local)
        return all_gather_heads(self.out_local, self.world, self.group)

    def capture(self, q, q_prev, k_new, v_new, lens):
        """Record one step over these tensors (append, decode, all-gather) into a CUDA graph.

        A decode step is a handful of short launches; at several GPUs per job each rank's share
        of the work takes less time than the host needs to issue it, so the step is replayed as
        one graph launch.  The tensors are the graph's inputs: refill them in place between
        replays.  Returns the gathered output tensor that every replay writes."""
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        self.eng.use_stream(side)
        try:
            with torch.cuda.stream(side):
                for _ in range(3):                      # warm-up on the side stream before the capture
                    self.step(q, q_prev, k_new, v_new, lens)
                side.synchronize()
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph, stream=side):
                    gathered = self.step(q, q_prev, k_new, v_new, lens)
        finally:
            self.eng.use_stream(torch.cuda.current_stream())
        torch.cuda.current_stream().wait_stream(side)
        self.graph, self.graph_out = graph, gathered
        return gathered

    def replay(self):
        """Launch the captured step on the current stream; returns the gathered output tensor."""
        self.graph.replay()
        return self.graph_out

    def step_host(self, q, q_prev, k_new, v_new, lens, out):
        """Pinned HOST tensors in (this rank's heads) and out ([B, H, DH] fp32, pinned host)."""
        if self.world == 1:
            return self.eng.decode_step_host(q, q_prev, k_new, v_new, self.kc, self.vc, self.ks, self.vs,
                                             lens, self.params, out)
        for dst, src in zip(self._stage, (q, q_prev, k_new, v_new)):
            dst.copy_(src, non_blocking=True)
        self._lens.copy_(lens, non_blocking=True)
        full = self.step(*self._stage, self._lens)
        out.copy_(full, non_blocking=True)
        torch.cuda.current_stream().synchronize()
        return out
