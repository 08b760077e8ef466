"""(batch x head) partition of the attention path over the GPUs of one node.

Every (sequence, head) pair is independent in all kernels and the INT8 cache is per
(sequence, head), so the H heads are cut into contiguous blocks, one block per rank;
each rank owns its heads' cache and scales for all sequences.  The only exchange is an
all-gather of the attention outputs along the head axis.  Two ways to do it:

  "peer"  the engine's own exchange (logos_comm): the decode kernel's epilogue stores each
          finished row into every rank's staging memory over NVLink and a second short kernel
          waits for all ranks and copies the slot out -- no library collective in the step;
  "nccl"  torch.distributed all_gather_into_tensor (NCCL on GPUs, gloo in CPU tests) into a
          preallocated rank-major buffer; the parity reference for "peer".

The single-GPU result is the parity reference for both: with the same split size
(LOGOS_OPT_DECODE_CHUNK) the N-GPU result is bit-identical per head.
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


def check_slices(local: torch.Tensor, world: int, group=None) -> None:
    """Every rank must bring a slice of the same shape and dtype; a rank that does not is named
    in a ValueError on every rank BEFORE any data collective is entered (a mismatched
    all-gather would otherwise hang or corrupt memory)."""
    if world == 1:
        return
    mine = (tuple(local.shape), str(local.dtype))
    seen = [None] * world
    dist.all_gather_object(seen, mine, group=group)
    bad = [r for r, s in enumerate(seen) if s != seen[0]]
    if bad:
        raise ValueError(f"head slices differ between ranks: rank 0 has {seen[0]}, rank(s) {bad} have "
                         f"{[seen[r] for r in bad]}")


def all_gather_heads(local: torch.Tensor, world: int, group=None, flat: torch.Tensor | None = None,
                     out: torch.Tensor | None = None) -> torch.Tensor:
    """[B, H_loc, ...] on every rank -> [B, H, ...] on every rank (head axis = 1).

    The collective fills a rank-major buffer `flat` ([world, B, H_loc, ...]); for B > 1 that is not
    the head-major layout, so one strided copy moves it into `out` ([B, H, ...]).  Both buffers may be
    passed in preallocated, so that a step allocates nothing."""
    if world == 1:
        return local
    local = local.contiguous()
    B, Hl = local.shape[:2]
    if flat is None:
        flat = torch.empty((world,) + tuple(local.shape), dtype=local.dtype, device=local.device)
    dist.all_gather_into_tensor(flat.view((world * B,) + tuple(local.shape[1:])), local, group=group)
    if out is None:
        out = torch.empty((B, world * Hl) + tuple(local.shape[2:]), dtype=local.dtype, device=local.device)
    out.view((B, world, Hl) + tuple(local.shape[2:])).copy_(flat.movedim(0, 1))
    return out


def connect_comm(comm, group=None) -> None:
    """Exchange the ranks' block handles over the process group and map the peers' blocks."""
    handles = [None] * comm.world
    dist.all_gather_object(handles, comm.handle(), group=group)
    comm.connect(handles)


class ShardedDecoder:
    """Decode steps over this rank's heads of an INT8 KV cache, outputs gathered on every rank.

    The cache tensors ([B, H_loc, S_max, DH] int8) and scales ([B, H_loc]) live on the
    device for the lifetime of the object, like HeadCache in the reference
    (cuda/ModelGPU.cuh:42-49).  `gather` is "peer" or "nccl" (module docstring); with one rank
    there is nothing to gather."""

    def __init__(self, engine, k_cache, v_cache, k_scale, v_scale, params, rank=0, world=1, group=None,
                 gather="peer", comm=None):
        if gather not in ("peer", "nccl"):
            raise ValueError(f"gather must be 'peer' or 'nccl', got {gather!r}")
        self.eng, self.params = engine, params
        self.kc, self.vc, self.ks, self.vs = k_cache, v_cache, k_scale, v_scale
        self.rank, self.world, self.group = rank, world, group
        self.gather = gather if world > 1 else "none"
        B, Hl, S_max, DH = k_cache.shape
        self.shape = (B, Hl, S_max, DH)
        engine.reserve(engine.decode_workspace_bytes(B, Hl, S_max, DH))
        dev = k_cache.device
        self.out_local = torch.empty((B, Hl, DH), dtype=torch.float32, device=dev)
        self.graph = None
        self.comm, self._own_comm = comm, False
        if self.gather == "peer":
            self.gathered = torch.empty((B, Hl * world, DH), dtype=torch.float32, device=dev)
            if comm is None:
                from .engine import Comm
                self.comm, self._own_comm = Comm(engine, rank, world, self.gathered.numel() * 4), True
                connect_comm(self.comm, group)
        elif self.gather == "nccl":
            self._flat = torch.empty((world, B, Hl, DH), dtype=torch.float32, device=dev)
            self.gathered = torch.empty((B, Hl * world, DH), dtype=torch.float32, device=dev)
        if world > 1:
            self._stage = [torch.empty((B, Hl, DH), dtype=torch.float16, device=dev) for _ in range(4)]
            self._lens = torch.empty((B,), dtype=torch.int32, device=dev)

    # ---- one step ---------------------------------------------------------------------
    def _local_step(self, q, q_prev, k_new, v_new, lens):
        """Append and decode on this rank; with the peer exchange the rows leave from the kernel."""
        if self.gather == "peer":
            self.eng.decode_step(q, q_prev, k_new, v_new, self.kc, self.vc, self.ks, self.vs, lens, self.params,
                                 out=self.gathered, comm=self.comm)
        else:
            self.eng.decode_step(q, q_prev, k_new, v_new, self.kc, self.vc, self.ks, self.vs, lens, self.params,
                                 out=self.out_local)

    def _finish(self):
        if self.gather == "peer":
            return self.gathered
        if self.gather == "nccl":
            return all_gather_heads(self.out_local, self.world, self.group, flat=self._flat, out=self.gathered)
        return self.out_local

    def step(self, q, q_prev, k_new, v_new, lens):
        """Device tensors in (this rank's heads), gathered [B, H, DH] fp32 out.
        lens[b] = context length after the append."""
        self._local_step(q, q_prev, k_new, v_new, lens)
        return self._finish()

    # ---- the step as a CUDA graph -------------------------------------------------------
    def capture(self, q, q_prev, k_new, v_new, lens):
        """Record one step over these tensors into a CUDA graph: append, decode and -- with the peer
        exchange -- the wait-and-copy kernel.  A library collective is never captured: with "nccl"
        the graph ends after the decode and replay() issues the all-gather eagerly behind it.
        (A graph that holds NCCL work keeps the communicator busy for as long as the graph lives;
        destroying the process group with such a graph alive does not return.)

        A decode step is a handful of short launches; with the work spread over several GPUs a
        rank's share takes less time than the host needs to issue it, so the step is replayed as
        one graph launch.  The tensors are the graph's inputs: refill them in place between replays.
        The graph holds the address of the context's workspace, so the workspace is locked against
        replacement until release()."""
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        self.eng.use_stream(side)
        try:
            with torch.cuda.stream(side):
                for _ in range(3):                      # warm-up on the side stream before the capture
                    self._local_step(q, q_prev, k_new, v_new, lens)
                side.synchronize()
                graph = torch.cuda.CUDAGraph()
                # thread-local mode: calls made by other threads of the process (a collective
                # library's watchdog, an allocator) do not invalidate this thread's capture
                with torch.cuda.graph(graph, stream=side, capture_error_mode="thread_local"):
                    self._local_step(q, q_prev, k_new, v_new, lens)
        finally:
            self.eng.use_stream(torch.cuda.current_stream())
        torch.cuda.current_stream().wait_stream(side)
        self.graph = graph
        self.eng.set_option(_opt().OPT_WORKSPACE_LOCK, 1)
        return self._finish() if self.gather != "nccl" else None

    def replay(self):
        """Launch the captured step on the current stream; returns the gathered output tensor."""
        self.graph.replay()
        return self._finish()

    def release(self):
        """Drop the captured graph (and unlock the workspace).  Call this on every decoder, and
        synchronise, before the process group or the engine goes away."""
        if self.graph is not None:
            torch.cuda.synchronize()
            self.graph.reset()
            self.graph = None
            self.eng.set_option(_opt().OPT_WORKSPACE_LOCK, 0)

    def close(self):
        self.release()
        if self._own_comm and self.comm is not None:
            torch.cuda.synchronize()
            self.comm.close()
            self.comm = None

    # ---- host buffers --------------------------------------------------------------------
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


def _opt():
    from . import lib
    return lib
