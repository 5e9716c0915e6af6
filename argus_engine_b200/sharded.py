"""Long-context decode sharded by KV sequence across the GPUs of one node.

Rank r of N owns the contiguous token range ``shard_range(T, N, r)`` as its own HeadMajor ``[Hkv, T_r, D]``
K/V buffers; q is replicated. One decode step per rank = the split-KV kernel over the local slice writing
``(o, lse)`` into one buffer, ONE all-gather of that buffer (Hq*(D+1) floats per rank), and a local merge.
There is no other communication. The reference has no multi-device mode; the algebra is its CPU chunk merge
(engine/src/backend/cpu/neon.rs:1028-1125).

The compute and merge steps are injected (``partial_fn`` / ``merge_fn``) so that the host-side logic —
partitioning, buffer layout, the gather — also runs under the ``gloo`` backend on CPU in the tests, where the
CPU oracle stands in for the kernels. The package itself ships no CPU implementation of either.
"""
from __future__ import annotations

from typing import Callable, Optional, Tuple

import torch
import torch.distributed as dist


def shard_range(total_tokens: int, world: int, rank: int, align: int = 1) -> Tuple[int, int]:
    """Contiguous token range of `rank`. Shard boundaries are multiples of `align` (the KIVI flush size when the
    cache is packed: whole flushes stay on one rank, the residual ring ends up on the last); the last rank
    takes the remainder. Ranks past the end get an empty range."""
    per = -(-total_tokens // world)
    per = -(-per // align) * align
    lo = min(rank * per, total_tokens)
    hi = min(lo + per, total_tokens) if rank < world - 1 else total_tokens
    return lo, max(lo, hi)


class ShardedDecoder:
    """One per rank. ``partial_fn(q, part)`` must fill ``part[:Hq*D]`` with the normalised local outputs and
    ``part[Hq*D:]`` with the natural-log lse per query head (-inf for an empty shard); ``merge_fn(parts, out)``
    merges ``parts [N, Hq*D+Hq]`` into ``out [Hq, D]``."""

    def __init__(self, num_heads_q: int, head_dim: int, partial_fn: Callable, merge_fn: Callable,
                 device: torch.device, group: Optional[dist.ProcessGroup] = None):
        self.hq, self.d = num_heads_q, head_dim
        self.partial_fn, self.merge_fn = partial_fn, merge_fn
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.part_len = num_heads_q * head_dim + num_heads_q
        self.part = torch.zeros(self.part_len, dtype=torch.float32, device=device)
        self.parts = torch.zeros(self.world, self.part_len, dtype=torch.float32, device=device)
        self.fused_step_fn = None   # set by make_gpu_decoder(..., fused=True): replaces the whole step

    def capture(self, q: torch.Tensor, out: torch.Tensor):
        """Record one step (kernel, gather, merge) on static tensors into a CUDA graph and return it; replaying it
        removes the host launch cost, which at 8 GPUs is larger than the device time of a step. Returns None when
        the capture is not possible (the caller keeps calling step())."""
        try:
            self.step(q, out)                      # warm-up outside the capture (lazy initialisation, NCCL setup)
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                self.step(q, out)
            return g
        except Exception:
            torch.cuda.synchronize()
            return None

    def step(self, q: torch.Tensor, out: torch.Tensor) -> None:
        if self.fused_step_fn is not None:   # decode, peer push, wait and merge in one launch
            self.fused_step_fn(q, out)
            return
        self.partial_fn(q, self.part)
        if self.world > 1:
            dist.all_gather_into_tensor(self.parts.view(-1), self.part, group=self.group)
        else:
            self.parts[0].copy_(self.part)
        self.merge_fn(self.parts, out)


class PeerBuffers:
    """Receive buffers of the in-kernel exchange, in memory every rank of the node can address (torch symmetric memory
    over NVLink). Per rank: two sets (even / odd steps) of [N][Hkv][lines_per_head] 16-byte units (128-byte lines of 30
    data words and the step number twice), zero-initialised; see argus_b200_attention_gen_sharded in the C header."""

    def __init__(self, be, num_heads_q: int, num_heads_kv: int, head_dim: int, group=None):
        import torch.distributed._symmetric_memory as symm_mem

        group = group or dist.group.WORLD
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        lph = be.exchange_lines_per_head(num_heads_q, num_heads_kv, head_dim)
        self.parity_stride_lines = self.world * num_heads_kv * lph
        n_words = 2 * self.parity_stride_lines * 4
        self.buf = symm_mem.empty(n_words, dtype=torch.int32, device=torch.device("cuda", torch.cuda.current_device()))
        self.buf.zero_()
        self.handle = symm_mem.rendezvous(self.buf, group.group_name)
        torch.cuda.synchronize()
        dist.barrier(group)
        self.peer_lines = [int(p) for p in self.handle.buffer_ptrs]


def make_gpu_decoder(be, k_shard: torch.Tensor, v_shard: torch.Tensor, shard_len: int, num_heads_q: int,
                     num_heads_kv: int, head_dim: int, group=None, fused=False) -> ShardedDecoder:
    """ShardedDecoder over the CUDA kernels of `be` (a B200Backend) for an F16 HeadMajor shard.
    fused=False: decode kernel, ONE NCCL all-gather into each rank's own memory, merge kernel.
    fused=True: ONE launch per step (argus_b200_attention_gen_sharded): the CTA of the decode kernel that completes a
    KV head stores the head group's (o, lse) rows into every rank's receive buffer over NVLink peer pointers, collects
    (bounded) the other ranks' rows of those heads and merges them. The step number lives in device memory."""
    from .backend import DecodeExtras

    hq, d = num_heads_q, head_dim

    def partial_fn(q, part):
        ex = DecodeExtras(lse=part[hq * d:])
        be.attention_gen(q, k_shard, v_shard, part[:hq * d], hq, num_heads_kv, d, shard_len, extras=ex)

    def merge_fn(parts, out):
        be.lse_merge(parts, hq, d, out)

    dec = ShardedDecoder(hq, d, partial_fn, merge_fn, k_shard.device, group)
    if fused and dec.world > 1:
        peers = PeerBuffers(be, hq, num_heads_kv, d, group)
        counters = torch.zeros(num_heads_kv, dtype=torch.int32, device=k_shard.device)

        def fused_step_fn(q, out):
            be.attention_gen_sharded(q, k_shard, v_shard, out, hq, num_heads_kv, d, shard_len, peers.peer_lines, peers.rank,
                                     counters, peers.parity_stride_lines)

        dec.fused_step_fn = fused_step_fn
        dec._peers = peers   # keep the symmetric allocation alive
        dec._counters = counters
    return dec
