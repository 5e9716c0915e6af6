"""Host-side logic of the sequence-sharded decode on CPU: partitioning, partial layout, the gather and the merge
plumbing, with world_size-2 `gloo` ranks. The CPU oracle stands in for the kernels (compute is not under test
here; tests/test_sharded_gpu.py covers it on the device)."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from argus_engine_b200.sharded import ShardedDecoder, shard_range
from oracle import oracle as orc


def test_shard_range_partitions_exactly():
    for T, N, align in [(1048576, 8, 1), (1000, 3, 1), (5, 8, 1), (32768, 4, 128), (1000, 4, 128), (0, 2, 1)]:
        spans = [shard_range(T, N, r, align) for r in range(N)]
        assert spans[0][0] == 0 and spans[-1][1] == T
        for (a0, a1), (b0, b1) in zip(spans[:-1], spans[1:]):
            assert a1 == b0 and a0 <= a1
            assert a1 % align == 0 or a1 == T


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, T, hq, hkv, d, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    rng = np.random.default_rng(0)                      # every rank draws the same full problem
    q = rng.standard_normal((hq, d), dtype=np.float32)
    k = rng.standard_normal((hkv, T, d), dtype=np.float32)
    v = rng.standard_normal((hkv, T, d), dtype=np.float32)
    lo, hi = shard_range(T, world, rank)
    g = hq // hkv

    def partial_fn(q_t, part):
        n = hi - lo
        if n == 0:
            part[:hq * d] = 0
            part[hq * d:] = float("-inf")
            return
        o, _ = orc.attention_gen(q_t.numpy(), np.ascontiguousarray(k[:, lo:hi]), np.ascontiguousarray(v[:, lo:hi]), hq, hkv,
                                 d, n)
        s = np.einsum("htd,hgd->hgt", k[:, lo:hi].astype(np.float64), q.reshape(hkv, g, d).astype(np.float64)) / np.sqrt(d)
        lse = np.log(np.exp(s - s.max(-1, keepdims=True)).sum(-1)) + s.max(-1)
        part[:hq * d] = torch.from_numpy(o.reshape(-1))
        part[hq * d:] = torch.from_numpy(lse.reshape(-1).astype(np.float32))

    def merge_fn(parts, out):
        pn = parts.numpy()
        for h in range(hq):
            out[h] = torch.from_numpy(orc.lse_merge(pn[:, h * d:(h + 1) * d], pn[:, hq * d + h]))

    dec = ShardedDecoder(hq, d, partial_fn, merge_fn, torch.device("cpu"))
    out = torch.zeros(hq, d)
    dec.step(torch.from_numpy(q), out)
    want, _ = orc.attention_gen(q, k, v, hq, hkv, d, T)
    ret[rank] = float(np.max(np.abs(out.numpy() - want)))
    dist.destroy_process_group()


@pytest.mark.parametrize("T", [1000, 1])   # T=1: the second rank holds an empty shard
def test_two_rank_gloo_matches_unsharded(T):
    world = 2
    ctx = mp.get_context("spawn")
    ret = ctx.Manager().dict()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, T, 8, 2, 32, ret)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    assert len(ret) == world and max(ret.values()) < 1e-5
