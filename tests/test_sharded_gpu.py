"""Sequence-sharded decode on the device: per-rank (o, lse) partials from the split-KV kernel and the merge
kernel against the unsharded oracle. With one GPU the ranks are emulated one after the other in this process
(same kernels, gather by copy); with two or more GPUs a real two-process NCCL run is added."""
import os
import socket
import subprocess
import sys

import numpy as np
import pytest
import torch

from argus_engine_b200 import workloads as wl
from argus_engine_b200.sharded import shard_range
from oracle import oracle as orc

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("T,N", [(20000, 4), (300, 8), (3, 4)])
def test_virtual_ranks_match_unsharded_oracle(T, N):
    from argus_engine_b200 import B200Backend, DecodeExtras

    hq, hkv, d = 64, 8, 128                      # the Llama-3-70B attention shape of the long-context workload
    case = wl.decode_case(4, [T], hq, hkv, d)
    be = B200Backend(0)
    q = torch.from_numpy(case.q[0]).cuda()
    parts = torch.zeros(N, hq * d + hq, device="cuda")
    for r in range(N):
        lo, hi = shard_range(T, N, r)
        k = torch.from_numpy(np.ascontiguousarray(case.k[0][:, lo:hi])).cuda()
        v = torch.from_numpy(np.ascontiguousarray(case.v[0][:, lo:hi])).cuda()
        be.attention_gen(q, k, v, parts[r, :hq * d], hq, hkv, d, hi - lo, extras=DecodeExtras(lse=parts[r, hq * d:]))
    out = torch.zeros(hq, d, device="cuda")
    lse = torch.zeros(hq, device="cuda")
    be.lse_merge(parts, hq, d, out, lse)
    torch.cuda.synchronize()
    want, _ = orc.attention_gen(case.q[0], case.k[0].view(np.uint16), case.v[0].view(np.uint16), hq, hkv, d, T)
    np.testing.assert_allclose(out.cpu().numpy(), want, atol=2e-3, rtol=1e-2)
    if T < N:   # some ranks were empty: their lse is -inf and they were skipped
        assert np.isneginf(parts[-1, hq * d:].cpu().numpy()).all()
    be.close()


def _line_buffers(be, n_ranks, hq, hkv, d):
    """One receive buffer per (virtual) rank: two sets of [n_ranks][Hkv][lines_per_head] 16-byte units, zeroed."""
    lph = be.exchange_lines_per_head(hq, hkv, d)
    stride = n_ranks * hkv * lph
    bufs = [torch.zeros(2 * stride * 4, dtype=torch.int32, device="cuda") for _ in range(n_ranks)]
    return bufs, [b.data_ptr() for b in bufs], stride


@pytest.mark.parametrize("T,N,hq", [(20000, 4, 64), (300, 8, 64), (3, 2, 64), (5000, 3, 8)])
def test_decode_with_in_kernel_push_virtual_ranks(T, N, hq):
    """The single-launch sharded step with all ranks' buffers on one GPU. Every virtual rank runs the decode kernel over
    its slice with the peer push in its epilogue (phase 1: the head groups' rows travel as flagged 128-byte lines into
    slot r of every rank's receive buffer, the step counters are bumped on the device); then every rank collects and
    merges with the stand-alone kernel (phase 2), so no kernel waits for a later launch. Three steps use both buffer
    sets and reuse one. hq = 8 gives one query head per KV head (an odd number of floats per head group). Against the
    unsharded oracle."""
    from argus_engine_b200 import B200Backend, DecodeExtras

    hkv, d = 8, 128
    case = wl.decode_case(4, [T], hq, hkv, d)
    be = B200Backend(0)
    bufs, lines, stride = _line_buffers(be, N, hq, hkv, d)
    counters = [torch.zeros(hkv, dtype=torch.int32, device="cuda") for _ in range(N)]
    q = torch.from_numpy(case.q[0]).cuda()
    shards = []
    for r in range(N):
        lo, hi = shard_range(T, N, r)
        n = hi - lo
        if n == 0:   # an empty slice still needs valid (unread) pointers
            shards.append((torch.zeros(hkv, 16, d, device="cuda", dtype=torch.float16), torch.zeros(hkv, 16, d, device="cuda", dtype=torch.float16), 0))
        else:
            shards.append((torch.from_numpy(np.ascontiguousarray(case.k[0][:, lo:hi])).cuda(),
                           torch.from_numpy(np.ascontiguousarray(case.v[0][:, lo:hi])).cuda(), n))
    want, _ = orc.attention_gen(case.q[0], case.k[0].view(np.uint16), case.v[0].view(np.uint16), hq, hkv, d, T)
    plen = hq * d + hq
    for step in (1, 2, 3):
        unused = torch.zeros(hq, d, device="cuda")
        parts = torch.zeros(N, plen, device="cuda")
        for r in range(N):
            k, v, n = shards[r]
            be.attention_gen_sharded(q, k, v, unused, hq, hkv, d, n, lines, r, counters[r], stride, phases=1)
            be.attention_gen(q, k, v, parts[r, :hq * d].view(hq, d), hq, hkv, d, n, extras=DecodeExtras(lse=parts[r, hq * d:]))
        for r in range(N):
            out = torch.full((hq, d), float("nan"), device="cuda")
            lse = torch.zeros(hq, device="cuda")
            be.exchange_wait_merge(parts[r], lines, r, step, stride, hq, hkv, d, out, merged_lse=lse)
            torch.cuda.synchronize()
            np.testing.assert_allclose(out.cpu().numpy(), want, atol=2e-3, rtol=1e-2)
            assert torch.isfinite(lse).all()
        assert be.check_status() == 0
        for r in range(N):
            assert (counters[r] == step).all()
    be.close()


def test_single_launch_sharded_step_one_rank_and_timeout():
    """phases = 3 in one launch. With one rank the result equals the plain decode on every step. With a second rank that
    never runs, the bounded wait for its lines runs out: status 3, zero output, and the context stays usable. The same
    for the stand-alone receiving kernel."""
    from argus_engine_b200 import B200Backend, DecodeExtras

    hq, hkv, d, T = 32, 8, 128, 5000
    case = wl.decode_case(9, [T], hq, hkv, d)
    be = B200Backend(0)
    q, k, v = (torch.from_numpy(a).cuda() for a in (case.q[0], case.k[0], case.v[0]))
    ref = torch.zeros(hq, d, device="cuda")
    ref_lse = torch.zeros(hq, device="cuda")
    be.attention_gen(q, k, v, ref, hq, hkv, d, T, extras=DecodeExtras(lse=ref_lse))
    bufs, lines, stride = _line_buffers(be, 1, hq, hkv, d)
    ctr = torch.zeros(hkv, dtype=torch.int32, device="cuda")
    for step in (1, 2, 3):
        out = torch.full((hq, d), float("nan"), device="cuda")
        lse = torch.zeros(hq, device="cuda")
        be.attention_gen_sharded(q, k, v, out, hq, hkv, d, T, lines, 0, ctr, stride, merged_lse=lse)
        torch.cuda.synchronize()
        assert torch.allclose(out, ref, atol=1e-6, rtol=1e-6)
        assert torch.allclose(lse, ref_lse, atol=1e-5)
    assert be.check_status() == 0
    # two ranks, the second never runs: rank 0's wait for rank 1's lines reaches its iteration limit
    bufs, lines, stride = _line_buffers(be, 2, hq, hkv, d)
    ctr = torch.zeros(hkv, dtype=torch.int32, device="cuda")
    out = torch.full((hq, d), float("nan"), device="cuda")
    be.attention_gen_sharded(q, k, v, out, hq, hkv, d, T, lines, 0, ctr, stride)
    assert be.check_status() == 3
    assert torch.count_nonzero(out) == 0
    part = torch.cat([ref.reshape(-1), ref_lse])
    out.fill_(float("nan"))
    be.exchange_wait_merge(part, lines, 0, 2, stride, hq, hkv, d, out)
    assert be.check_status() == 3 and torch.count_nonzero(out) == 0
    be.attention_gen(q, k, v, out, hq, hkv, d, T)
    torch.cuda.synchronize()
    assert be.check_status() == 0 and torch.allclose(out, ref)
    be.close()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_process_nccl():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", str(port), os.path.join(root, "tests", "sharded_nccl_worker.py")]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=300, cwd=root)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "SHARDED_OK" in r.stdout
