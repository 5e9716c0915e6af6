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


def test_fused_exchange_phases_on_one_gpu():
    """The fused exchange + merge kernel with all ranks' buffers on one GPU: the ranks push one after the other
    (phase 1), then each rank merges (phase 2) - no kernel ever waits for a later launch. Two consecutive steps
    use the two buffer sets; results equal the plain merge kernel."""
    from argus_engine_b200 import B200Backend

    be = B200Backend(0)
    N, hq, d = 4, 16, 128
    plen = hq * d + hq
    bufs = [torch.zeros(2 * N * plen + 2 * N * hq, device="cuda") for _ in range(N)]   # one "rank" each
    peer_parts = [b.data_ptr() for b in bufs]
    peer_flags = [b.data_ptr() + 4 * 2 * N * plen for b in bufs]
    gen = torch.Generator(device="cuda").manual_seed(0)
    for step in (1, 2):
        parts = torch.randn(N, plen, device="cuda", generator=gen)
        parts[1, hq * d:] = float("-inf")        # an empty shard
        want = torch.zeros(hq, d, device="cuda")
        be.lse_merge(parts, hq, d, want)
        out = [torch.full((hq, d), float("nan"), device="cuda") for _ in range(N)]
        for r in range(N):
            be.exchange_merge(parts[r], peer_parts, peer_flags, r, hq, d, out[r], step=step, parts_parity_stride=N * plen,
                              flags_parity_stride=N * hq, phases=1)
        for r in range(N):
            be.exchange_merge(parts[r], peer_parts, peer_flags, r, hq, d, out[r], step=step, parts_parity_stride=N * plen,
                              flags_parity_stride=N * hq, phases=2)
        torch.cuda.synchronize()
        assert be.check_status() == 0
        for r in range(N):
            assert torch.allclose(out[r], want, atol=1e-6, rtol=1e-6)
    be.close()


@pytest.mark.parametrize("T,N", [(20000, 4), (300, 8), (3, 2)])
def test_decode_with_fused_push_virtual_ranks(T, N):
    """The single-launch sharded step with all ranks' buffers on one GPU. Every virtual rank runs the decode kernel over
    its slice with the peer push in its epilogue (phase 1: rows + lse into slot r of every rank's receive buffer, flags
    raised, step counters bumped on the device); then every rank waits and merges with the stand-alone kernel (phase 2),
    so no kernel waits for a later launch. Two steps use the two buffer sets. Against the unsharded oracle."""
    from argus_engine_b200 import B200Backend

    hq, hkv, d = 64, 8, 128
    case = wl.decode_case(4, [T], hq, hkv, d)
    be = B200Backend(0)
    plen = hq * d + hq
    bufs = [torch.zeros(2 * N * plen + 2 * N * hq, device="cuda") for _ in range(N)]
    peer_parts = [b.data_ptr() for b in bufs]
    peer_flags = [b.data_ptr() + 4 * 2 * N * plen for b in bufs]
    counters = [torch.zeros(hkv, dtype=torch.int32, device="cuda") for _ in range(N)]
    q = torch.from_numpy(case.q[0]).cuda()
    shards = []
    for r in range(N):
        lo, hi = shard_range(T, N, r)
        shards.append((torch.from_numpy(np.ascontiguousarray(case.k[0][:, lo:hi])).cuda(),
                       torch.from_numpy(np.ascontiguousarray(case.v[0][:, lo:hi])).cuda(), hi - lo))
    want, _ = orc.attention_gen(case.q[0], case.k[0].view(np.uint16), case.v[0].view(np.uint16), hq, hkv, d, T)
    dummy = torch.zeros(plen, device="cuda")
    for step in (1, 2):
        unused = torch.zeros(hq, d, device="cuda")
        for r in range(N):
            k, v, n = shards[r]
            if n == 0:   # an empty slice still needs valid (unused) pointers
                k = v = torch.zeros(hkv, 16, d, device="cuda", dtype=torch.float16)
            be.attention_gen_sharded(q, k, v, unused, hq, hkv, d, n, peer_parts, peer_flags, r, counters[r], N * plen, N * hq,
                                     phases=1)
        for r in range(N):
            out = torch.full((hq, d), float("nan"), device="cuda")
            be.exchange_merge(dummy, peer_parts, peer_flags, r, hq, d, out, step=step, parts_parity_stride=N * plen,
                              flags_parity_stride=N * hq, phases=2)
            torch.cuda.synchronize()
            np.testing.assert_allclose(out.cpu().numpy(), want, atol=2e-3, rtol=1e-2)
        assert be.check_status() == 0
        for r in range(N):
            assert (counters[r] == step).all()
    be.close()


def test_single_launch_sharded_step_one_rank_and_timeout():
    """phases = 3 in one launch. With one rank the CTA that completes a KV head finds its own flags and the result equals
    the plain decode (also on the second step, which uses the other buffer set). With a second rank that never pushes
    the bounded wait runs out: status 3, zero output, and the context stays usable."""
    from argus_engine_b200 import B200Backend, DecodeExtras

    hq, hkv, d, T = 32, 8, 128, 5000
    case = wl.decode_case(9, [T], hq, hkv, d)
    be = B200Backend(0)
    q, k, v = (torch.from_numpy(a).cuda() for a in (case.q[0], case.k[0], case.v[0]))
    ref = torch.zeros(hq, d, device="cuda")
    ref_lse = torch.zeros(hq, device="cuda")
    be.attention_gen(q, k, v, ref, hq, hkv, d, T, extras=DecodeExtras(lse=ref_lse))
    plen = hq * d + hq
    buf = torch.zeros(2 * plen + 2 * hq, device="cuda")
    ctr = torch.zeros(hkv, dtype=torch.int32, device="cuda")
    for step in (1, 2, 3):
        out = torch.full((hq, d), float("nan"), device="cuda")
        lse = torch.zeros(hq, device="cuda")
        be.attention_gen_sharded(q, k, v, out, hq, hkv, d, T, [buf.data_ptr()], [buf.data_ptr() + 4 * 2 * plen], 0, ctr, plen, hq,
                                 merged_lse=lse)
        torch.cuda.synchronize()
        assert torch.allclose(out, ref, atol=1e-6, rtol=1e-6)
        assert torch.allclose(lse, ref_lse, atol=1e-5)
    assert be.check_status() == 0
    # two ranks, the second never runs: rank 0's wait for rank 1's flags reaches its iteration limit
    N = 2
    bufs = [torch.zeros(2 * N * plen + 2 * N * hq, device="cuda") for _ in range(N)]
    ctr = torch.zeros(hkv, dtype=torch.int32, device="cuda")
    out = torch.full((hq, d), float("nan"), device="cuda")
    be.attention_gen_sharded(q, k, v, out, hq, hkv, d, T, [b.data_ptr() for b in bufs],
                             [b.data_ptr() + 4 * 2 * N * plen for b in bufs], 0, ctr, N * plen, N * hq)
    assert be.check_status() == 3
    assert torch.count_nonzero(out) == 0
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


def test_exchange_wait_runs_out_when_a_rank_never_pushes():
    """Failure detection without a fault: rank 1 never pushes, so rank 0's wait for rank 1's flags reaches its iteration
    limit; the kernel returns, the status word reads 3, the unmerged heads are zero and the context stays usable."""
    from argus_engine_b200 import B200Backend

    be = B200Backend(0)
    N, hq, d = 2, 4, 128
    plen = hq * d + hq
    bufs = [torch.zeros(2 * N * plen + 2 * N * hq, device="cuda") for _ in range(N)]
    peer_parts = [b.data_ptr() for b in bufs]
    peer_flags = [b.data_ptr() + 4 * 2 * N * plen for b in bufs]
    part = torch.randn(plen, device="cuda")
    out = torch.full((hq, d), float("nan"), device="cuda")
    be.exchange_merge(part, peer_parts, peer_flags, 0, hq, d, out, step=1, parts_parity_stride=N * plen,
                      flags_parity_stride=N * hq, phases=1)          # rank 0 pushes ...
    be.exchange_merge(part, peer_parts, peer_flags, 0, hq, d, out, step=1, parts_parity_stride=N * plen,
                      flags_parity_stride=N * hq, phases=2)          # ... and waits for a rank 1 that never comes
    assert be.check_status() == 3
    assert torch.count_nonzero(out) == 0
    # the context and the device are fine: a complete exchange on the next step works
    want = torch.zeros(hq, d, device="cuda")
    parts = torch.stack([part, part])
    be.lse_merge(parts, hq, d, want)
    for r in range(N):
        be.exchange_merge(part, peer_parts, peer_flags, r, hq, d, out, step=2, parts_parity_stride=N * plen,
                          flags_parity_stride=N * hq, phases=1)
    be.exchange_merge(part, peer_parts, peer_flags, 0, hq, d, out, step=2, parts_parity_stride=N * plen,
                      flags_parity_stride=N * hq, phases=2)
    torch.cuda.synchronize()
    assert be.check_status() == 0
    assert torch.allclose(out, want, atol=1e-6, rtol=1e-6)
    be.close()
