"""Where a sequence-sharded decode step spends its time, per rank: the whole launch (CUDA events), per KV head the
three globaltimer stamps of the exchange in the decode kernel's epilogue - tail start (the head's last split has merged
locally), rows pushed to every peer, peers' rows collected and merged - and, over the CTAs of one launch, the earliest
and latest first-tile arrival, end of the tile loop and end of the epilogue.

Needs the time-stamped twin of the library (`python -m argus_engine_b200.build --stamped`, never the default build) and
one process per GPU:

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port 29531 \\
        -m argus_engine_b200.exchange_stamps [--tokens 1048576]

The cache is random F16 of the 1M-token decode shape (Hq=64, Hkv=8, D=128), each rank holding its slice.
"""
from __future__ import annotations

import argparse
import ctypes as C
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
os.environ.setdefault("ARGUS_B200_LIB_PATH", os.path.join(HERE, "libargus_b200_stamped.so"))

import numpy as np  # noqa: E402
import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402

from . import B200Backend, load_library  # noqa: E402
from .sharded import make_gpu_decoder, shard_range  # noqa: E402


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=1 << 20)
    ap.add_argument("--replays", type=int, default=20)
    args = ap.parse_args()
    lib = load_library()
    if not hasattr(lib, "argus_b200_debug_xc_profile"):
        sys.stderr.write("this library has no time stamps: build it with `python -m argus_engine_b200.build --stamped`\n")
        return 2
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    rank, world = dist.get_rank(), dist.get_world_size()
    hq, hkv, d = 64, 8, 128
    lo, hi = shard_range(args.tokens, world, rank)
    n = hi - lo
    gen = torch.Generator(device="cuda").manual_seed(1000 + rank)
    k = torch.randn(hkv, n, d, device="cuda", generator=gen, dtype=torch.float16)
    v = torch.randn(hkv, n, d, device="cuda", generator=gen, dtype=torch.float16)
    q = torch.randn(hq, d, device="cuda", generator=torch.Generator(device="cuda").manual_seed(99))
    out = torch.zeros(hq, d, device="cuda")
    be = B200Backend(local)
    dec = make_gpu_decoder(be, k, v, n, hq, hkv, d, fused=True)
    for _ in range(5):
        dec.step(q, out)
    dist.barrier()
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        dec.step(q, out)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for _ in range(5):
        graph.replay()
    dist.barrier()
    torch.cuda.synchronize()
    e0.record()
    for _ in range(args.replays):
        graph.replay()
    e1.record()
    torch.cuda.synchronize()
    step_us = e0.elapsed_time(e1) * 1e3 / args.replays
    ph = (C.c_ulonglong * 8)()
    lib.argus_b200_debug_phase_profile(ph)   # re-arm the min / max phase stamps, then one more replay
    dist.barrier()
    graph.replay()
    torch.cuda.synchronize()
    lib.argus_b200_debug_phase_profile(ph)
    pv = np.array(list(ph), dtype=np.float64)
    pv = (pv - pv[0]) / 1e3   # us after the first CTA's entry: [entry min,max | first tile min,max | loop end min,max | epilogue end min,max]
    buf = (C.c_ulonglong * 512)()
    lib.argus_b200_debug_xc_profile(buf)   # stamps of the last replay, ns of this GPU's globaltimer
    a = np.array(list(buf), dtype=np.int64).reshape(64, 8)[:hkv, :3]
    mine = {"rank": rank, "step_us": step_us, "status": be.check_status(),
            "pushed_after_tail_us": ((a[:, 1] - a[:, 0]) / 1e3).tolist(),
            "merged_after_tail_us": ((a[:, 2] - a[:, 0]) / 1e3).tolist(),
            "tail_spread_us": float((a[:, 0].max() - a[:, 0].min()) / 1e3),
            "first_tail_to_last_merge_us": float((a[:, 2].max() - a[:, 0].min()) / 1e3),
            "phases_us": pv.tolist()}
    rows = [None] * world
    dist.all_gather_object(rows, mine)
    if rank == 0:
        print(f"sharded decode, {args.tokens} tokens over {world} GPUs, {args.replays} graph replays")
        print("rank  step us  status  pushed-after-tail us (min..max over KV heads)  merged-after-tail us (min..max)  "
              "tail spread us  first tail -> last merge us")
        for r in (rows if world > 1 else []):   # one rank has no exchange: its step is the decode kernel + the merge kernel
            p_, m_ = r["pushed_after_tail_us"], r["merged_after_tail_us"]
            print(f"{r['rank']:4d}  {r['step_us']:7.1f}  {r['status']:6d}  {min(p_):6.2f} .. {max(p_):6.2f}"
                  f"{'':24s}{min(m_):6.2f} .. {max(m_):6.2f}{'':9s}{r['tail_spread_us']:8.2f}  "
                  f"{r['first_tail_to_last_merge_us']:8.2f}")
        print("rank  first tile ready us (earliest..latest CTA)  tile loop ends us  epilogue ends us   (after the first CTA's entry)")
        for r in rows:
            p_ = r["phases_us"]
            print(f"{r['rank']:4d}  {p_[2]:6.1f} .. {p_[3]:6.1f}{'':22s}{p_[4]:6.1f} .. {p_[5]:6.1f}   {p_[6]:6.1f} .. {p_[7]:6.1f}")
        print(f"max over ranks: step {max(r['step_us'] for r in rows):.1f} us; "
              f"merged-after-tail {max(max(r['merged_after_tail_us']) for r in rows):.2f} us")
    dist.barrier()
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
