"""Worker of tests/test_sharded_gpu.py::test_two_process_nccl (launched by torch.distributed.run)."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from argus_engine_b200 import B200Backend, workloads as wl  # noqa: E402
from argus_engine_b200.sharded import make_gpu_decoder, shard_range  # noqa: E402
from oracle import oracle as orc  # noqa: E402

local = int(os.environ["LOCAL_RANK"])
torch.cuda.set_device(local)
dist.init_process_group("nccl", device_id=torch.device("cuda", local))
rank, world = dist.get_rank(), dist.get_world_size()
T, hq, hkv, d = 30000, 64, 8, 128
case = wl.decode_case(4, [T], hq, hkv, d)
lo, hi = shard_range(T, world, rank)
be = B200Backend(local)
k = torch.from_numpy(np.ascontiguousarray(case.k[0][:, lo:hi])).cuda()
v = torch.from_numpy(np.ascontiguousarray(case.v[0][:, lo:hi])).cuda()
want, _ = orc.attention_gen(case.q[0], case.k[0].view(np.uint16), case.v[0].view(np.uint16), hq, hkv, d, T)
qd = torch.from_numpy(case.q[0]).cuda()
# NCCL all-gather + merge, then the single-launch step (flagged lines pushed with plain peer stores)
for fused in (False, True):
    dec = make_gpu_decoder(be, k, v, hi - lo, hq, hkv, d, fused=fused)
    for _ in range(3):           # several steps: the fused paths alternate their two buffer sets
        out = torch.full((hq, d), float("nan"), device="cuda")
        dec.step(qd, out)
        torch.cuda.synchronize()
        np.testing.assert_allclose(out.cpu().numpy(), want, atol=2e-3, rtol=1e-2)
    assert be.check_status() == 0
dist.barrier()
if rank == 0:
    print("SHARDED_OK")
dist.destroy_process_group()
