"""The allocation-free decode entry point (argus_b200_attention_gen_static).

It serves callers that may not allocate device memory (stream capture, serving loops, embedders with their
own pool): its scratch is a fixed 4 MiB array inside the library, shared by all calls on a device and never
cleared between them. The test calls it twice in a row through the C ABI, on different inputs, back to back on
one stream with no synchronisation between the two calls (the documented way to share the array), and compares
each result with the context-based entry point and with the CPU oracle (max-abs 2e-3 / rel 1e-2, the tolerance
of the decode tests); the second call must not be disturbed by what the first one left in the array. This file
sorts last so that a run stopping at the first failure has already run every other test.
"""
import numpy as np
import pytest
import torch

from argus_engine_b200 import workloads as wl
from oracle import oracle as orc

pytestmark = pytest.mark.gpu


def test_static_entry_matches_context_entry_twice():
    from argus_engine_b200 import B200Backend, DecodeExtras, load_library

    lib = load_library()
    be = B200Backend(0)
    assert lib.argus_b200_static_scratch_bytes() == 4 << 20
    stream = torch.cuda.current_stream().cuda_stream
    shapes = [(5000, 32, 8, 128), (333, 16, 2, 64)]
    cases, dev, wants = [], [], []
    for call, (T, hq, hkv, d) in enumerate(shapes):
        case = wl.decode_case(40 + call, [T], hq, hkv, d)
        q = torch.from_numpy(case.q[0]).cuda()
        k = torch.from_numpy(case.k[0]).cuda()
        v = torch.from_numpy(case.v[0]).cuda()
        want = torch.zeros(hq, d, device="cuda")
        want_lse = torch.zeros(hq, device="cuda")
        be.attention_gen(q, k, v, want, hq, hkv, d, T, extras=DecodeExtras(lse=want_lse))
        got = torch.full((hq, d), float("nan"), device="cuda")
        got_lse = torch.full((hq,), float("nan"), device="cuda")
        cases.append(case)
        dev.append((q, k, v, got, got_lse))
        wants.append((want, want_lse))
    torch.cuda.synchronize()
    # the two calls go out back to back on one stream: the second starts from whatever the first left in the array
    for (T, hq, hkv, d), (q, k, v, got, got_lse) in zip(shapes, dev):
        rc = lib.argus_b200_attention_gen_static(stream, q.data_ptr(), k.data_ptr(), v.data_ptr(), got.data_ptr(),
                                                 got_lse.data_ptr(), hq, hkv, d, T, 1, T * d, d)
        assert rc == 0, lib.argus_b200_static_last_error().decode()
    torch.cuda.synchronize()
    for (T, hq, hkv, d), case, (q, k, v, got, got_lse), (want, want_lse) in zip(shapes, cases, dev, wants):
        np.testing.assert_allclose(got.cpu().numpy(), want.cpu().numpy(), atol=2e-3, rtol=1e-2)
        np.testing.assert_allclose(got_lse.cpu().numpy(), want_lse.cpu().numpy(), atol=1e-3)
        ref, _ = orc.attention_gen(case.q[0], case.k[0].view(np.uint16), case.v[0].view(np.uint16), hq, hkv, d, T)
        np.testing.assert_allclose(got.cpu().numpy(), ref, atol=2e-3, rtol=1e-2)
    # sizes beyond the fixed array are refused with a clear message, not served by allocating
    q = torch.zeros(2048, 128, device="cuda")
    k = torch.zeros(2048, 64, 128, dtype=torch.float16, device="cuda")
    rc = lib.argus_b200_attention_gen_static(stream, q.data_ptr(), k.data_ptr(), k.data_ptr(), q.data_ptr(), None, 2048,
                                             2048, 128, 64, 1, 64 * 128, 128)
    assert rc == -4 and b"ticket" in lib.argus_b200_static_last_error()
    be.close()
