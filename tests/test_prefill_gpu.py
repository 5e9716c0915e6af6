"""GPU parity of the tcgen05 causal prefill against the CPU oracle (tiled F32 flash attention on the same
16-bit-rounded inputs), through the C ABI. Tolerance max-abs 2e-3 / rel 1e-2 on F32 outputs; 16-bit outputs
are compared after rounding the oracle to the same type, with one extra unit of output rounding allowed."""
import numpy as np
import pytest
import torch

from argus_engine_b200 import workloads as wl
from oracle import oracle as orc

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def be():
    from argus_engine_b200 import B200Backend

    b = B200Backend(0, workspace_bytes=256 << 20)
    yield b
    b.close()


def _t(a, dtype):
    return torch.from_numpy(np.ascontiguousarray(a)).to(dtype).cuda()


def _run(be, case, mode):
    tq = {"f32": torch.float32, "bf16": torch.bfloat16, "f16": torch.float16}[mode]
    tkv = torch.float16 if mode == "f32" else tq
    q, k, v = _t(case.q, tq), _t(case.k, tkv), _t(case.v, tkv)
    B = case.q.shape[0]
    out = torch.full((B, case.S, case.hq, case.d), float("nan"), dtype=tq, device="cuda")
    ok = be.flash_attention_prefill(q, k, v, out, case.hq, case.hkv, case.S, case.T, case.d, case.cap, B, True)
    torch.cuda.synchronize()
    assert be.check_status() == 0
    return ok, out.float().cpu().numpy()


def _check(got, want, mode):
    if mode == "f32":
        np.testing.assert_allclose(got, want, atol=2e-3, rtol=1e-2)
    else:
        eps = 2.0 ** -8 if mode == "bf16" else 2.0 ** -11   # one unit of output rounding on top of the tolerance
        np.testing.assert_allclose(got, want, atol=2e-3, rtol=1e-2 + eps)


@pytest.mark.parametrize("mode", ["bf16", "f16", "f32"])
@pytest.mark.parametrize("S,T,g", [(128, 128, 1), (256, 256, 4), (200, 200, 2), (1, 1, 4), (77, 300, 4), (384, 512, 8),
                                   (130, 130, 4)])
def test_prefill_vs_oracle(be, mode, S, T, g):
    """GQA 1/2/4/8, ragged tiles, single token (=> out = V), continuation (cache_seq_len > seq_len), capacity > T
    with NaN rows past T — the matrix of engine/tests/test_prefill_flash_attention.rs and
    engine/src/backend/cuda_pc.rs:2272-2577."""
    hkv = 2
    case = wl.prefill_case(50 + S + T + g, 2, S, T, hkv * g, hkv, 128, cap=T + 9, dtype="f16" if mode != "bf16" else "bf16")
    want = orc.flash_prefill(case.q, case.k, case.v, case.hq, hkv, S, T, 128, case.cap)
    case.k[:, :, T:] = np.nan
    case.v[:, :, T:] = np.nan
    ok, got = _run(be, case, mode)
    assert ok
    _check(got, want, mode)
    if S == 1 and T == 1:
        np.testing.assert_allclose(got[:, 0], case.v[:, :, 0].repeat(g, axis=1), atol=1e-6)


def test_prefill_causal_uniform(be):
    """K = 0 => row r is the mean of V[0..=r] (engine/src/kv/quant_window_format.rs:524-586)."""
    case = wl.prefill_case(9, 1, 300, 300, 4, 1, 128, dtype="f16")
    case.k[:] = 0
    ok, got = _run(be, case, "f32")
    want = np.cumsum(case.v[0, 0].astype(np.float64), axis=0) / np.arange(1, 301)[:, None]
    np.testing.assert_allclose(got[0, :, 2], want, atol=2e-3, rtol=1e-2)


def test_prefill_bf16_llama_shape_reduced(be):
    """The benchmarked prefill shape at reduced size (B=1, S=1024, Hq=32, Hkv=8, D=128, BF16, seed 3) against the oracle
    (the full size is covered in tests/test_full_size_gpu.py)."""
    case = wl.prefill_case(3, 1, 1024, 1024, 32, 8, 128, dtype="bf16")
    want = orc.flash_prefill(case.q, case.k, case.v, 32, 8, 1024, 1024, 128, 1024)
    ok, got = _run(be, case, "bf16")
    assert ok
    _check(got, want, "bf16")


def test_prefill_declines_other_head_dims(be):
    q = torch.zeros(1, 16, 4, 64, dtype=torch.bfloat16, device="cuda")
    k = torch.zeros(1, 2, 16, 64, dtype=torch.bfloat16, device="cuda")
    assert be.flash_attention_prefill(q, k, k, torch.zeros_like(q), 4, 2, 16, 16, 64, 16, 1, True) is False


def test_bf16_v_beyond_f16_range_is_clamped_and_reported(be):
    """BF16 inputs are served with an F16 copy of each V tile: exact up to |v| = 65504 (largest finite F16), clamped
    beyond, and the clamp is reported through the status word (4). With a single key the output row IS the V row, so
    the boundary shows directly."""
    B, S, hq, hkv, d = 1, 128, 4, 1, 128
    case = wl.prefill_case(5, B, S, S, hq, hkv, d, dtype="bf16")
    case.k[:] = 0                      # uniform attention: row r is the mean of V rows 0..=r
    case.v[:] = 0
    case.v[0, 0, 0, 0] = 65280.0       # the largest BF16 value below 65504: representable in both types
    case.v[0, 0, 0, 1] = -65280.0
    ok, got = _run(be, case, "bf16")
    assert ok and be.check_status() == 0
    assert got[0, 0, 0, 0] == 65280.0 and got[0, 0, 0, 1] == -65280.0
    case.v[0, 0, 0, 2] = 131072.0      # finite in BF16, beyond F16
    tq = torch.bfloat16
    q, k, v = _t(case.q, tq), _t(case.k, tq), _t(case.v, tq)
    out = torch.zeros(B, S, hq, d, dtype=tq, device="cuda")
    assert be.flash_attention_prefill(q, k, v, out, hq, hkv, S, S, d, S, B, True)
    torch.cuda.synchronize()
    assert be.check_status() == 4
    o = out.float().cpu().numpy()
    assert o[0, 0, 0, 2] == 65504.0 or o[0, 0, 0, 2] == 65536.0   # the clamped value, rounded to BF16 on output
    assert o[0, 0, 0, 0] == 65280.0
    assert be.check_status() == 0      # cleared by the read
