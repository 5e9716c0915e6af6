"""CPU-only checks of the C-ABI boundary: the library loads without a GPU, exports every symbol that
include/argus_b200.h declares, and the ctypes mirrors of the reference's #[repr(C)] structs have the sizes
the header asserts. No compute call is made here."""
import ctypes as C
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    text = open(os.path.join(ROOT, "include", "argus_b200.h")).read()
    return sorted(set(re.findall(r"ARGUS_B200_API[^;(]*?\b(argus_b200_\w+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    from argus_engine_b200 import load_library

    lib = load_library()
    names = _declared()
    assert len(names) >= 20
    for n in names:
        assert hasattr(lib, n), f"{n} is declared in the header but not exported"
    assert lib.argus_b200_version() >= 1 and lib.argus_b200_sm_arch() == 100


def test_struct_mirrors_match_reference_layouts():
    from argus_engine_b200 import _lib

    assert C.sizeof(_lib.QuantAttnArgs) == 128 and _lib.QuantAttnArgs.scale.offset == 120
    assert C.sizeof(_lib.QuantGatherArgs) == 64
    assert C.sizeof(_lib.QuantDequantFlushArgs) == 72 and _lib.QuantDequantFlushArgs.bits.offset == 64
    assert C.sizeof(_lib.QuantScatterResidualArgs) == 64
    assert C.sizeof(_lib.ScoreReduceArgs) == 96 and _lib.ScoreReduceArgs.n_layers.offset == 40
    assert C.sizeof(_lib.DecodeExtrasC) == 48 and C.sizeof(_lib.Seq) == 40 and C.sizeof(_lib.KiviSeq) == 48


def test_no_gpu_means_loud_failure_not_fallback():
    import pytest
    import torch

    from argus_engine_b200 import B200Backend

    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    with pytest.raises(RuntimeError):
        B200Backend(0)


def test_product_never_imports_the_oracle():
    """Nothing in the shipped package imports, loads or runs anything under oracle/."""
    pkg = os.path.join(ROOT, "argus_engine_b200")
    for fn in os.listdir(pkg):
        if fn.endswith(".py"):
            text = open(os.path.join(pkg, fn)).read()
            assert not re.search(r"^\s*(from|import)\s+oracle", text, re.M), fn
            assert "libargus_oracle" not in text, fn


def test_rust_ffi_crate_declares_every_export():
    """crates/argus-b200-sys cannot be compiled where no Rust toolchain exists, so its completeness is checked as text:
    every function the C header exports has a `pub fn` declaration in the crate's extern block."""
    text = open(os.path.join(ROOT, "crates", "argus-b200-sys", "src", "lib.rs")).read()
    declared = set(re.findall(r"pub fn (argus_b200_\w+)\s*\(", text))
    missing = [n for n in _declared() if n not in declared]
    assert not missing, f"missing from the Rust FFI crate: {missing}"


def test_ctypes_offsets_match_the_guards_of_the_header_and_crate():
    from argus_engine_b200 import _lib

    qa = _lib.QuantAttnArgs
    assert (qa.scores_out.offset, qa.scores_len.offset, qa.num_heads_q.offset, qa.scale.offset, qa.bits.offset) == (56, 64, 72, 120, 124)
    assert _lib.QuantGatherArgs.kv_heads.offset == 24 and _lib.QuantScatterResidualArgs.kv_heads.offset == 24
    df = _lib.QuantDequantFlushArgs
    assert (df.kv_heads.offset, df.bits.offset, df.is_key.offset) == (24, 64, 65)
    sr = _lib.ScoreReduceArgs
    assert (sr.decay_factor.offset, sr.n_layers.offset, sr.layer_flat_importance.offset) == (32, 40, 88)
    assert C.sizeof(_lib.ExchangeC) == 48 and _lib.ExchangeC.n_ranks.offset == 32


def test_exchange_buffer_units_cover_the_head_group_in_whole_lines():
    """argus_b200_exchange_lines_per_head (host-only, no GPU): 16-byte units of a head group's receive slot. The wire
    format is 128-byte lines of 30 data words + 2 flag words, four lines per warp store, so the count is a multiple of
    32 units and holds g*(D+1) floats."""
    from argus_engine_b200 import load_library

    lib = load_library()
    for hq, hkv, d in [(64, 8, 128), (32, 8, 128), (8, 8, 128), (32, 8, 64), (16, 2, 64)]:
        units = lib.argus_b200_exchange_lines_per_head(hq, hkv, d)
        g = hq // hkv
        lines = units // 8
        assert units % 32 == 0 and lines * 30 >= g * (d + 1) and (lines - 4) * 30 < g * (d + 1)
