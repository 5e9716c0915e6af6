"""Seeded synthetic inputs with the shapes, dtypes and value distributions of the five benchmark
configurations. No public dataset belongs to them; these stand in for one. All draws use
``numpy.random.Generator(PCG64(seed)).standard_normal(float32)`` in the stated order, so the CPU oracle and
the GPU path see bit-identical inputs.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List

import numpy as np


def _rng(seed: int) -> np.random.Generator:
    return np.random.Generator(np.random.PCG64(seed))


def _normal_f16(rng: np.random.Generator, shape) -> np.ndarray:
    return rng.standard_normal(shape, dtype=np.float32).astype(np.float16)


@dataclass
class DecodeCase:
    """q [B,Hq,D] f32; per sequence K/V f16 HeadMajor [Hkv,cap,D] (cap == T unless stated)."""
    q: np.ndarray
    k: List[np.ndarray]
    v: List[np.ndarray]
    lens: List[int]
    hq: int
    hkv: int
    d: int


def decode_case(seed: int, lens, hq: int, hkv: int, d: int, cap_extra: int = 0) -> DecodeCase:
    """Draw order: q for all sequences, then per sequence K then V."""
    rng = _rng(seed)
    lens = [int(t) for t in lens]
    q = rng.standard_normal((len(lens), hq, d), dtype=np.float32)
    k, v = [], []
    for t in lens:
        k.append(_normal_f16(rng, (hkv, t + cap_extra, d)))
        v.append(_normal_f16(rng, (hkv, t + cap_extra, d)))
    return DecodeCase(q, k, v, lens, hq, hkv, d)


def config1() -> DecodeCase:
    """B=1, Hq=32, Hkv=8, D=64, T=2048, seed 0."""
    return decode_case(0, [2048], 32, 8, 64)


def config2_lengths(batch: int = 16, lo: int = 1024, hi: int = 8192, seed: int = 1) -> List[int]:
    """Per-sequence KV lengths, uniform in [lo, hi] (first draw of the seed-1 stream)."""
    return _rng(seed).integers(lo, hi, size=batch, endpoint=True).tolist()


def config2(batch: int = 16, lo: int = 1024, hi: int = 8192) -> DecodeCase:
    """Llama-3-8B layer shape: B=16, Hq=32, Hkv=8, D=128, lengths U[1024,8192], seed 1."""
    rng = _rng(1)
    lens = rng.integers(lo, hi, size=batch, endpoint=True).tolist()
    q = rng.standard_normal((batch, 32, 128), dtype=np.float32)
    k = [_normal_f16(rng, (8, t, 128)) for t in lens]
    v = [_normal_f16(rng, (8, t, 128)) for t in lens]
    return DecodeCase(q, k, v, lens, 32, 8, 128)


# ── long-context decode sharded by sequence: Hq=64, Hkv=8, D=128, T=2^20, seed 4 ──
C5_T, C5_HQ, C5_HKV, C5_D, C5_SEED = 1 << 20, 64, 8, 128, 4
C5_BLOCK = 1 << 16   # tokens per independently seeded block


def config5_q() -> np.ndarray:
    """q [64,128] float32: the first draw of PCG64(4)."""
    return _rng(C5_SEED).standard_normal((C5_HQ, C5_D), dtype=np.float32)


def config5_block(which: int, head: int, block: int) -> np.ndarray:
    """Tokens [block*65536, (block+1)*65536) of one KV head of K (which=0) or V (which=1): [65536,128] float16 drawn
    from its own stream PCG64(SeedSequence([4, which, head, block])). Independent streams per (tensor, head, block) let
    every rank of a sharded run draw exactly its slice, in parallel, and let a checker redraw one head alone."""
    rng = np.random.Generator(np.random.PCG64(np.random.SeedSequence([C5_SEED, which, head, block])))
    return rng.standard_normal((C5_BLOCK, C5_D), dtype=np.float32).astype(np.float16)


def config5_slice(lo: int, hi: int, heads=None, threads: int = 0):
    """K and V [len(heads), hi-lo, 128] float16 (HeadMajor) for tokens [lo, hi) of the listed KV heads (default all 8).
    Blocks are drawn on a thread pool (numpy's generators release the GIL)."""
    from concurrent.futures import ThreadPoolExecutor
    import os

    heads = list(range(C5_HKV)) if heads is None else list(heads)
    n = max(0, hi - lo)
    k = np.empty((len(heads), n, C5_D), dtype=np.float16)
    v = np.empty((len(heads), n, C5_D), dtype=np.float16)
    if n == 0:
        return k, v
    jobs = [(w, i, h, b) for w in (0, 1) for i, h in enumerate(heads) for b in range(lo // C5_BLOCK, (hi - 1) // C5_BLOCK + 1)]

    def run(job):
        w, i, h, b = job
        blk = config5_block(w, h, b)
        t0, t1 = max(lo, b * C5_BLOCK), min(hi, (b + 1) * C5_BLOCK)
        (k if w == 0 else v)[i, t0 - lo:t1 - lo] = blk[t0 - b * C5_BLOCK:t1 - b * C5_BLOCK]

    workers = threads or min(32, len(os.sched_getaffinity(0)))
    with ThreadPoolExecutor(max_workers=max(1, workers)) as ex:
        list(ex.map(run, jobs))
    return k, v


@dataclass
class KiviSource:
    """Un-quantised source tensors of a KIVI configuration: per sequence K and V [T,Hkv,D] float32 in token
    order (what the engine hands to the container token by token) and q [B,Hq,D]."""
    q: np.ndarray
    k: List[np.ndarray]
    v: List[np.ndarray]
    hq: int
    hkv: int
    d: int
    res_cap: int
    bits: int


def kivi_source(seed: int, lens, hq: int, hkv: int, d: int, res_cap: int = 128, bits: int = 4,
                outlier_frac: float = 0.01, outlier_scale: float = 8.0) -> KiviSource:
    """Draw order per sequence: K [T,Hkv,D], V [T,Hkv,D], the outlier (kv_head, channel) set; q after all
    sequences. `outlier_frac` of the Hkv*D K channels are multiplied by `outlier_scale` for every token."""
    rng = _rng(seed)
    ks, vs = [], []
    for t in lens:
        k = rng.standard_normal((t, hkv, d), dtype=np.float32)
        v = rng.standard_normal((t, hkv, d), dtype=np.float32)
        n_out = int(round(outlier_frac * hkv * d))
        if n_out > 0:
            idx = rng.choice(hkv * d, n_out, replace=False)
            k.reshape(t, hkv * d)[:, idx] *= outlier_scale
        ks.append(k)
        vs.append(v)
    q = rng.standard_normal((len(lens), hq, d), dtype=np.float32)
    return KiviSource(q, ks, vs, hq, hkv, d, res_cap, bits)


def config3_source(batch: int = 8, T: int = 32768) -> KiviSource:
    """KIVI Q4 decode with H2O scores: B=8, Hq=32, Hkv=8, D=128, T=32768 (32640 packed + 128 residual), seed 2."""
    return kivi_source(2, [T] * batch, 32, 8, 128, 128, 4)


def kivi_step_bytes(q_tokens, res_tokens, hq: int, hkv: int, d: int, bits: int, res_itemsize: int,
                    with_head_scores: bool = True) -> int:
    """Algorithmic bytes of one KIVI decode step: packed K and V blocks and residual rows read once, q read,
    out written, and the [Hkv,T] F32 group-mean score vector written."""
    bb = {2: 12, 4: 20, 8: 36}[bits]
    total = 0
    for qt, rt in zip(q_tokens, res_tokens):
        total += 2 * qt * hkv * (d // 32) * bb
        total += 2 * hkv * rt * d * res_itemsize
        if with_head_scores:
            total += hkv * (qt + rt) * 4
    return total + 2 * len(q_tokens) * hq * d * 4


@dataclass
class PrefillCase:
    """Q [B,S,Hq,D], K/V HeadMajor [B,Hkv,cap,D] as float32 arrays already rounded to the 16-bit input type
    (`dtype` "bf16" or "f16"); the GPU gets the same values in 16 bits, the oracle the float32 copies."""
    q: np.ndarray
    k: np.ndarray
    v: np.ndarray
    S: int
    T: int
    cap: int
    hq: int
    hkv: int
    d: int
    dtype: str


def _round_bf16(x: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even float32 -> bfloat16 -> float32."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
    r = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16) << 16
    return r.astype(np.uint32).view(np.float32).reshape(x.shape)


def prefill_case(seed: int, B: int, S: int, T: int, hq: int, hkv: int, d: int = 128, cap: int = 0,
                 dtype: str = "bf16") -> PrefillCase:
    """Draw order: Q [B,S,Hq,D], K [B,T,Hkv,D], V [B,T,Hkv,D] (token-major draws, then placed HeadMajor)."""
    rng = _rng(seed)
    cap = cap or T
    q = rng.standard_normal((B, S, hq, d), dtype=np.float32)
    k = rng.standard_normal((B, T, hkv, d), dtype=np.float32)
    v = rng.standard_normal((B, T, hkv, d), dtype=np.float32)
    rnd = _round_bf16 if dtype == "bf16" else (lambda a: a.astype(np.float16).astype(np.float32))
    kh = np.zeros((B, hkv, cap, d), dtype=np.float32)
    vh = np.zeros((B, hkv, cap, d), dtype=np.float32)
    kh[:, :, :T] = rnd(k).transpose(0, 2, 1, 3)
    vh[:, :, :T] = rnd(v).transpose(0, 2, 1, 3)
    return PrefillCase(rnd(q), kh, vh, S, T, cap, hq, hkv, d, dtype)


def config4(B: int = 4, S: int = 4096) -> PrefillCase:
    """Causal GQA prefill: B=4, S=4096, Hq=32, Hkv=8, D=128, BF16, seed 3."""
    return prefill_case(3, B, S, S, 32, 8, 128, dtype="bf16")


def prefill_flops(B: int, S: int, T: int, hq: int, d: int) -> float:
    """Causal-useful FLOPs: 4*D per (query row, visible key) pair; row r sees T-S+r+1 keys."""
    pairs = S * (T - S) + S * (S + 1) / 2.0
    return 4.0 * B * hq * d * pairs
