"""Test helper: packs a KiviSource with the CPU oracle's container (the checker's view of the engine's flush)."""
from dataclasses import dataclass
from typing import List

import numpy as np

from oracle import oracle as orc


@dataclass
class KiviCase:
    q: np.ndarray
    qk: List[np.ndarray]
    qv: List[np.ndarray]
    res_k: List[np.ndarray]
    res_v: List[np.ndarray]
    q_tokens: List[int]
    res_tokens: List[int]
    hq: int
    hkv: int
    d: int
    res_cap: int
    bits: int


def pack_with_oracle(src, res_f16: bool = False) -> KiviCase:
    out = KiviCase(src.q, [], [], [], [], [], [], src.hq, src.hkv, src.d, src.res_cap, src.bits)
    for k, v in zip(src.k, src.v):
        c = orc.KiviCache(src.hkv, src.d, src.res_cap, src.bits)
        c.update(k, v)
        qk, qv, rk, rv = c.export()
        if res_f16:
            rk, rv = rk.astype(np.float16), rv.astype(np.float16)
        out.qk.append(qk)
        out.qv.append(qv)
        out.res_k.append(rk)
        out.res_v.append(rv)
        out.q_tokens.append(c.q_tokens)
        out.res_tokens.append(c.res_tokens)
    return out
