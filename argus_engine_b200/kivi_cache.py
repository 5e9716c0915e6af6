"""Device-resident KIVI container: the GPU mode of the engine's QuantizedRecentWindowCache
(engine/src/kv/quant_window_cache.rs: `new_gpu` :380-583, `update_gpu`, `flush_residual_gpu` :1688-1866),
with the flush done by the bit-exact device pack kernel instead of quantising on the CPU and uploading.

Buffers and their layouts are the engine's: packed K blocks [flush][Hkv][group][channel], packed V blocks
[flush][Hkv][token][D/32], F32 residual ring [Hkv][res_cap][D]. A token written when the ring is full first
flushes the whole ring (same timing as the reference: the flush happens at the next write).
"""
from __future__ import annotations

import torch

_BLOCK_BYTES = {2: 12, 4: 20, 8: 36}


class KiviDeviceCache:
    def __init__(self, be, kv_heads: int, head_dim: int, max_seq_len: int, res_cap: int = 128, bits: int = 4):
        if res_cap <= 0 or res_cap % 32 or head_dim % 32 or bits not in _BLOCK_BYTES:
            raise ValueError("res_cap and head_dim must be positive multiples of 32, bits one of 2/4/8")
        self.be, self.hkv, self.d, self.res_cap, self.bits = be, kv_heads, head_dim, res_cap, bits
        self.max_seq_len = max_seq_len
        bb = _BLOCK_BYTES[bits]
        max_flushes = max_seq_len // res_cap
        self.k_blocks_per_flush = kv_heads * (res_cap // 32) * head_dim
        self.v_blocks_per_flush = kv_heads * res_cap * (head_dim // 32)
        self.qk = torch.zeros(max(1, max_flushes * self.k_blocks_per_flush * bb), dtype=torch.uint8, device="cuda")
        self.qv = torch.zeros(max(1, max_flushes * self.v_blocks_per_flush * bb), dtype=torch.uint8, device="cuda")
        self.res_k = torch.zeros(kv_heads, res_cap, head_dim, device="cuda")
        self.res_v = torch.zeros(kv_heads, res_cap, head_dim, device="cuda")
        self.q_tokens = 0
        self.res_pos = 0

    @property
    def total_tokens(self) -> int:
        return self.q_tokens + self.res_pos

    def flush(self) -> None:
        """Quantise the (full) ring into blocks appended behind the existing flushes."""
        n_groups = self.res_pos // 32
        if n_groups == 0:
            return
        if n_groups * 32 != self.res_cap:
            raise RuntimeError("only a full ring is flushed (the reference flushes when res_pos == res_cap)")
        f = self.q_tokens // self.res_cap
        self.be.kivi_flush_pack(self.res_k, self.res_v, self.qk, self.qv, self.hkv, self.d, self.res_cap, n_groups,
                                self.bits, f * self.k_blocks_per_flush, f * self.v_blocks_per_flush)
        self.q_tokens += self.res_cap
        self.res_pos = 0

    def update(self, new_k: torch.Tensor, new_v: torch.Tensor) -> None:
        """new_k/new_v: [seq_len, Hkv, D] F32 device tensors (SeqMajor rows, as the engine passes them)."""
        seq_len = new_k.shape[0]
        if self.total_tokens + seq_len > self.max_seq_len:
            raise ValueError(f"KIVI cache overflow: {self.total_tokens} + {seq_len} > {self.max_seq_len}")
        s = 0
        while s < seq_len:
            if self.res_pos >= self.res_cap:
                self.flush()
            n = min(seq_len - s, self.res_cap - self.res_pos)
            for src, ring in ((new_k, self.res_k), (new_v, self.res_v)):
                rc = self.be.gather_update_quant(src[s:s + n], ring, self.hkv, self.res_cap, self.d, n, self.res_pos)
                if rc != 0:
                    raise RuntimeError(f"gather_update_quant failed: {rc}")
            self.res_pos += n
            s += n

    def seq(self, res_f16: bool = False):
        """(qk, qv, res_k, res_v, q_tokens, res_tokens) for B200Backend.kivi_attention_batched."""
        rk, rv = (self.res_k.half(), self.res_v.half()) if res_f16 else (self.res_k, self.res_v)
        return (self.qk, self.qv, rk, rv, self.q_tokens, self.res_pos)
