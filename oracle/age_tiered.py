"""TEST INFRASTRUCTURE ONLY -- CPU restatement (NumPy) of the reference's AgeTieredKV path.

Follows ``veloxquant_mlx/quantizers/age_tiered.py`` (``assign_age_tiers`` :61-88,
``age_tier_quantize_batched`` :108-170, byte helpers :173-199) and the cache policy of
``veloxquant_mlx/cache/age_tiered_cache.py:154-214`` (every call: ages from the current position,
a group of ``group_size`` position-aligned tokens takes the tier of its first token, each group's
output is one round trip of its RAW rows at that tier's width, a ragged last group padded with its
last row). The reference's splice of unchanged groups (:248-333) returns the same values as
recomputing every group from raw, which is what this model does.

Pinning: ``tests/golden/group_quant.npz`` (the reference's modules executed with a NumPy stand-in
for ``mlx.core``) pins the quantizer functions; the cache model reproduces what the reference's
``AgeTieredKVCache`` class returns over a call script, executed over the same stand-in and a minimal
container for its ``mlx_lm`` base class (``tests/golden/cache_traces.npz``).
"""

from __future__ import annotations

import numpy as np

from .kitty import group_quant_dequant_batched

RECENT, MID, OLD = 0, 1, 2


def assign_age_tiers(ages, recent_boundary: int, mid_boundary: int):
    return [RECENT if a < recent_boundary else MID if a < mid_boundary else OLD for a in ages]


def age_tier_quantize_batched(raw: np.ndarray, group_tier, bits_by_tier, gs: int = 32) -> np.ndarray:
    """``raw [G, N, D]``; ``bits_by_tier = (recent, mid, old)``; result in ``raw.dtype``."""
    g, n, d = raw.shape
    if n == 0:
        return raw
    token_tier = np.repeat(np.asarray(group_tier), gs)[:n]
    out = None
    for tier, bits in enumerate(bits_by_tier):
        q = raw if bits >= 16 else group_quant_dequant_batched(raw, bits, gs).astype(raw.dtype)
        out = q if out is None else np.where((token_tier == tier)[None, :, None], q, out)
    return out


def age_tiered_bytes(tier_counts: dict, bits_by_tier, head_dim: int) -> int:
    return sum(n * ((head_dim * bits_by_tier[t] + 7) // 8) * 2 for t, n in tier_counts.items() if n > 0)


def full_fp16_bytes(tokens_seen: int, head_dim: int) -> int:
    return tokens_seen * head_dim * 2 * 2


class AgeTieredCacheModel:
    def __init__(self, head_dim, recent_boundary=128, mid_boundary=1024, bits=(8, 4, 2), group_size=32):
        self.D, self.rb, self.mb, self.bits, self.gs = head_dim, recent_boundary, mid_boundary, tuple(bits), group_size
        self.raw_k = self.raw_v = None
        self.position = 0
        self.age_tiered_bytes = self.full_seq_bytes = 0

    def update_and_fetch(self, keys, values):
        B, H, S, D = keys.shape
        self.full_seq_bytes += full_fp16_bytes(B * H * S, D)
        self.position += S
        k, v = keys.reshape(B * H, S, D), values.reshape(B * H, S, D)
        self.raw_k = k if self.raw_k is None else np.concatenate([self.raw_k, k], axis=1)
        self.raw_v = v if self.raw_v is None else np.concatenate([self.raw_v, v], axis=1)
        n = self.raw_k.shape[1]
        tiers = assign_age_tiers([self.position - (i + 1) for i in range(n)], self.rb, self.mb)
        group_tier = [tiers[g * self.gs] for g in range(-(-n // self.gs))]
        ko = age_tier_quantize_batched(self.raw_k, group_tier, self.bits, self.gs)
        vo = age_tier_quantize_batched(self.raw_v, group_tier, self.bits, self.gs)
        counts = {t: tiers.count(t) * B * H for t in (RECENT, MID, OLD)}
        self.age_tiered_bytes = age_tiered_bytes(counts, self.bits, D)
        return ko.reshape(B, H, n, D), vo.reshape(B, H, n, D)
