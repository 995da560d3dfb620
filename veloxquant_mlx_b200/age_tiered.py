"""AgeTieredKV primitives: three precision tiers gated by a token's age.

Same functions and results as ``veloxquant_mlx/quantizers/age_tiered.py`` (``assign_age_tiers``
:61-88, ``age_tier_quantize`` :91-105, ``age_tier_quantize_batched`` :108-170, byte helpers
:173-199) on CUDA tensors; the round trips are the native group-quantization kernel.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

from .quant_utils import _group_quant_dequant, _group_quant_dequant_batched

RECENT, MID, OLD = 0, 1, 2


@dataclass(frozen=True)
class AgeTierConfig:
    tier: int
    bits: int


def default_age_tiers(bits_recent: int, bits_mid: int, bits_old: int):
    return (AgeTierConfig(RECENT, bits_recent), AgeTierConfig(MID, bits_mid), AgeTierConfig(OLD, bits_old))


def assign_age_tiers(ages, age_recent_boundary: int, age_mid_boundary: int):
    return [RECENT if a < age_recent_boundary else MID if a < age_mid_boundary else OLD for a in ages]


def age_tier_quantize(x: torch.Tensor, bits: int, group_size: int = 32) -> torch.Tensor:
    if x.shape[0] == 0 or bits >= 16:
        return x
    return _group_quant_dequant(x, bits, group_size).to(x.dtype)


def age_tier_quantize_batched(raw: torch.Tensor, group_tier, tiers_config, group_size: int = 32) -> torch.Tensor:
    """``raw [G, N, D]``: every position-aligned group of ``group_size`` tokens round-tripped at the
    width of its tier (``group_tier[i]``); a ragged last group is padded with its last row. One round
    trip per tier that occurs, selected per token."""
    g, n, d = raw.shape
    if n == 0:
        return raw
    gs = group_size
    token_tier = torch.as_tensor(list(group_tier), device=raw.device).repeat_interleave(gs)[:n]
    present = set(int(t) for t in group_tier)
    out = None
    for cfg in tiers_config:
        if out is not None and cfg.tier not in present:
            continue
        q = raw if cfg.bits >= 16 else _group_quant_dequant_batched(raw, cfg.bits, gs).to(raw.dtype)
        out = q if out is None else torch.where((token_tier == cfg.tier)[None, :, None], q, out)
    return out


def age_tiered_bytes(tier_counts: dict, tiers, head_dim: int) -> int:
    by_tier = {cfg.tier: cfg.bits for cfg in tiers}
    return sum(n * ((head_dim * by_tier[t] + 7) // 8) * 2 for t, n in tier_counts.items() if n > 0)


def full_fp16_bytes(tokens_seen: int, head_dim: int) -> int:
    return tokens_seen * head_dim * 2 * 2


__all__ = ["RECENT", "MID", "OLD", "AgeTierConfig", "default_age_tiers", "assign_age_tiers", "age_tier_quantize",
           "age_tier_quantize_batched", "age_tiered_bytes", "full_fp16_bytes"]
