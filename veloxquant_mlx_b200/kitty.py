"""Kitty: channel-wise mixed-precision key quantization (top-variance channels at ``hi_bit``,
the rest at ``lo_bit``), groups along the token axis.

Same functions and results as ``veloxquant_mlx/quantizers/kitty.py`` (``rank_channels_by_sensitivity``
:41-64, ``quantize_mixed_channels`` :67-120, ``hi_mask_from_variance_batched`` :123-147,
``quantize_mixed_channels_batched`` :150-182, ``compute_running_variance`` :185-203) on CUDA
tensors; the round trips are the native group-quantization kernel (``quant_utils``).
"""

from __future__ import annotations

import torch

from .quant_utils import _group_quant_dequant_batched


def hi_mask_from_variance_batched(variance: torch.Tensor, hi_fraction: float) -> torch.Tensor:
    """``variance [N, D]`` -> bool ``[N, D]``: the ``max(1, int(D*hi_fraction))`` highest-variance
    channels of every row (ties: the lower channel index first)."""
    n, d = variance.shape
    n_hi = max(1, int(d * hi_fraction))
    order = torch.argsort(-variance, dim=-1, stable=True)
    rank = torch.argsort(order, dim=-1, stable=True)
    return rank < n_hi


def rank_channels_by_sensitivity(keys: torch.Tensor, hi_fraction: float = 0.25):
    """``keys [S, D]`` -> ``(hi_indices, lo_indices)``, ascending lists of column indices."""
    variance = torch.var(keys.float(), dim=0, unbiased=False)
    mask = hi_mask_from_variance_batched(variance[None], hi_fraction)[0]
    idx = torch.arange(keys.shape[-1], device=keys.device)
    return idx[mask].tolist(), idx[~mask].tolist()


def quantize_mixed_channels_batched(keys: torch.Tensor, hi_mask: torch.Tensor, hi_bit: int = 4, lo_bit: int = 2,
                                    group_size: int = 32) -> torch.Tensor:
    """``keys [N, S, D]``, ``hi_mask [N, D]`` -> float16 ``[N, S, D]``: every channel round-tripped at
    its row's width (channels quantize independently, so this is a select between two full round trips)."""
    recon_hi = _group_quant_dequant_batched(keys, hi_bit, group_size)
    recon_lo = _group_quant_dequant_batched(keys, lo_bit, group_size)
    return torch.where(hi_mask[:, None, :], recon_hi, recon_lo).to(torch.float16)


def quantize_mixed_channels(keys: torch.Tensor, hi_indices, lo_indices, hi_bit: int = 4, lo_bit: int = 2,
                            group_size: int = 32) -> torch.Tensor:
    """``keys [S, D]`` with explicit channel lists -> float16 ``[S, D]`` (channels in neither list pass
    through as float16, as in the reference)."""
    s, d = keys.shape
    out = keys.to(torch.float16).clone()
    if len(hi_indices):
        hi = torch.as_tensor(list(hi_indices), device=keys.device, dtype=torch.long)
        out[:, hi] = _group_quant_dequant_batched(keys[None], hi_bit, group_size)[0][:, hi]
    if len(lo_indices):
        lo = torch.as_tensor(list(lo_indices), device=keys.device, dtype=torch.long)
        out[:, lo] = _group_quant_dequant_batched(keys[None], lo_bit, group_size)[0][:, lo]
    return out


def compute_running_variance(key_sum: torch.Tensor, key_sq_sum: torch.Tensor, n: int) -> torch.Tensor:
    """Per-channel variance from running sums (zeros while fewer than two tokens were seen)."""
    if n < 2:
        return torch.zeros_like(key_sum)
    mean = key_sum / n
    return torch.clamp_min(key_sq_sum / n - mean * mean, 0.0)


__all__ = ["rank_channels_by_sensitivity", "quantize_mixed_channels", "compute_running_variance",
           "hi_mask_from_variance_batched", "quantize_mixed_channels_batched"]
