"""TEST INFRASTRUCTURE ONLY -- CPU restatement (NumPy) of the reference's Kitty path.

Follows ``veloxquant_mlx/quantizers/kitty.py`` (``hi_mask_from_variance_batched`` :123-147,
``quantize_mixed_channels_batched`` :150-182, ``compute_running_variance`` :185-203) and the
cache ``veloxquant_mlx/cache/kitty_cache.py`` (ranking from the batch at prefill and from running
statistics afterwards :86-114, accumulators fed with the stored keys :116-137, byte accounting
:153-167, trim :180-210).

Pinning: ``tests/golden/group_quant.npz`` holds outputs of the reference's modules executed with a
NumPy stand-in for ``mlx.core``; the quantizer functions here reproduce them bit for bit, and the
cache model reproduces what the reference's ``KittyKVCache`` class returns over a call script with a
trim, executed over the same stand-in and a minimal container for its ``mlx_lm`` base class
(``tests/golden/cache_traces.npz``). Its variance and accumulator sums are float32 NumPy
reductions, whose order MLX need not share.
"""

from __future__ import annotations

import math

import numpy as np

from . import kivi

f32 = np.float32


def group_quant_dequant_batched(x: np.ndarray, b: int, gs: int) -> np.ndarray:
    """``[N, S, D]`` round trip along axis 1, float16 (``quantizers/_quant_utils.py:171-215``)."""
    x32 = np.asarray(x).astype(f32)
    codes, scale, zero = kivi.quant_keys(x32[None], gs, (1 << b) - 1)
    return kivi.dequant_keys(codes, scale, zero, gs)[0].astype(np.float16)


def hi_mask_from_variance_batched(variance: np.ndarray, hi_fraction: float) -> np.ndarray:
    n, d = variance.shape
    n_hi = max(1, int(d * hi_fraction))
    order = np.argsort(-variance, axis=-1, kind="stable")
    rank = np.argsort(order, axis=-1, kind="stable")
    return rank < n_hi


def quantize_mixed_channels_batched(keys, hi_mask, hi_bit=4, lo_bit=2, group_size=32) -> np.ndarray:
    hi = group_quant_dequant_batched(keys, hi_bit, group_size)
    lo = group_quant_dequant_batched(keys, lo_bit, group_size)
    return np.where(hi_mask[:, None, :], hi, lo).astype(np.float16)


def compute_running_variance(key_sum, key_sq_sum, n: int) -> np.ndarray:
    if n < 2:
        return np.zeros_like(key_sum)
    mean = (key_sum / f32(n)).astype(f32)
    return np.maximum((key_sq_sum / f32(n)).astype(f32) - (mean * mean).astype(f32), f32(0.0)).astype(f32)


class KittyCacheModel:
    def __init__(self, head_dim, hi_fraction=0.25, hi_bit=4, lo_bit=2, group_size=32):
        self.D, self.hi_fraction, self.hi_bit, self.lo_bit, self.gs = head_dim, hi_fraction, hi_bit, lo_bit, group_size
        self.key_sum = self.key_sq_sum = None
        self.n_keys = 0
        self.keys = self.values = None
        self.compressed_key_bytes = self.fp16_key_bytes = self.value_fp16_bytes = 0

    def update_and_fetch(self, keys, values):
        B, H, S, D = keys.shape
        flat = keys.reshape(B * H, S, D)
        if self.n_keys == 0:
            variance = np.var(flat.astype(f32), axis=1)
        else:
            var_h = compute_running_variance(self.key_sum, self.key_sq_sum, self.n_keys)
            variance = np.broadcast_to(var_h[None], (B, H, D)).reshape(B * H, D)
        mask = hi_mask_from_variance_batched(variance, self.hi_fraction)
        k_out = quantize_mixed_channels_batched(flat, mask, self.hi_bit, self.lo_bit, self.gs).reshape(B, H, S, D)
        k32 = k_out.astype(f32)
        k_mean_b = np.mean(k32, axis=0)
        new_sum, new_sq = np.sum(k_mean_b, axis=1), np.sum(k_mean_b * k_mean_b, axis=1)
        if self.key_sum is None:
            self.key_sum, self.key_sq_sum = new_sum, new_sq
        else:
            self.key_sum, self.key_sq_sum = self.key_sum + new_sum, self.key_sq_sum + new_sq
        self.n_keys += S
        n_hi = max(1, int(D * self.hi_fraction))

        def channel_bytes(n_ch, b):
            return (math.ceil(S * n_ch * b / 8) + math.ceil(S / self.gs) * n_ch * 2 * 2) * H * B

        self.compressed_key_bytes += channel_bytes(n_hi, self.hi_bit) + channel_bytes(D - n_hi, self.lo_bit)
        self.fp16_key_bytes += B * H * S * D * 2
        self.value_fp16_bytes += B * H * S * D * 2
        k_store = k_out.astype(keys.dtype)
        self.keys = k_store if self.keys is None else np.concatenate([self.keys, k_store], axis=2)
        self.values = values.copy() if self.values is None else np.concatenate([self.values, values], axis=2)
        return self.keys, self.values

    def trim(self, n: int) -> int:
        """``kitty_cache.py:180-210``: the trimmed rows leave the running statistics and the accounting."""
        old = self.keys.shape[2] if self.keys is not None else 0
        trimmed = min(old, max(int(n), 0))
        if trimmed:
            gone = self.keys[:, :, old - trimmed:old]
            B, H = gone.shape[:2]
            if self.n_keys - trimmed <= 0:
                self.key_sum = self.key_sq_sum = None
                self.n_keys = 0
            else:
                g32 = np.mean(gone.astype(f32), axis=0)
                self.key_sum = self.key_sum - np.sum(g32, axis=1)
                self.key_sq_sum = self.key_sq_sum - np.sum(g32 * g32, axis=1)
                self.n_keys -= trimmed
            n_hi = max(1, int(self.D * self.hi_fraction))

            def channel_bytes(n_ch, b):
                return (math.ceil(trimmed * n_ch * b / 8) + math.ceil(trimmed / self.gs) * n_ch * 2 * 2) * H * B

            self.compressed_key_bytes = max(0, self.compressed_key_bytes - channel_bytes(n_hi, self.hi_bit) - channel_bytes(self.D - n_hi, self.lo_bit))
            self.fp16_key_bytes = max(0, self.fp16_key_bytes - B * H * trimmed * self.D * 2)
            self.value_fp16_bytes = max(0, self.value_fp16_bytes - B * H * trimmed * self.D * 2)
            self.keys, self.values = self.keys[:, :, : old - trimmed], self.values[:, :, : old - trimmed]
        return trimmed
