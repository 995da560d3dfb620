"""Kitty cache (method ``kitty``) and AgeTieredKV cache (method ``age_tiered``): the two remaining
group-affine sibling methods, on the native group-quantization kernel.

``KittyKVCache`` follows ``veloxquant_mlx/cache/kitty_cache.py:49-256``: keys are round-tripped per
call with the top-variance channels at ``kitty_hi_bit`` and the rest at ``kitty_lo_bit`` (ranking
from the block itself on the first call, from running statistics of the stored keys afterwards),
values pass through. Like the reference it stores the round-tripped keys densely (a one-token
decode block is its own quantization group, i.e. is stored exactly, so there is nothing to pack).

``AgeTieredKVCache`` follows ``veloxquant_mlx/cache/age_tiered_cache.py:38-388``: every
position-aligned group of ``age_group_size`` tokens is one round trip of its RAW rows at the width of
its tier (recent / mid / old, by the age of the group's first token). The reference keeps a raw
copy of every token for that. Here a group that has reached the last tier and is full is final:
its raw rows are dropped and it is kept as packed codes with float32 (scale, zero) (the KIVI key
format, for keys and values alike); raw rows are kept only for the younger groups (at most
``age_mid_boundary + age_group_size`` tokens). ``update_and_fetch`` returns the same tensors as the
reference's dense bookkeeping.
"""

from __future__ import annotations

import math
from typing import Any

import torch

from . import age_tiered as at
from . import kernels, kitty
from .cache import _CACHE_CLASS_BY_METHOD, QuantizerConfigError, _native_only
from .core import StandaloneProtocol


def _sdpa_dense(q, k, v, scale, causal):
    rep = q.shape[1] // k.shape[1]
    if rep > 1:
        k, v = k.repeat_interleave(rep, dim=1), v.repeat_interleave(rep, dim=1)
    S_q, S_kv = q.shape[2], k.shape[2]
    mask = None
    if causal and S_q > 1:
        pos = torch.arange(S_kv - S_q, S_kv, device=q.device)[:, None]
        mask = torch.arange(S_kv, device=q.device)[None, :] <= pos
    return torch.nn.functional.scaled_dot_product_attention(q, k.to(q.dtype), v.to(q.dtype), attn_mask=mask, scale=float(scale))


class KittyKVCache(StandaloneProtocol):
    """Mixed-precision keys by channel variance; values unchanged. No ``.bits`` attribute."""

    step = 256

    def __init__(self, config: Any) -> None:
        _native_only(config, "KittyKVCache")
        self._D = self._head_dim = int(config.head_dim)
        self._hi_fraction = float(getattr(config, "kitty_hi_fraction", 0.25))
        if not 0.0 <= self._hi_fraction <= 1.0:
            raise QuantizerConfigError(f"kitty: kitty_hi_fraction must be in [0, 1], got {self._hi_fraction}")
        self._hi_bit = int(getattr(config, "kitty_hi_bit", 4))
        self._lo_bit = int(getattr(config, "kitty_lo_bit", 2))
        self._group_size = int(getattr(config, "kitty_group_size", 32))
        for name, b in (("kitty_hi_bit", self._hi_bit), ("kitty_lo_bit", self._lo_bit)):
            if not 1 <= b <= 8:
                raise QuantizerConfigError(f"kitty: {name}={b} must be in [1, 8] for the native kernels")
        if self._group_size < 1:
            raise QuantizerConfigError(f"kitty: kitty_group_size={self._group_size} must be >= 1")
        self._reset_tokens()

    def _reset_tokens(self) -> None:
        self.keys = self.values = None
        self.offset = 0
        self._key_sum = self._key_sq_sum = None
        self._n_keys = 0
        self._compressed_key_bytes = self._fp16_key_bytes = self._value_fp16_bytes = 0

    def _quantize_keys(self, keys: torch.Tensor) -> torch.Tensor:
        B, H, S, D = keys.shape
        flat = keys.reshape(B * H, S, D)
        if self._n_keys == 0:
            variance = torch.var(flat.float(), dim=1, unbiased=False)
        else:
            var_h = kitty.compute_running_variance(self._key_sum, self._key_sq_sum, self._n_keys)
            variance = var_h[None].expand(B, H, D).reshape(B * H, D)
        mask = kitty.hi_mask_from_variance_batched(variance, self._hi_fraction)
        return kitty.quantize_mixed_channels_batched(flat, mask, self._hi_bit, self._lo_bit, self._group_size).reshape(B, H, S, D)

    def _update_accumulators(self, k_out: torch.Tensor) -> None:
        k_mean_b = k_out.float().mean(dim=0)                      # [H, S, D]
        new_sum, new_sq = k_mean_b.sum(dim=1), (k_mean_b * k_mean_b).sum(dim=1)
        if self._key_sum is None:
            self._key_sum, self._key_sq_sum = new_sum, new_sq
        else:
            self._key_sum, self._key_sq_sum = self._key_sum + new_sum, self._key_sq_sum + new_sq
        self._n_keys += k_out.shape[2]

    def _key_bytes_for(self, n_tokens: int, B: int, H: int) -> int:
        n_hi = max(1, int(self._D * self._hi_fraction))

        def channel_bytes(n_ch: int, b: int) -> int:
            return (math.ceil(n_tokens * n_ch * b / 8) + math.ceil(n_tokens / self._group_size) * n_ch * 2 * 2) * H * B

        return channel_bytes(n_hi, self._hi_bit) + channel_bytes(self._D - n_hi, self._lo_bit)

    def update_and_fetch(self, keys: torch.Tensor, values: torch.Tensor):
        if keys.ndim != 4 or values.ndim != 4 or keys.shape[:3] != values.shape[:3]:
            raise ValueError(f"KittyKVCache.update_and_fetch: keys/values must be 4D with equal leading shapes, got "
                             f"{tuple(keys.shape)} / {tuple(values.shape)}")
        B, H, S, D = keys.shape
        if D != self._D:
            raise QuantizerConfigError(f"KittyKVCache: expected head_dim {self._D}, got {D}.")
        k_out = self._quantize_keys(keys)
        self._update_accumulators(k_out)      # the statistics see what is stored
        self._compressed_key_bytes += self._key_bytes_for(S, B, H)
        self._fp16_key_bytes += B * H * S * D * 2
        self._value_fp16_bytes += B * H * S * D * 2
        prev = self.offset
        if self.keys is None or prev + S > self.keys.shape[2]:
            cap = prev + -(-(self.step + S - 1) // self.step) * self.step
            nk = torch.zeros((B, H, cap, D), dtype=keys.dtype, device=keys.device)
            nv = torch.zeros((B, H, cap, values.shape[3]), dtype=values.dtype, device=values.device)
            if prev:
                nk[:, :, :prev], nv[:, :, :prev] = self.keys[:, :, :prev], self.values[:, :, :prev]
            self.keys, self.values = nk, nv
        self.keys[:, :, prev:prev + S] = k_out.to(keys.dtype)
        self.values[:, :, prev:prev + S] = values
        self.offset += S
        return self.keys[:, :, : self.offset], self.values[:, :, : self.offset]

    def fused_sdpa(self, q, scale, *, causal: bool = True, sliding_window: int = 0):
        """PyTorch's attention over the stored (round-tripped) keys: the reference has no fused kernel here either."""
        if sliding_window:
            raise ValueError("KittyKVCache.fused_sdpa: sliding_window is not supported")
        if self.offset == 0:
            raise RuntimeError("KittyKVCache.fused_sdpa: the cache is empty")
        return _sdpa_dense(q, self.keys[:, :, : self.offset], self.values[:, :, : self.offset], scale, causal)

    def check_status(self) -> None:
        """Nothing to report: these kernels have no device-side waits."""

    def is_trimmable(self) -> bool:
        return True

    def trim(self, n: int) -> int:
        """Drop the last ``n`` tokens; their contribution leaves the running statistics and the byte
        accounting (``kitty_cache.py:180-210``)."""
        old = self.offset
        trimmed = min(old, max(int(n), 0))
        if trimmed and self.keys is not None:
            gone = self.keys[:, :, old - trimmed:old]
            B, H = gone.shape[0], gone.shape[1]
            if self._n_keys - trimmed <= 0:
                self._key_sum = self._key_sq_sum = None
                self._n_keys = 0
            else:
                g32 = gone.float().mean(dim=0)
                self._key_sum = self._key_sum - g32.sum(dim=1)
                self._key_sq_sum = self._key_sq_sum - (g32 * g32).sum(dim=1)
                self._n_keys -= trimmed
            self._compressed_key_bytes = max(0, self._compressed_key_bytes - self._key_bytes_for(trimmed, B, H))
            self._fp16_key_bytes = max(0, self._fp16_key_bytes - B * H * trimmed * self._D * 2)
            self._value_fp16_bytes = max(0, self._value_fp16_bytes - B * H * trimmed * self._D * 2)
        self.offset -= trimmed
        return trimmed

    def empty(self) -> bool:
        return self.keys is None

    def size(self) -> int:
        return self.offset

    @property
    def state(self):
        if self.keys is None:
            return (None, None, None, None)
        n = self.offset
        return (self.keys[:, :, :n].contiguous(), self.values[:, :, :n].contiguous(), self._key_sum, self._key_sq_sum)

    @state.setter
    def state(self, v) -> None:
        self.keys, self.values, self._key_sum, self._key_sq_sum = v
        self.offset = 0 if self.keys is None else self.keys.shape[2]

    @property
    def meta_state(self):
        return tuple(map(str, (self._D, repr(self._hi_fraction), self._hi_bit, self._lo_bit, self._group_size, self._n_keys,
                               self._compressed_key_bytes, self._fp16_key_bytes, self._value_fp16_bytes)))

    @meta_state.setter
    def meta_state(self, v) -> None:
        self._D = self._head_dim = int(v[0])
        self._hi_fraction = float(v[1])
        (self._hi_bit, self._lo_bit, self._group_size, self._n_keys, self._compressed_key_bytes, self._fp16_key_bytes,
         self._value_fp16_bytes) = (int(x) for x in v[2:9])

    @property
    def nbytes(self) -> int:
        if self.keys is None:
            return 0
        B, H = self.keys.shape[:2]
        return B * H * self.offset * (self._D * self.keys.element_size() + self.values.shape[3] * self.values.element_size())

    compressed_key_bytes = property(lambda self: self._compressed_key_bytes)
    fp16_key_bytes = property(lambda self: self._fp16_key_bytes)
    value_fp16_bytes = property(lambda self: self._value_fp16_bytes)
    hi_fraction = property(lambda self: self._hi_fraction)
    hi_bit = property(lambda self: self._hi_bit)
    lo_bit = property(lambda self: self._lo_bit)
    group_size = property(lambda self: self._group_size)

    @property
    def assigned_avg_bits(self) -> float:
        n_hi = max(1, int(self._D * self._hi_fraction))
        return (n_hi * self._hi_bit + (self._D - n_hi) * self._lo_bit) / self._D


class AgeTieredKVCache(StandaloneProtocol):
    """Three precision tiers by token age; final (oldest-tier, full) groups packed, younger rows raw."""

    def __init__(self, config: Any) -> None:
        _native_only(config, "AgeTieredKVCache")
        self._age_recent_boundary = int(getattr(config, "age_recent_boundary", 128))
        self._age_mid_boundary = int(getattr(config, "age_mid_boundary", 1024))
        if self._age_recent_boundary <= 0:
            raise QuantizerConfigError(f"AgeTieredKVCache: age_recent_boundary must be > 0, got {self._age_recent_boundary}.")
        if self._age_mid_boundary < self._age_recent_boundary:
            raise QuantizerConfigError(f"AgeTieredKVCache: age_mid_boundary ({self._age_mid_boundary}) must be >= "
                                       f"age_recent_boundary ({self._age_recent_boundary}).")
        bits = tuple(int(getattr(config, n, d)) for n, d in (("age_bits_recent", 8), ("age_bits_mid", 4), ("age_bits_old", 2)))
        for name, b in zip(("age_bits_recent", "age_bits_mid", "age_bits_old"), bits):
            if not 1 <= b <= 16:
                raise QuantizerConfigError(f"AgeTieredKVCache: {name} must be in [1, 16], got {b}.")
            if 8 < b < 16:
                raise QuantizerConfigError(f"AgeTieredKVCache: {name}={b}: the native kernels quantize at 1..8 bits (16 = keep as is).")
        self._tiers = at.default_age_tiers(*bits)
        self._group_size = int(getattr(config, "age_group_size", 32))
        if self._group_size < 1:
            raise QuantizerConfigError(f"AgeTieredKVCache: age_group_size={self._group_size} must be >= 1")
        self._head_dim = int(getattr(config, "head_dim", 128))
        self._reset_tokens()

    def _reset_tokens(self) -> None:
        self._B = self._H = 0
        self._final = None      # {"k": (codes, scale, zero), "v": ...} of the final groups, [1, G, n_final, *]
        self._n_final = 0       # tokens in final groups (a multiple of the group size)
        self._raw_k = self._raw_v = None   # [G, n - n_final, D]: raw rows of the younger groups
        self.offset = 0
        self._tokens_seen_total = self._current_position = 0
        self._age_tiered_bytes = self._full_seq_bytes = 0
        self._dtype = torch.float16
        self._last = None       # what the last update_and_fetch returned (fused_sdpa attends over it)

    def _tier_list(self, n: int):
        return at.assign_age_tiers([self._current_position - (i + 1) for i in range(n)], self._age_recent_boundary, self._age_mid_boundary)

    def _pack_final(self, rows_k: torch.Tensor, rows_v: torch.Tensor) -> None:
        """Append whole groups that reached the last tier to the packed store (quantized from raw)."""
        bits, gs = self._tiers[at.OLD].bits, self._group_size
        n_new = rows_k.shape[1]
        if self._final is None:
            self._final = {}
        for name, rows in (("k", rows_k), ("v", rows_v)):
            q = kernels.kivi_quantize(rows[None].contiguous(), -2, gs, bits, eps=1e-8)   # codes per token, (scale, zero) per group
            have = self._final.get(name)
            per = (1, gs, gs)                                   # tokens per row of (codes, scale, zero)
            if have is None or any((self._n_final + n_new) // p > t.shape[2] for t, p in zip(have, per)):
                # grow geometrically: the store is appended to every group_size tokens
                cap = max(2 * (self._n_final + n_new), 64 * gs)
                grown = tuple(torch.empty((*t.shape[:2], cap // p, t.shape[3]), dtype=t.dtype, device=t.device) for t, p in zip(q, per))
                if have is not None:
                    for g, t, p in zip(grown, have, per):
                        g[:, :, : self._n_final // p] = t[:, :, : self._n_final // p]
                have = self._final[name] = grown
            for t, new, p in zip(have, q, per):
                t[:, :, self._n_final // p:(self._n_final + n_new) // p] = new
        self._n_final += n_new

    def _dense_final(self, which: str) -> torch.Tensor:
        gs, n = self._group_size, self._n_final
        codes, scale, zero = (t[:, :, : n // p].contiguous() for t, p in zip(self._final[which], (1, gs, gs)))
        bits = self._tiers[at.OLD].bits
        # float32 reconstruction rounded to float16, then to the storage dtype: the reference's two casts
        out = kernels.scalar_decode_once(codes, scale, zero, self._group_size, "K", store_bits=kernels.storage_bits(bits),
                                         out_dtype=torch.float16)
        return out[0].to(self._dtype)

    def update_and_fetch(self, keys: torch.Tensor, values: torch.Tensor):
        if keys.ndim != 4 or values.ndim != 4 or keys.shape != values.shape:
            raise ValueError(f"AgeTieredKVCache.update_and_fetch: keys/values must be 4D with equal shapes, got "
                             f"{tuple(keys.shape)} / {tuple(values.shape)}")
        B, H, S, D = keys.shape
        if self._raw_k is None and self._final is None:
            self._B, self._H = B, H
            self._dtype = torch.bfloat16 if keys.dtype == values.dtype == torch.bfloat16 else torch.float16
        self._full_seq_bytes += at.full_fp16_bytes(B * H * S, D)
        self._tokens_seen_total += B * H * S
        self._current_position += S
        G, gs = B * H, self._group_size
        k_step, v_step = keys.reshape(G, S, D).to(self._dtype), values.reshape(G, S, D).to(self._dtype)
        self._raw_k = k_step if self._raw_k is None else torch.cat([self._raw_k, k_step], dim=1)
        self._raw_v = v_step if self._raw_v is None else torch.cat([self._raw_v, v_step], dim=1)
        self.offset += S
        n = self.offset
        tiers = self._tier_list(n)
        n_groups = -(-n // gs)
        group_tier = [tiers[g * gs] for g in range(n_groups)]
        # groups that are full and in the last tier leave the raw window for the packed store
        old_bits = self._tiers[at.OLD].bits
        g0 = self._n_final // gs
        g1 = g0
        while old_bits <= 8 and g1 < n_groups and group_tier[g1] == at.OLD and (g1 + 1) * gs <= n:
            g1 += 1
        if g1 > g0:
            cut = (g1 - g0) * gs
            self._pack_final(self._raw_k[:, :cut], self._raw_v[:, :cut])
            self._raw_k, self._raw_v = self._raw_k[:, cut:].contiguous(), self._raw_v[:, cut:].contiguous()
        counts = {t: tiers.count(t) * G for t in (at.RECENT, at.MID, at.OLD)}
        self._age_tiered_bytes = at.age_tiered_bytes(counts, self._tiers, self._head_dim)
        self._last = self._dense_view()
        return self._last[0], self._last[1]

    def _dense_view(self):
        """``(keys, values)`` ``[B, H, offset, D]``: final groups dequantized, younger groups round-tripped at their tier."""
        gs, n = self._group_size, self.offset
        tiers = self._tier_list(n)
        group_tier = [tiers[g * gs] for g in range(-(-n // gs))]
        outs = []
        for which, raw in (("k", self._raw_k), ("v", self._raw_v)):
            parts = []
            if self._n_final:
                parts.append(self._dense_final(which))
            if raw is not None and raw.shape[1]:
                parts.append(at.age_tier_quantize_batched(raw, group_tier[self._n_final // gs:], self._tiers, gs))
            outs.append((parts[0] if len(parts) == 1 else torch.cat(parts, dim=1)).reshape(self._B, self._H, n, self._head_dim))
        return outs

    def fused_sdpa(self, q, scale, *, causal: bool = True, sliding_window: int = 0):
        """PyTorch's attention over what the last ``update_and_fetch`` returned."""
        if sliding_window:
            raise ValueError("AgeTieredKVCache.fused_sdpa: sliding_window is not supported")
        if self.offset == 0:
            raise RuntimeError("AgeTieredKVCache.fused_sdpa: the cache is empty")
        if getattr(self, "_last", None) is None:      # (restored from state: rebuild what update_and_fetch would have returned)
            self._last = self._dense_view()
        return _sdpa_dense(q, self._last[0], self._last[1], scale, causal)

    def check_status(self) -> None:
        """Nothing to report: these kernels have no device-side waits."""

    def is_trimmable(self) -> bool:
        """False: the per-group tier state does not follow a rolled-back offset (``age_tiered_cache.py:335-341``)."""
        return False

    def empty(self) -> bool:
        return self.offset == 0

    def size(self) -> int:
        return self.offset

    @property
    def nbytes(self) -> int:
        """Resident bytes: packed final groups with float32 parameters, raw rows of the younger groups."""
        total = 0
        if self._final is not None:
            gs, n = self._group_size, self._n_final
            total += sum(t.shape[0] * t.shape[1] * (n // p) * t.shape[3] * t.element_size()
                         for bufs in self._final.values() for t, p in zip(bufs, (1, gs, gs)))
        for t in (self._raw_k, self._raw_v):
            if t is not None:
                total += t.numel() * t.element_size()
        return total

    @property
    def state(self):
        """The stored tensors: packed codes, scale, zero of the final groups (keys, then values; live
        rows), then the raw rows of the younger groups (keys, values)."""
        if self.offset == 0:
            return (None,) * 8
        gs, n = self._group_size, self._n_final
        packed = [None] * 6
        if n:
            packed = [t[:, :, : n // p].contiguous() for name in ("k", "v") for t, p in zip(self._final[name], (1, gs, gs))]
        return (*packed, self._raw_k, self._raw_v)

    @state.setter
    def state(self, v) -> None:
        kc, ks, kz, vc, vs, vz, rk, rv = v
        self._final = None if kc is None else {"k": (kc, ks, kz), "v": (vc, vs, vz)}
        self._n_final = 0 if kc is None else kc.shape[2]
        self._raw_k, self._raw_v = rk, rv
        self.offset = self._n_final + (0 if rk is None else rk.shape[1])
        if rk is not None:
            self._dtype = rk.dtype
        self._last = None

    @property
    def meta_state(self):
        """Configuration and counters as strings."""
        return tuple(map(str, (self._head_dim, self._age_recent_boundary, self._age_mid_boundary, *(t.bits for t in self._tiers),
                               self._group_size, self._B, self._H, self._tokens_seen_total, self._current_position,
                               self._age_tiered_bytes, self._full_seq_bytes, "bfloat16" if self._dtype == torch.bfloat16 else "float16")))

    @meta_state.setter
    def meta_state(self, v) -> None:
        (self._head_dim, self._age_recent_boundary, self._age_mid_boundary, b0, b1, b2, self._group_size, self._B, self._H,
         self._tokens_seen_total, self._current_position, self._age_tiered_bytes, self._full_seq_bytes) = (int(x) for x in v[:13])
        self._tiers = at.default_age_tiers(b0, b1, b2)
        self._dtype = torch.bfloat16 if v[13] == "bfloat16" else torch.float16

    age_tiered_bytes = property(lambda self: self._age_tiered_bytes)
    full_seq_bytes = property(lambda self: self._full_seq_bytes)
    tokens_seen = property(lambda self: self._tokens_seen_total)
    tokens_kept = property(lambda self: self.offset)

    @property
    def compression_ratio(self) -> float:
        return 1.0 if self._age_tiered_bytes == 0 else self._full_seq_bytes / self._age_tiered_bytes

    def _tier_count(self, tier: int) -> int:
        if self.offset == 0:
            return 0
        return self._tier_list(self.offset).count(tier) * self._B * self._H

    tokens_recent = property(lambda self: self._tier_count(at.RECENT))
    tokens_mid = property(lambda self: self._tier_count(at.MID))
    tokens_old = property(lambda self: self._tier_count(at.OLD))

    @property
    def merge(self):
        raise AttributeError("AgeTieredKVCache does not support merge()")


_CACHE_CLASS_BY_METHOD["kitty"] = KittyKVCache
_CACHE_CLASS_BY_METHOD["age_tiered"] = AgeTieredKVCache

__all__ = ["KittyKVCache", "AgeTieredKVCache"]
