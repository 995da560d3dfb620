"""Caches whose keys are scored without reconstruction: ``VecInferKVCache`` (product-VQ
indices, reference ``cache/vecinfer_cache.py``) and ``RaBitQKVCache`` (1-bit sign codes; the
reference has the quantizer and kernels but no cache class, ``cache/base.py:60-104``).
"""

from __future__ import annotations

import math
import warnings
from typing import Any

import torch

from . import rabitq as rq
from . import vecinfer as vi
from .cache import QuantizerConfigError, _CACHE_CLASS_BY_METHOD, _native_only
from .core import StandaloneProtocol

_SMOOTH_FLOOR = 1e-8


def _grow(old, shape, dtype, device):
    t = torch.zeros(shape, dtype=dtype, device=device)
    if old is not None and old.shape[2] > 0:
        t[:, :, : old.shape[2]] = old
    return t


class _VQByteAccounting:
    """Byte and token counters of the reference's VecInfer cache: estimated packed bytes of the index
    streams and their float16 equivalents, added per append (``cache/vecinfer_cache.py:653-664``),
    scaled with the token count on ``trim`` (``:627-637``), read through the reference's properties
    (``:736-761``). Needs ``_key_sub_dim``, ``_value_sub_dim``, ``_key_bits``, ``_value_bits``."""

    def _reset_bytes(self) -> None:
        self._key_bytes_compressed = self._value_bytes_compressed = 0
        self._key_bytes_fp16 = self._value_bytes_fp16 = 0
        self._tokens_seen = 0

    def _account_bytes(self, B: int, H: int, S: int, D: int) -> None:
        k_bits_per_tok = (D // self._key_sub_dim) * self._key_bits
        v_bits_per_tok = (D // self._value_sub_dim) * self._value_bits
        self._key_bytes_compressed += math.ceil(k_bits_per_tok / 8) * H * B * S
        self._value_bytes_compressed += math.ceil(v_bits_per_tok / 8) * H * B * S
        self._key_bytes_fp16 += H * B * S * D * 2
        self._value_bytes_fp16 += H * B * S * D * 2
        self._tokens_seen += S

    def _scale_bytes(self, keep: float) -> None:
        for name in ("_key_bytes_compressed", "_value_bytes_compressed", "_key_bytes_fp16", "_value_bytes_fp16", "_tokens_seen"):
            setattr(self, name, int(getattr(self, name) * keep))

    @property
    def compressed_key_bytes(self) -> int:
        return self._key_bytes_compressed

    @property
    def fp16_key_bytes(self) -> int:
        return self._key_bytes_fp16

    @property
    def compressed_value_bytes(self) -> int:
        return self._value_bytes_compressed

    @property
    def fp16_value_bytes(self) -> int:
        return self._value_bytes_fp16

    @property
    def codebook_bytes(self) -> int:
        """Both codebooks at two bytes an entry."""
        return (2 ** self._key_bits) * self._key_sub_dim * 2 + (2 ** self._value_bits) * self._value_sub_dim * 2


class VecInferKVCache(_VQByteAccounting, StandaloneProtocol):
    """Keys dual-transformed (smooth + Hadamard) and product-VQ coded on append; values
    product-VQ coded. Only codebook indices are stored (one byte each for <= 256 centroids);
    :meth:`fused_sdpa` attends over them through a per-query lookup table.

    ``update_and_fetch`` returns the dequantized history (the reference's standard mode) or,
    with ``fused_sdpa_memory_bound=True``, empty sentinels (``cache/vecinfer_cache.py:491-532``).
    """

    def __init__(self, config: Any) -> None:
        _native_only(config, "VecInferKVCache")
        self._head_dim = D = int(config.head_dim)
        self._key_sub_dim, self._value_sub_dim = int(config.key_sub_dim), int(config.value_sub_dim)
        self._key_bits, self._value_bits = int(config.key_codebook_bits), int(config.value_codebook_bits)
        if D & (D - 1):
            raise QuantizerConfigError(f"VecInferKVCache: head_dim={D} must be a power of 2 (Hadamard transform).")
        if D % self._key_sub_dim or D % self._value_sub_dim:
            raise QuantizerConfigError(
                f"VecInferKVCache: head_dim={D} must be divisible by key_sub_dim={self._key_sub_dim} "
                f"and value_sub_dim={self._value_sub_dim}.")
        self._smooth = None
        sm = getattr(config, "smooth_factors", None)
        if sm is not None:
            self._smooth = torch.as_tensor(sm, dtype=torch.float32)
            bad = ~(torch.isfinite(self._smooth) & (self._smooth > _SMOOTH_FLOOR))
            if int(bad.sum()):
                raise QuantizerConfigError(
                    f"VecInferKVCache: smooth_factors must be finite and > {_SMOOTH_FLOOR:g}; "
                    f"{int(bad.sum())} of {self._smooth.numel()} entries are zero, negative, non-finite or too small.")
        self._smooth_kv_heads = None
        seed = int(getattr(config, "seed", 42))
        missing = [n for n in ("key_codebook", "value_codebook") if getattr(config, n, None) is None]
        if missing:
            warnings.warn(
                f"VecInferKVCache: no {' / '.join(missing)} given, so random N(0,1) codebooks are used. "
                "They are only meant for shape/wiring tests and distort real keys/values badly.",
                UserWarning, stacklevel=2)

        def codebook(given, n_c, sub, s):
            if given is not None:
                return torch.as_tensor(given).to(torch.float32)
            g = torch.Generator().manual_seed(s)
            return torch.randn((n_c, sub), generator=g, dtype=torch.float32)

        self._key_codebook = codebook(getattr(config, "key_codebook", None), 2 ** self._key_bits, self._key_sub_dim, seed)
        self._value_codebook = codebook(getattr(config, "value_codebook", None), 2 ** self._value_bits,
                                        self._value_sub_dim, seed + 1)
        if self._key_codebook.shape[-1] != self._key_sub_dim or self._value_codebook.shape[-1] != self._value_sub_dim:
            raise QuantizerConfigError("VecInferKVCache: codebook width does not match its sub_dim")
        self._memory_bound = bool(getattr(config, "fused_sdpa_memory_bound", False))
        if self._memory_bound and not getattr(config, "fused_sdpa", False):
            raise RuntimeError("VecInferKVCache: fused_sdpa_memory_bound=True requires fused_sdpa=True -- the "
                               "memory-bound path only exists as a variant of the fused path.")
        cap = getattr(config, "fused_sdpa_max_ctx", None)
        self._max_ctx = None if cap is None else int(cap)
        self._n_sub_k, self._n_sub_v = D // self._key_sub_dim, D // self._value_sub_dim
        self._k_idx = self._v_idx = None
        self._H = None
        self.offset = 0
        self._dtype = None
        self._reset_bytes()

    # ------------------------------------------------------------------ helpers
    def _index_dtype(self, n_c: int):
        return torch.uint8 if n_c <= 256 else torch.int32

    def _to_device(self, device) -> None:
        if self._H is None or self._H.device != device:
            self._H = vi.walsh_hadamard_matrix(self._head_dim, device=device)
            self._key_codebook = self._key_codebook.to(device)
            self._value_codebook = self._value_codebook.to(device)
            if self._smooth is not None:
                self._smooth = self._smooth.to(device)

    def _resolve_smooth_heads(self, n_kv_heads: int) -> None:
        """Rows in {1, H_kv} are used as they are; a multiple of H_kv (factors calibrated
        per query head under GQA) is averaged per KV group; anything else is rejected
        (``cache/vecinfer_cache.py:233-294``)."""
        sm = self._smooth
        if sm is None or sm.ndim != 2 or self._smooth_kv_heads == n_kv_heads:
            return
        rows = int(sm.shape[0])
        if rows not in (1, n_kv_heads):
            if rows > n_kv_heads and rows % n_kv_heads == 0:
                self._smooth = sm.reshape(n_kv_heads, rows // n_kv_heads, sm.shape[-1]).mean(dim=1)
            else:
                raise QuantizerConfigError(
                    f"VecInferKVCache: smooth_factors has {rows} rows but the keys have {n_kv_heads} KV heads. "
                    f"Provide a [1, D], [{n_kv_heads}, D] or a multiple-of-{n_kv_heads}-row smooth.")
        self._smooth_kv_heads = n_kv_heads

    def _smooth_or_ones(self, device):
        return self._smooth if self._smooth is not None else torch.ones(self._head_dim, device=device)

    def _ensure_index_capacity(self, B, H, n_tokens, device) -> None:
        if self._max_ctx is not None and n_tokens > self._max_ctx:
            raise RuntimeError(f"VecInferKVCache: context length {n_tokens} exceeded fused_sdpa_max_ctx={self._max_ctx}.  "
                               "Raise or unset KVCacheConfig.fused_sdpa_max_ctx.")
        cap = 0 if self._k_idx is None else self._k_idx.shape[2]
        if n_tokens <= cap:
            return
        new_cap = max(256, cap)
        while new_cap < n_tokens:
            new_cap *= 2
        if self._max_ctx is not None:
            new_cap = min(new_cap, max(self._max_ctx, n_tokens))
        self._k_idx = _grow(self._k_idx, (B, H, new_cap, self._n_sub_k), self._index_dtype(self._key_codebook.shape[0]), device)
        self._v_idx = _grow(self._v_idx, (B, H, new_cap, self._n_sub_v), self._index_dtype(self._value_codebook.shape[0]), device)

    # ------------------------------------------------------------------ protocol
    def update_and_fetch(self, keys: torch.Tensor, values: torch.Tensor):
        if keys.ndim != 4 or keys.shape != values.shape:
            raise ValueError("VecInferKVCache.update_and_fetch: keys/values must be equal 4D shapes")
        B, H, S, D = keys.shape
        if D != self._head_dim:
            raise QuantizerConfigError(f"VecInferKVCache: expected head_dim {self._head_dim}, got {D}.")
        self._dtype = self._dtype or keys.dtype
        self._to_device(keys.device)
        self._resolve_smooth_heads(H)
        self._ensure_index_capacity(B, H, self.offset + S, keys.device)
        # smooth divide + Walsh-Hadamard butterfly in one native launch, fixed summation order
        k_tilde = vi.dual_transform_keys_wht(keys, self._smooth)
        lo, hi = self.offset, self.offset + S
        self._k_idx[:, :, lo:hi] = vi.quantize_vq(k_tilde, self._key_codebook, self._key_sub_dim, index_dtype=self._k_idx.dtype)
        self._v_idx[:, :, lo:hi] = vi.quantize_vq(values, self._value_codebook, self._value_sub_dim, index_dtype=self._v_idx.dtype)
        self.offset = hi
        self._account_bytes(B, H, S, D)
        if self._memory_bound:
            z = keys.new_zeros((B, H, 0, D))
            return z, z
        return self.dequantized()

    def dequantized(self):
        """``(K_hat, V_hat)`` of the whole history in the activation dtype."""
        n = self.offset
        k_t = vi.dequantize_vq(self._k_idx[:, :, :n].contiguous(), self._key_codebook, out_dtype=torch.float32)
        k_hat = (k_t @ self._H.T) * vi._smooth_for(k_t, self._smooth_or_ones(k_t.device), False, "VecInferKVCache")
        v_hat = vi.dequantize_vq(self._v_idx[:, :, :n].contiguous(), self._value_codebook, out_dtype=self._dtype)
        return k_hat.to(self._dtype), v_hat

    def fused_sdpa(self, q: torch.Tensor, scale: float, *, causal: bool = True, sliding_window: int = 0):
        """``softmax(q K_hat^T * scale) V_hat`` over the stored indices
        (``cache/vecinfer_cache.py:670-731``): the query takes the dual transform, keys are
        scored by table lookup, values are gathered from their codebook."""
        if self.offset == 0:
            raise RuntimeError("VecInferKVCache.fused_sdpa: the cache is empty")
        q_tilde = vi.dual_transform_queries_wht(q, self._smooth)
        return vi.fused_sdpa_vq(q_tilde, self._k_idx, self._key_codebook, self._v_idx, self._value_codebook, scale,
                                causal=causal, sliding_window=sliding_window, out_dtype=q.dtype, s_kv=self.offset)

    def trim(self, n: int) -> int:
        old = self.offset
        n = int(min(max(n, 0), old))
        self.offset -= n
        if n:
            self._scale_bytes(self.offset / old)
        return n

    def _reset_tokens(self) -> None:
        self.offset = 0
        self._reset_bytes()

    def check_status(self) -> None:
        """Raise if a bounded device-side wait of an earlier quantize or attention call ran out."""
        from . import kernels
        kernels.quantize_status()
        kernels.attend_status()

    def is_trimmable(self) -> bool:
        return True

    def empty(self) -> bool:
        return self.offset == 0

    def size(self) -> int:
        return self.offset

    @property
    def state(self):
        if self._k_idx is None:
            return ()
        return (self._k_idx[:, :, : self.offset].contiguous(), self._v_idx[:, :, : self.offset].contiguous())

    @state.setter
    def state(self, st) -> None:
        if not st:
            return
        k, v = st
        B, H, n, _ = k.shape
        self._k_idx = self._v_idx = None
        self._to_device(k.device)
        self._ensure_index_capacity(B, H, n, k.device)
        self._k_idx[:, :, :n], self._v_idx[:, :, :n] = k, v
        self.offset = n

    @property
    def meta_state(self):
        """``(head_dim, key_sub_dim, value_sub_dim, key_codebook_bits, value_codebook_bits, offset)``
        as strings; the codebooks and smooth factors are configuration, not state."""
        return tuple(map(str, (self._head_dim, self._key_sub_dim, self._value_sub_dim, self._key_bits, self._value_bits,
                               self.offset)))

    @meta_state.setter
    def meta_state(self, v) -> None:
        hd, ks, vs, kb, vb, off = (int(x) for x in v)
        mine = (self._head_dim, self._key_sub_dim, self._value_sub_dim, self._key_bits, self._value_bits)
        if (hd, ks, vs, kb, vb) != mine:
            raise QuantizerConfigError(
                f"VecInferKVCache.meta_state: stored indices were made with (head_dim, sub_dims, bits) = {(hd, ks, vs, kb, vb)}, "
                f"this cache is configured with {mine}; indices are only meaningful with their own codebooks")
        if off == 0:
            self._reset_tokens()

    @property
    def merge(self):
        """Not a method but a property that raises ``AttributeError``, as in the reference
        (``cache/vecinfer_cache.py:785-789``): a serving loop that asks ``hasattr(cache, "merge")`` before
        batching caches must be told no, instead of merging them into an uncompressed batch cache."""
        raise AttributeError("VecInferKVCache does not support merge()")

    @property
    def nbytes(self) -> int:
        """Live index bytes (the codebooks are shared constants)."""
        if self._k_idx is None:
            return 0
        B, H = self._k_idx.shape[:2]
        return B * H * self.offset * (self._n_sub_k * self._k_idx.element_size() + self._n_sub_v * self._v_idx.element_size())

    @property
    def assigned_avg_bits(self) -> float:
        return (self._key_bits / self._key_sub_dim + self._value_bits / self._value_sub_dim) / 2.0


class RaBitQKVCache(StandaloneProtocol):
    """1-bit keys (seeded randomized-Hadamard rotation, sign bits, L1 magnitude per key) with
    values kept in the activation dtype -- the pairing the reference documents for RaBitQ
    (``docs-site/docs/algorithms/rabitq.md:12``). Centroid-free: the score of key ``t`` is
    ``(D - 2*hamming(sign(q'), bits_t)) * mean|q'| * mag_t * scale`` with ``q'`` the rotated
    query (``metal/_rabitq_attend.py:10-19``). ``method="rabitq"`` has no reference cache
    class; this one follows the interface of the other caches here.
    """

    def __init__(self, config: Any) -> None:
        _native_only(config, "RaBitQKVCache")
        self._head_dim = D = int(config.head_dim)
        if D & (D - 1) or D % 32 or D > 256:
            raise QuantizerConfigError(f"RaBitQKVCache: head_dim={D} must be a power of 2 in 32..256.")
        self._seed = int(getattr(config, "seed", 42))
        # the keys exist as sign bits only: update_and_fetch always returns sentinels and attention
        # always goes through fused_sdpa, whatever the configuration's flag says
        self._memory_bound = True
        self._diag_np = rq.make_hadamard_diagonal(D, seed=self._seed)
        self._diag = self._H = None
        self._bits = self._mag = self._v = None
        self.offset = 0

    def _to_device(self, device) -> None:
        if self._diag is None or self._diag.device != device:
            self._diag = torch.from_numpy(self._diag_np).to(device)
            self._H = vi.walsh_hadamard_matrix(self._head_dim, device=device)

    def _ensure_capacity(self, B, H, n, v_dtype, device) -> None:
        cap = 0 if self._bits is None else self._bits.shape[2]
        if n <= cap:
            return
        D = self._head_dim
        new_cap = max(256, cap)
        while new_cap < n:
            new_cap *= 2
        self._bits = _grow(self._bits, (B, H, new_cap, D // 8), torch.uint8, device)
        self._mag = _grow(None if self._mag is None else self._mag[..., None], (B, H, new_cap, 1), torch.float32,
                          device)[..., 0].contiguous()
        self._v = _grow(self._v, (B, H, new_cap, D), v_dtype, device)

    def update_and_fetch(self, keys: torch.Tensor, values: torch.Tensor):
        if keys.ndim != 4 or keys.shape != values.shape:
            raise ValueError("RaBitQKVCache.update_and_fetch: keys/values must be equal 4D shapes")
        B, H, S, D = keys.shape
        if D != self._head_dim:
            raise QuantizerConfigError(f"RaBitQKVCache: expected head_dim {self._head_dim}, got {D}.")
        self._to_device(keys.device)
        n = self.offset + S
        self._ensure_capacity(B, H, n, values.dtype, keys.device)
        bits, mag = rq.rabitq_encode(keys.reshape(B * H * S, D), self._diag)
        self._bits[:, :, self.offset : n] = bits.view(B, H, S, D // 8)
        self._mag[:, :, self.offset : n] = mag.view(B, H, S)
        self._v[:, :, self.offset : n] = values
        self.offset = n
        z = keys.new_zeros((B, H, 0, D))
        return z, z

    def fused_sdpa(self, q: torch.Tensor, scale: float, *, causal: bool = True, sliding_window: int = 0):
        """One query row: the popcount estimator of the decode kernel. Several rows (a prompt
        chunk): the tiled kernel, whose scores are exact dots of the rotated query with the
        decoded keys ``signs * mag`` -- the same pairing of two score models as the reference's
        ``rabitq_fused_attend`` / ``rabitq_prefill_attend``; ``causal`` aligns the rows to the
        tail of the cache."""
        if q.ndim != 4:
            raise ValueError(f"RaBitQKVCache.fused_sdpa: q must be 4D, got {tuple(q.shape)}")
        if sliding_window:
            raise ValueError("RaBitQKVCache.fused_sdpa: sliding_window is not supported")
        if self.offset == 0:
            raise RuntimeError("RaBitQKVCache.fused_sdpa: the cache is empty")
        q_rot = vi.dual_transform_queries_wht(q, self._diag)  # = WHT(q*diag)/sqrt(D), native butterfly
        if q.shape[2] > 1:
            if causal and q.shape[2] > self.offset:
                raise ValueError(f"RaBitQKVCache.fused_sdpa: {q.shape[2]} query rows but only {self.offset} cached tokens")
            return rq.rabitq_prefill_attend(q_rot.to(torch.float16), float(scale), self._bits, self._mag, None, self._v, None,
                                            causal=bool(causal), s_kv=self.offset, out_dtype=q.dtype)
        q_scale = q_rot.abs().mean(dim=-1) * float(scale)
        return rq.rabitq_fused_attend(q_rot, q_scale, self._bits, self._mag, None, self._v, None, s_kv=self.offset,
                                      out_dtype=q.dtype)

    def trim(self, n: int) -> int:
        n = int(min(max(n, 0), self.offset))
        self.offset -= n
        return n

    def _reset_tokens(self) -> None:
        self.offset = 0

    def check_status(self) -> None:
        """Raise if a bounded device-side wait of an earlier attention call ran out."""
        from . import kernels
        kernels.attend_status()

    def is_trimmable(self) -> bool:
        return True

    def empty(self) -> bool:
        return self.offset == 0

    def size(self) -> int:
        return self.offset

    @property
    def state(self):
        n = self.offset
        return () if self._bits is None else (self._bits[:, :, :n].contiguous(), self._mag[:, :, :n].contiguous(),
                                              self._v[:, :, :n].contiguous())

    @state.setter
    def state(self, st) -> None:
        if not st:
            return
        bits, mag, v = st
        self._to_device(bits.device)
        B, H, n = bits.shape[:3]
        # the same capacity rule as a cache that grew to n tokens by appends (the attention kernel
        # picks its path by the buffers' row pitch, so a restored cache must not differ there)
        self._bits = self._mag = self._v = None
        self._ensure_capacity(B, H, n, v.dtype, bits.device)
        self._bits[:, :, :n], self._mag[:, :, :n], self._v[:, :, :n] = bits, mag, v
        self.offset = n

    @property
    def meta_state(self):
        """``(head_dim, rotation seed, offset)`` as strings: the sign bits are only meaningful with
        the rotation they were made with."""
        return tuple(map(str, (self._head_dim, self._seed, self.offset)))

    @meta_state.setter
    def meta_state(self, v) -> None:
        hd, seed, off = (int(x) for x in v)
        if hd != self._head_dim:
            raise QuantizerConfigError(f"RaBitQKVCache.meta_state: stored head_dim {hd}, configured {self._head_dim}")
        if seed != self._seed:
            self._seed = seed
            self._diag_np = rq.make_hadamard_diagonal(hd, seed=seed)
            self._diag = self._H = None
        if off == 0:
            self._reset_tokens()

    @property
    def nbytes(self) -> int:
        if self._bits is None:
            return 0
        B, H = self._bits.shape[:2]
        return B * H * self.offset * (self._head_dim // 8 + 4 + self._head_dim * self._v.element_size())

    @property
    def assigned_avg_bits(self) -> float:
        return 1.0


_CACHE_CLASS_BY_METHOD["vecinfer"] = VecInferKVCache
_CACHE_CLASS_BY_METHOD["rabitq"] = RaBitQKVCache

__all__ = ["VecInferKVCache", "RaBitQKVCache"]
