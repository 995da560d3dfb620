"""Packed TurboQuant-RVQ key cache (method ``turboquant_rvq``).

Interface and storage follow ``TurboQuantRVQKVCache`` (``veloxquant_mlx/cache/
turboquant_rvq_cache.py:129-499``): every key is split into its float32 norm (kept as bfloat16)
and its unit direction, the direction is rotated and residual-quantized in two stages, and the
two code streams are kept bit-packed as uint32 words ``[B, H, cap, n_words]``; values are stored
as they arrive. ``update_and_fetch`` returns the keys dequantized (one fused launch over the
packed streams, read in place) and the raw values: dequantize-on-fetch, as the reference does.
Buffers grow in steps of 256 tokens.
"""

from __future__ import annotations

import dataclasses
from typing import Any

import torch

from . import rvq
from .cache import _CACHE_CLASS_BY_METHOD, KVCacheConfig, QuantizerConfigError, _native_only
from .core import StandaloneProtocol


class TurboQuantRVQKVCache(StandaloneProtocol):
    """Keys as two packed RVQ code streams + a bfloat16 norm per vector; values unchanged."""

    step = 256

    def __init__(self, config: Any) -> None:
        _native_only(config, "TurboQuantRVQKVCache")
        b = config.bit_width_inlier
        if isinstance(b, list):
            raise TypeError("TurboQuantRVQKVCache cannot accept list-form bit_width_inlier; this list-form is consumed by "
                            "KVCacheBuilder.for_model() which dispatches to the per-layer factory.")
        self._head_dim, self._bits, self._seed = int(config.head_dim), int(b), int(getattr(config, "seed", 42))
        self._build_derived_state()
        self._packed1 = self._packed2 = self._norms = None  # [B,H,cap,n_words] uint32 x2, [B,H,cap,1] bf16
        self.values = None
        self.offset = 0

    def _build_derived_state(self) -> None:
        d, b = self._head_dim, self._bits
        if not 1 <= b <= 4:
            raise QuantizerConfigError(f"TurboQuantRVQKVCache: bit_width_inlier={b} must be in 1..4 for packed storage.")
        if d < 32 or d & (d - 1) or d > 1024:
            raise QuantizerConfigError(f"TurboQuantRVQKVCache: head_dim={d} must be a power of two in 32..1024.")
        self._quantizer = rvq.TurboQuantRVQ(d=d, b=b, seed=self._seed, use_hadamard=True)
        self._n_words = rvq.n_words_for(d, b)
        self._key_bytes_compressed = 0
        self._key_bytes_fp16 = 0

    def _grow(self, B: int, H: int, S: int, device, v_dtype, v_dim: int) -> None:
        prev = self.offset
        if self._packed1 is not None and prev + S <= self._packed1.shape[2]:
            return
        extra = -(-(self.step + S - 1) // self.step) * self.step   # (turboquant_rvq_cache.py:222)
        cap = prev + extra

        def grown(old, last, dt):
            t = torch.zeros((B, H, cap, last), dtype=dt, device=device)
            if old is not None and prev:
                t[:, :, :prev] = old[:, :, :prev]
            return t

        self._packed1 = self._grown_u32(self._packed1, B, H, cap, prev, device)
        self._packed2 = self._grown_u32(self._packed2, B, H, cap, prev, device)
        self._norms = grown(self._norms, 1, torch.bfloat16)
        self.values = grown(self.values, v_dim, v_dtype)

    def _grown_u32(self, old, B, H, cap, prev, device):
        # (slice assignment is not implemented for uint32 tensors: copy through the int32 view)
        t = torch.zeros((B, H, cap, self._n_words), dtype=torch.int32, device=device)
        if old is not None and prev:
            t[:, :, :prev] = old.view(torch.int32)[:, :, :prev]
        return t.view(torch.uint32)

    # -- protocol ------------------------------------------------------------------------
    def update_and_fetch(self, keys: torch.Tensor, values: torch.Tensor):
        """Normalize keys to unit vectors + norm, quantize and pack the direction, store the values;
        return the dequantized history of keys and the raw values (``turboquant_rvq_cache.py:244-310``)."""
        if keys.ndim != 4 or values.ndim != 4 or keys.shape[:3] != values.shape[:3]:
            raise ValueError(f"TurboQuantRVQKVCache.update_and_fetch: keys/values must be 4D with equal leading shapes, got "
                             f"{tuple(keys.shape)} / {tuple(values.shape)}")
        B, H, S, D = keys.shape
        if D != self._head_dim:
            raise QuantizerConfigError(f"TurboQuantRVQKVCache: expected head_dim {self._head_dim}, got {D}.")
        prev = self.offset
        self._grow(B, H, S, keys.device, values.dtype, values.shape[3])
        k32 = keys.reshape(-1, D).float()
        norms = torch.linalg.vector_norm(k32, dim=-1, keepdim=True)
        k_unit = (k32 / norms.clamp_min(1e-4)).to(torch.float16)
        p1, p2 = self._quantizer.encode_pack(k_unit)
        self.offset += S
        sl = slice(prev, self.offset)
        self._packed1.view(torch.int32)[:, :, sl] = p1.view(torch.int32).reshape(B, H, S, self._n_words)
        self._packed2.view(torch.int32)[:, :, sl] = p2.view(torch.int32).reshape(B, H, S, self._n_words)
        self._norms[:, :, sl] = norms.reshape(B, H, S, 1).to(torch.bfloat16)
        self.values[:, :, sl] = values
        self._key_bytes_compressed += (2 * self._n_words * 4 + 2) * H * B * S
        self._key_bytes_fp16 += H * B * S * D * 2
        return self._dequantize_live(keys.dtype), self.values[:, :, : self.offset]

    def _dequantize_live(self, dtype) -> torch.Tensor:
        B, H, cap, nw = self._packed1.shape
        n = self.offset
        if n == 0:
            return torch.zeros((B, H, 0, self._head_dim), dtype=dtype, device=self._packed1.device)
        k = self._quantizer.decode_packed(self._packed1.reshape(B * H, cap, nw), self._packed2.reshape(B * H, cap, nw),
                                          self._norms.reshape(B * H, cap, 1), seq_len=n)
        return k.reshape(B, H, n, self._head_dim).to(dtype)

    def fused_sdpa(self, q: torch.Tensor, scale: float, *, causal: bool = True, sliding_window: int = 0) -> torch.Tensor:
        """Attention of ``q [B,H_q,S_q,D]`` over the cache: keys are dequantized on fetch (the reference's
        cache has no fused attention either; its prototype kernel is not wired in,
        ``metal/_rvq_attend.py:97-104``) and PyTorch's attention runs over them."""
        if sliding_window:
            raise ValueError("TurboQuantRVQKVCache.fused_sdpa: sliding_window is not supported")
        if self.offset == 0:
            raise RuntimeError("TurboQuantRVQKVCache.fused_sdpa: the cache is empty")
        k = self._dequantize_live(q.dtype)
        v = self.values[:, :, : self.offset].to(q.dtype)
        rep = q.shape[1] // k.shape[1]
        if rep > 1:
            k, v = k.repeat_interleave(rep, dim=1), v.repeat_interleave(rep, dim=1)
        S_q, S_kv = q.shape[2], k.shape[2]
        mask = None
        if causal and S_q > 1:
            pos = torch.arange(S_kv - S_q, S_kv, device=q.device)[:, None]
            mask = torch.arange(S_kv, device=q.device)[None, :] <= pos
        return torch.nn.functional.scaled_dot_product_attention(q, k, v, attn_mask=mask, scale=float(scale))

    def check_status(self) -> None:
        """Nothing to report: these kernels have no device-side waits."""

    # -- trim / state --------------------------------------------------------------------
    def is_trimmable(self) -> bool:
        return True

    def trim(self, n: int) -> int:
        old = self.offset
        n = int(min(old, max(n, 0)))
        self.offset -= n
        if n and old:
            keep = self.offset / old
            self._key_bytes_compressed = int(self._key_bytes_compressed * keep)
            self._key_bytes_fp16 = int(self._key_bytes_fp16 * keep)
        return n

    def empty(self) -> bool:
        return self._packed1 is None

    def size(self) -> int:
        return self.offset

    def _reset_tokens(self) -> None:
        self.offset = 0
        self._key_bytes_compressed = self._key_bytes_fp16 = 0

    @property
    def state(self):
        """``(packed1, packed2, norms, values)``: the stored (not reconstructed) live rows. The packed
        streams are handed out as int32 bit patterns (safetensors and slicing both know int32)."""
        if self._packed1 is None:
            return (None, None, None, None)
        n = self.offset
        return (self._packed1.view(torch.int32)[:, :, :n].contiguous(), self._packed2.view(torch.int32)[:, :, :n].contiguous(),
                self._norms[:, :, :n].contiguous(), self.values[:, :, :n].contiguous())

    @state.setter
    def state(self, v) -> None:
        p1, p2, norms, values = v
        if p1 is None:
            self._packed1 = self._packed2 = self._norms = self.values = None
            self.offset = 0
            return
        as_u32 = lambda t: (t if t.dtype == torch.uint32 else t.view(torch.uint32)).contiguous()  # noqa: E731
        self._packed1, self._packed2, self._norms, self.values = as_u32(p1), as_u32(p2), norms.contiguous(), values.contiguous()
        self.offset = self._packed1.shape[2]

    @property
    def meta_state(self):
        """``(head_dim, bits, seed, offset)`` as strings (``turboquant_rvq_cache.py:396-405``)."""
        return tuple(map(str, (self._head_dim, self._bits, self._seed, self.offset)))

    @meta_state.setter
    def meta_state(self, v) -> None:
        self._head_dim, self._bits, self._seed, self.offset = map(int, v)
        self._build_derived_state()

    @classmethod
    def from_state(cls, state, meta_state=None, config=None):
        if meta_state is None:
            raise TypeError("TurboQuantRVQKVCache.from_state() requires meta_state")
        hd, b, seed = (int(x) for x in meta_state[:3])
        cfg = config if config is not None else KVCacheConfig(method="turboquant_rvq")
        obj = cls(dataclasses.replace(cfg, method="turboquant_rvq", head_dim=hd, bit_width_inlier=b, seed=seed))
        obj.state = state
        obj.meta_state = meta_state   # (after state: the stored offset wins over the buffers' length)
        return obj

    @property
    def merge(self):
        raise AttributeError("TurboQuantRVQKVCache does not support merge()")

    # -- accounting ----------------------------------------------------------------------
    @property
    def nbytes(self) -> int:
        n = self.offset
        if n == 0 or self._packed1 is None:
            return 0
        B, H = self._packed1.shape[:2]
        return B * H * n * (2 * self._n_words * 4 + 2 + self.values.shape[3] * self.values.element_size())

    @property
    def compressed_key_bytes(self) -> int:
        return self._key_bytes_compressed

    @property
    def fp16_key_bytes(self) -> int:
        return self._key_bytes_fp16

    @property
    def assigned_bits(self) -> int:
        return self._bits


_CACHE_CLASS_BY_METHOD["turboquant_rvq"] = TurboQuantRVQKVCache

__all__ = ["TurboQuantRVQKVCache"]
