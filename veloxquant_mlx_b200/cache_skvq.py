"""SKVQ cache (method ``skvq``): sliding full-precision window, per-head channel reordering and
clipped per-token group quantization of everything that ages out of the window.

Interface, flush policy and accounting follow ``SKVQKVCache`` (``veloxquant_mlx/cache/
skvq_cache.py:69-403``): tokens accumulate unquantized; every time ``skvq_window`` tokens lie past
the quantized frontier, that chunk is quantized once and frozen (so one prefill and token-by-token
decode give the same state); the first chunk also fixes the per-head channel permutations (kept
only where they lower that chunk's round-trip error) and its first ``skvq_n_sink`` rows stay exact.

What differs from the reference is the storage: the reference overwrites its dense buffer with the
dequantized round trip, this cache keeps the packed codes and float32 ``(lo, scale)`` of the
frozen region and dequantizes on fetch (one launch per tensor, channel order restored inside it),
so ``update_and_fetch`` returns the same dense tensors while the resident bytes are the packed ones.
"""

from __future__ import annotations

import dataclasses
from typing import Any

import torch

from . import skvq
from .cache import _CACHE_CLASS_BY_METHOD, KVCacheConfig, QuantizerConfigError, _native_only
from .core import StandaloneProtocol


class SKVQKVCache(StandaloneProtocol):
    """Packed SKVQ cache of one layer. Never exposes ``.bits`` (see ``assigned_avg_bits``)."""

    step = 256   # growth granularity of the packed buffers, in tokens

    def __init__(self, config: Any) -> None:
        _native_only(config, "SKVQKVCache")
        self._D = self._head_dim = int(config.head_dim)
        self._bits_k = int(getattr(config, "skvq_bits_key", 4))
        self._bits_v = int(getattr(config, "skvq_bits_value", 4))
        self._group_size = int(getattr(config, "skvq_group_size", 32))
        self._window = int(getattr(config, "skvq_window", 128))
        self._n_sink = int(getattr(config, "skvq_n_sink", 5))
        self._reorder = bool(getattr(config, "skvq_reorder", True))
        self._clip_search = bool(getattr(config, "skvq_clip_search", True))
        self._clip_alpha = float(getattr(config, "skvq_clip_alpha", 1.0))
        max_ctx = getattr(config, "skvq_max_ctx", None)
        self._max_ctx = None if max_ctx is None else int(max_ctx)
        self._validate()
        self._alphas = skvq.DEFAULT_ALPHA_GRID if self._clip_search else (self._clip_alpha,)
        self._packed = None        # {"k": (codes, lo, scale), "v": ...}: [B*H, cap, *] buffers of the frozen region
        self._tail_k = self._tail_v = None   # [B, H, tail_cap, D]: tokens past the frontier, as they arrived
        self._sink_k = self._sink_v = None   # [B, H, n_sink, D]: exact first rows (set by chunk 0's flush)
        self._perm_k = self._inv_k = self._perm_v = self._inv_v = None
        self._q_end = 0
        self.offset = 0
        self._compressed_key_bytes = self._compressed_value_bytes = 0
        self._fp16_key_bytes = self._fp16_value_bytes = 0
        self._tokens_seen = 0
        self._B = self._H = 1
        self._device, self._dtype = None, torch.float16

    def _validate(self) -> None:
        for name, b in (("skvq_bits_key", self._bits_k), ("skvq_bits_value", self._bits_v)):
            if not (1 <= b <= 8):
                raise QuantizerConfigError(f"SKVQKVCache: {name}={b} must be in [1, 8] (uint8 codes)")
        if self._group_size < 1:
            raise QuantizerConfigError(f"SKVQKVCache: skvq_group_size={self._group_size} must be >= 1")
        if self._window < 2:
            raise QuantizerConfigError(f"SKVQKVCache: skvq_window={self._window} must be >= 2 (the first chunk supplies the "
                                       f"channel statistics)")
        if not (0 <= self._n_sink < self._window):
            raise QuantizerConfigError(f"SKVQKVCache: skvq_n_sink={self._n_sink} must be in [0, skvq_window) so sinks live "
                                       f"entirely inside chunk 0")
        if not (0.0 < self._clip_alpha <= 1.0):
            raise QuantizerConfigError(f"SKVQKVCache: skvq_clip_alpha={self._clip_alpha} must be in (0, 1]")
        if self._group_size not in (8, 16, 32, 64) or self._D % self._group_size:
            raise QuantizerConfigError(f"SKVQKVCache: skvq_group_size={self._group_size} must be 8, 16, 32 or 64 and divide "
                                       f"head_dim={self._D} for the packed kernels")

    # -- buffers ---------------------------------------------------------------------------
    def _grow_packed(self, n_bh: int, need: int, device) -> None:
        have = 0 if self._packed is None else self._packed["k"][0].shape[1]
        if need <= have:
            return
        cap = -(-need // self.step) * self.step
        G = self._D // self._group_size
        new = {}
        for name, bits in (("k", self._bits_k), ("v", self._bits_v)):
            bufs = (torch.zeros((n_bh, cap, self._D * bits // 8), dtype=torch.uint8, device=device),
                    torch.zeros((n_bh, cap, G), dtype=torch.float32, device=device),
                    torch.zeros((n_bh, cap, G), dtype=torch.float32, device=device))
            if self._packed is not None and self._q_end:
                for t, old in zip(bufs, self._packed[name]):
                    t[:, : self._q_end] = old[:, : self._q_end]
            new[name] = bufs
        self._packed = new

    def _grow_tail(self, B: int, H: int, need: int, n_live: int, like_k: torch.Tensor, like_v: torch.Tensor) -> None:
        """Room for ``need`` waiting rows; the first ``n_live`` of the old buffer are kept."""
        have = 0 if self._tail_k is None else self._tail_k.shape[2]
        if need <= have:
            return
        cap = max(need, self._window)
        tk = torch.empty((B, H, cap, self._D), dtype=like_k.dtype, device=like_k.device)
        tv = torch.empty((B, H, cap, like_v.shape[3]), dtype=like_v.dtype, device=like_v.device)
        if n_live:
            tk[:, :, :n_live] = self._tail_k[:, :, :n_live]
            tv[:, :, :n_live] = self._tail_v[:, :, :n_live]
        self._tail_k, self._tail_v = tk, tv

    # -- quantization ----------------------------------------------------------------------
    def _per_head_perms(self, chunk: torch.Tensor, bits: int):
        """Candidate: a head's channels sorted by dynamic range over the first chunk's non-sink rows;
        kept only where it lowers the head's round-trip error on those rows, ties keep the identity
        (``skvq_cache.py:137-175``)."""
        B, H, r, D = chunk.shape
        x = chunk[:, :, self._n_sink:, :].float().contiguous()
        xh = x.transpose(0, 1).reshape(H, -1, D)
        rng = xh.amax(dim=1) - xh.amin(dim=1)
        cand = torch.argsort(rng, dim=-1, stable=True).to(torch.int32)
        cand_inv = torch.argsort(cand.long(), dim=-1, stable=True).to(torch.int32)
        flat = x.reshape(B * H, r - self._n_sink, D)

        def err(p, i):
            packed = skvq.quantize_pack(flat, bits, self._group_size, self._alphas, perm=p)
            rt = skvq.unpack_dequant(*packed, bits, self._group_size, flat.shape[1], torch.float32, inv_perm=i)
            d = rt - flat
            return (d * d).double().reshape(B, H, -1).mean(dim=(0, 2))

        keep = (err(cand.contiguous(), cand_inv.contiguous()) < err(None, None))[:, None]
        identity = torch.arange(D, dtype=torch.int32, device=chunk.device)[None, :].expand(H, D)
        return torch.where(keep, cand, identity).contiguous(), torch.where(keep, cand_inv, identity).contiguous()

    def _flush(self, k_rows: torch.Tensor, v_rows: torch.Tensor) -> None:
        """Quantize whole chunks ``[B, H, m*window, D]`` (views with contiguous rows) at the frontier."""
        B, H, n, D = k_rows.shape
        r = self._window
        if self._q_end == 0:
            if self._reorder:
                self._perm_k, self._inv_k = self._per_head_perms(k_rows[:, :, :r], self._bits_k)
                self._perm_v, self._inv_v = self._per_head_perms(v_rows[:, :, :r], self._bits_v)
            if self._n_sink > 0:
                self._sink_k = k_rows[:, :, : self._n_sink].clone()
                self._sink_v = v_rows[:, :, : self._n_sink].clone()
        self._grow_packed(B * H, self._q_end + n, k_rows.device)
        for rows, name, bits, perm in ((k_rows, "k", self._bits_k, self._perm_k), (v_rows, "v", self._bits_v, self._perm_v)):
            skvq.quantize_pack(rows.reshape(B * H, n, D), bits, self._group_size, self._alphas, perm=perm,
                               out=self._packed[name], tok_offset=self._q_end)
        for c in range(n // r):
            n_q = r - (self._n_sink if self._q_end == 0 and c == 0 else 0)
            self._compressed_key_bytes += skvq.skvq_compressed_bytes(n_q, D, self._bits_k, self._group_size) * B * H
            self._compressed_value_bytes += skvq.skvq_compressed_bytes(n_q, D, self._bits_v, self._group_size) * B * H
        self._q_end += n

    # -- protocol ------------------------------------------------------------------------
    def update_and_fetch(self, keys: torch.Tensor, values: torch.Tensor):
        """Append the block, freeze every completed chunk, return the dense history
        (``skvq_cache.py:199-254``)."""
        if keys.ndim != 4 or values.ndim != 4 or keys.shape != values.shape:
            raise ValueError(f"SKVQKVCache.update_and_fetch: keys/values must be 4D with equal shapes, got "
                             f"{tuple(keys.shape)} / {tuple(values.shape)}")
        B, H, S, D = keys.shape
        if D != self._D:
            raise QuantizerConfigError(f"SKVQKVCache: expected head_dim {self._D}, got {D}.")
        if self._max_ctx is not None and self.offset + S > self._max_ctx:
            raise ValueError(f"SKVQKVCache: context {self.offset + S} exceeds skvq_max_ctx={self._max_ctx}")
        self._B, self._H, self._device, self._dtype = B, H, keys.device, keys.dtype
        keys, values = keys.contiguous(), values.contiguous()
        r = self._window
        n_tail = self.offset - self._q_end
        pos = 0
        if n_tail and n_tail + S >= r:
            # complete the chunk that the waiting rows started, and freeze it
            take = r - n_tail
            self._grow_tail(B, H, r, n_tail, keys, values)
            self._tail_k[:, :, n_tail:r] = keys[:, :, :take]
            self._tail_v[:, :, n_tail:r] = values[:, :, :take]
            self._flush(self._tail_k[:, :, :r], self._tail_v[:, :, :r])
            pos, n_tail = take, 0
        whole = ((S - pos) // r) * r if n_tail == 0 else 0
        if whole:
            # chunks that lie inside the incoming block are frozen straight from it; the first chunk
            # ever goes alone (its rows decide the permutations the others are quantized with)
            if self._q_end == 0 and whole > r:
                self._flush(keys[:, :, pos:pos + r], values[:, :, pos:pos + r])
                pos, whole = pos + r, whole - r
            self._flush(keys[:, :, pos:pos + whole], values[:, :, pos:pos + whole])
            pos += whole
        rest = S - pos
        if rest:
            self._grow_tail(B, H, n_tail + rest, n_tail, keys, values)
            self._tail_k[:, :, n_tail:n_tail + rest] = keys[:, :, pos:]
            self._tail_v[:, :, n_tail:n_tail + rest] = values[:, :, pos:]
        self.offset += S
        self._fp16_key_bytes += B * H * S * D * 2
        self._fp16_value_bytes += B * H * S * D * 2
        self._tokens_seen += S
        return self._dense("k", keys.dtype), self._dense("v", values.dtype)

    def _dense(self, which: str, dtype) -> torch.Tensor:
        """``[B, H, offset, D]``: the frozen region dequantized (sink rows exact), then the waiting rows."""
        tail = self._tail_k if which == "k" else self._tail_v
        B, H, D, n, q = self._B, self._H, self._D, self.offset, self._q_end
        out = torch.empty((B, H, n, D), dtype=dtype, device=self._device)
        if q:
            bits, inv = (self._bits_k, self._inv_k) if which == "k" else (self._bits_v, self._inv_v)
            skvq.unpack_dequant(*self._packed[which], bits, self._group_size, q, dtype, inv_perm=inv,
                                out=out[:, :, :q].reshape(B * H, q, D) if n == q else out.reshape(B * H, n, D)[:, :q])
            if self._n_sink:
                out[:, :, : self._n_sink] = self._sink_k if which == "k" else self._sink_v
        if n > q:
            out[:, :, q:] = tail[:, :, : n - q]
        return out

    @property
    def keys(self):
        return None if self.offset == 0 else self._dense("k", self._dtype)

    @property
    def values(self):
        return None if self.offset == 0 else self._dense("v", self._dtype)

    def fused_sdpa(self, q: torch.Tensor, scale: float, *, causal: bool = True, sliding_window: int = 0) -> torch.Tensor:
        """Attention of ``q [B,H_q,S_q,D]`` over the cache. The reference has no fused attention for
        this method (its cache hands dense tensors to the stock attention); neither has this one:
        the history is dequantized on fetch and PyTorch's attention runs over it."""
        if sliding_window:
            raise ValueError("SKVQKVCache.fused_sdpa: sliding_window is not supported")
        if self.offset == 0:
            raise RuntimeError("SKVQKVCache.fused_sdpa: the cache is empty")
        k, v = self._dense("k", q.dtype), self._dense("v", q.dtype)
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
        """False: a frozen chunk cannot be un-quantized, and the frontier and the permutations
        fixed by the first chunk would not follow a rolled-back offset (``skvq_cache.py:357-376``)."""
        return False

    def empty(self) -> bool:
        return self.offset == 0

    def size(self) -> int:
        return self.offset

    def _reset_tokens(self) -> None:
        self._packed = self._tail_k = self._tail_v = self._sink_k = self._sink_v = None
        self._perm_k = self._inv_k = self._perm_v = self._inv_v = None
        self._q_end = self.offset = 0
        self._compressed_key_bytes = self._compressed_value_bytes = 0
        self._fp16_key_bytes = self._fp16_value_bytes = self._tokens_seen = 0

    @property
    def state(self):
        """The stored (not reconstructed) tensors: packed codes, lo, scale of keys and values
        (live rows), the waiting rows, the exact sink rows, the two permutations."""
        if self.offset == 0:
            return (None,) * 12
        q, n_tail = self._q_end, self.offset - self._q_end
        packed = [None] * 6 if not q else [t[:, :q].contiguous() for t in (*self._packed["k"], *self._packed["v"])]
        tails = [None, None] if not n_tail else [self._tail_k[:, :, :n_tail].contiguous(), self._tail_v[:, :, :n_tail].contiguous()]
        return (*packed, *tails, self._sink_k, self._sink_v, self._perm_k, self._perm_v)

    @state.setter
    def state(self, v) -> None:
        kc, klo, ksc, vc, vlo, vsc, tk, tv, sk, sv, pk, pv = v
        self._packed = None if kc is None else {"k": (kc.contiguous(), klo.contiguous(), ksc.contiguous()),
                                                "v": (vc.contiguous(), vlo.contiguous(), vsc.contiguous())}
        self._tail_k, self._tail_v, self._sink_k, self._sink_v = tk, tv, sk, sv
        self._perm_k = None if pk is None else pk.to(torch.int32).contiguous()
        self._perm_v = None if pv is None else pv.to(torch.int32).contiguous()
        self._inv_k = None if pk is None else torch.argsort(self._perm_k.long(), dim=-1, stable=True).to(torch.int32).contiguous()
        self._inv_v = None if pv is None else torch.argsort(self._perm_v.long(), dim=-1, stable=True).to(torch.int32).contiguous()
        self._q_end = 0 if kc is None else kc.shape[1]
        self.offset = self._q_end + (0 if tk is None else tk.shape[2])
        ref = tk if tk is not None else sk
        if ref is not None:
            self._B, self._H, self._dtype = ref.shape[0], ref.shape[1], ref.dtype
        any_t = next((t for t in v if t is not None), None)
        if any_t is not None:
            self._device = any_t.device

    @property
    def meta_state(self):
        """Configuration and counters as strings."""
        return tuple(map(str, (self._D, self._bits_k, self._bits_v, self._group_size, self._window, self._n_sink,
                               int(self._reorder), int(self._clip_search), repr(self._clip_alpha), self._B, self._H,
                               self._compressed_key_bytes, self._compressed_value_bytes, self._fp16_key_bytes,
                               self._fp16_value_bytes, self._tokens_seen)))

    @meta_state.setter
    def meta_state(self, v) -> None:
        (self._D, self._bits_k, self._bits_v, self._group_size, self._window, self._n_sink) = (int(x) for x in v[:6])
        self._head_dim = self._D
        self._reorder, self._clip_search, self._clip_alpha = bool(int(v[6])), bool(int(v[7])), float(v[8])
        (self._B, self._H, self._compressed_key_bytes, self._compressed_value_bytes, self._fp16_key_bytes,
         self._fp16_value_bytes, self._tokens_seen) = (int(x) for x in v[9:16])
        self._validate()
        self._alphas = skvq.DEFAULT_ALPHA_GRID if self._clip_search else (self._clip_alpha,)

    @classmethod
    def from_state(cls, state, meta_state=None, config=None):
        if meta_state is None:
            raise TypeError("SKVQKVCache.from_state() requires meta_state")
        cfg = config if config is not None else KVCacheConfig(method="skvq")
        obj = cls(dataclasses.replace(cfg, method="skvq", head_dim=int(meta_state[0]), skvq_group_size=int(meta_state[3]),
                                      skvq_window=int(meta_state[4]), skvq_n_sink=int(meta_state[5])))
        obj.meta_state = meta_state
        obj.state = state
        return obj

    @property
    def merge(self):
        raise AttributeError("SKVQKVCache does not support merge()")

    # -- accounting ----------------------------------------------------------------------
    @property
    def nbytes(self) -> int:
        """Bytes resident for the live tokens: packed codes and float32 (lo, scale) of the frozen
        region, the waiting rows, the exact sink rows, the permutations."""
        total = 0
        if self._packed is not None and self._q_end:
            for bufs in self._packed.values():
                total += sum(t.shape[0] * self._q_end * t.shape[2] * t.element_size() for t in bufs)
        n_tail = self.offset - self._q_end
        if n_tail:
            total += n_tail * (self._tail_k[:, :, :1].numel() * self._tail_k.element_size()
                               + self._tail_v[:, :, :1].numel() * self._tail_v.element_size())
        for t in (self._sink_k, self._sink_v, self._perm_k, self._inv_k, self._perm_v, self._inv_v):
            if t is not None:
                total += t.numel() * t.element_size()
        return total

    @property
    def compressed_key_bytes(self) -> int:
        return self._compressed_key_bytes

    @property
    def compressed_value_bytes(self) -> int:
        return self._compressed_value_bytes

    @property
    def fp16_key_bytes(self) -> int:
        return self._fp16_key_bytes

    @property
    def fp16_value_bytes(self) -> int:
        return self._fp16_value_bytes

    @property
    def residual_fp16_bytes(self) -> int:
        """Bytes held unquantized (keys + values): the waiting rows plus the sink rows (``skvq_cache.py:296-303``)."""
        n_res = self.offset - self._q_end
        return skvq.skvq_fp16_bytes(n_res + min(self._n_sink, self._q_end), self._D) * 2 * self._B * self._H

    @property
    def perm_bytes(self) -> int:
        if self._perm_k is None and self._perm_v is None:
            return 0
        return 2 * self._H * self._D * 4

    @property
    def quantized_tokens(self) -> int:
        return self._q_end

    @property
    def tokens_seen(self) -> int:
        return self._tokens_seen

    @property
    def key_perms(self):
        return self._perm_k

    @property
    def value_perms(self):
        return self._perm_v

    @property
    def assigned_avg_bits(self) -> float:
        n_q = self._q_end - min(self._n_sink, self._q_end)
        if n_q == 0:
            return 16.0
        return 8.0 * self._compressed_key_bytes / (n_q * self._D * self._B * self._H)


_CACHE_CLASS_BY_METHOD["skvq"] = SKVQKVCache

__all__ = ["SKVQKVCache"]
