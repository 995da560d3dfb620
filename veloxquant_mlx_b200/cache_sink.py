"""Sink-protected KIVI cache (method ``kivi_sink``) on the packed store.

Interface and policy follow ``SinkProtectedKVCache`` (``veloxquant_mlx/cache/sink_cache.py``):
per batch element a running top-``n_sink_tokens`` of token positions by key L2 norm (mean over
the KV heads) is kept; when a block of rows ages out of the residual window, the rows that are
sinks of their batch element are replaced by their nearest non-sink row before the group
parameters are computed, and the sinks themselves stay exact.

The reference holds a dense fp16 buffer and writes the exact rows back into it. Here the history
stays packed, so a protected token is represented three ways:

* its slot in the packed store holds the codes of the neighbour copy (what the reference
  quantizes in its place) with the value scale and zero-point set to 0: the slot adds nothing
  to ``P.V``;
* its exact key and value rows sit in a small side buffer ``[B, H, rows, D]`` and are attended as
  extra tail rows;
* the dequantized key of the slot (float32) sits beside them and is attended with weight -1, which
  removes the slot's share of the softmax sum.

Everything the selection needs runs on the device without a host round trip (a stable sort for
the running top-k, cumulative max / min for the nearest non-sink row, scatters with a spare row for
entries that do not apply); appending synchronises only when the side buffer's conservative row
bound reaches its capacity, and the reporting properties (``sink_positions``, byte counts) read
device values back.
"""

from __future__ import annotations

import dataclasses
from typing import Any

import torch

from . import kernels
from .cache import _CACHE_CLASS_BY_METHOD, KIVIKVCache, KVCacheConfig, QuantizerConfigError


class SinkProtectedKVCache(KIVIKVCache):
    """KIVI cache that keeps the ``n_sink_tokens`` highest-key-norm tokens of every batch
    element exact (``cache/sink_cache.py:43-76``). ``n_sink_tokens = 0`` is plain KIVI."""

    def __init__(self, config: Any) -> None:
        super().__init__(config)
        self._n_sink = int(getattr(config, "n_sink_tokens", 5))
        if self._n_sink < 0:
            raise QuantizerConfigError(f"SinkProtectedKVCache: n_sink_tokens={self._n_sink} must be >= 0.")
        if self._n_sink > 1024:
            raise QuantizerConfigError(f"SinkProtectedKVCache: n_sink_tokens={self._n_sink} exceeds the supported 1024.")
        self._clear_sinks()

    def _clear_sinks(self) -> None:
        self._sink_pos = None      # [B, n_sink] int64 absolute positions of the candidates, -1 = none
        self._sink_norm = None     # [B, n_sink] float32, -inf = none
        self._fs_k = self._fs_v = self._fs_kdead = None  # [B, H, cap + 1, D]: flushed sinks (+ one spare row)
        self._fs_pos = None        # [B, cap + 1] int64
        self._fs_count = None      # [B] int32 rows in use
        self._fs_cap = 0
        self._fs_upper = 0         # host-side upper bound of max(_fs_count)
        self._acct = None          # device int64 [3]: corrections to the compressed key / value bytes, sink bytes
        self._blk_sinks = None     # 0-d int64: sinks inside the block flushed last (max over the batch)

    # -- sink bookkeeping ----------------------------------------------------------------
    def _update_sinks(self, keys: torch.Tensor, start: int) -> None:
        """Fold the block's per-token key norms into every batch element's running top-k
        (``sink_cache.py:83-107``): a stable descending sort keeps earlier entries on ties."""
        B, _, S, _ = keys.shape
        dev = keys.device
        if self._sink_pos is None or self._sink_pos.shape[0] != B:
            self._sink_pos = torch.full((B, self._n_sink), -1, dtype=torch.int64, device=dev)
            self._sink_norm = torch.full((B, self._n_sink), float("-inf"), dtype=torch.float32, device=dev)
        per_tok = torch.linalg.vector_norm(keys.float(), dim=-1).mean(dim=1)  # [B, S]
        cand_norm = torch.cat([self._sink_norm, per_tok], dim=1)
        cand_pos = torch.cat([self._sink_pos, torch.arange(start, start + S, device=dev).expand(B, S)], dim=1)
        order = torch.sort(cand_norm, dim=1, descending=True, stable=True).indices[:, : self._n_sink]
        self._sink_norm = torch.gather(cand_norm, 1, order)
        self._sink_pos = torch.gather(cand_pos, 1, order)

    def _ensure_sink_rows(self, B, H, D, rows, device, dtype) -> None:
        if self._fs_k is not None and rows <= self._fs_cap:
            return
        cap = max(4 * max(self._n_sink, 1), self._fs_cap)
        while cap < rows:
            cap *= 2

        def grow(old, shape, dt, fill=0):
            t = torch.full(shape, fill, dtype=dt, device=device)
            if old is not None:
                n = old.shape[-2] - 1 if old.ndim == 4 else old.shape[-1] - 1
                if old.ndim == 4:
                    t[:, :, :n] = old[:, :, :n]
                else:
                    t[:, :n] = old[:, :n]
            return t

        self._fs_k = grow(self._fs_k, (B, H, cap + 1, D), dtype)
        self._fs_v = grow(self._fs_v, (B, H, cap + 1, D), dtype)
        self._fs_kdead = grow(self._fs_kdead, (B, H, cap + 1, D), torch.float32)
        self._fs_pos = grow(self._fs_pos, (B, cap + 1), torch.int64, -1)
        if self._fs_count is None:
            self._fs_count = torch.zeros(B, dtype=torch.int32, device=device)
            self._acct = torch.zeros(3, dtype=torch.int64, device=device)
        self._fs_cap = cap
        self._version += 1

    def _quantize_rows(self, src_k, src_v, n_flush) -> None:
        if self._n_sink == 0 or self._sink_pos is None:
            return super()._quantize_rows(src_k, src_v, n_flush)
        B, H, _, D = src_k.shape
        dev, n, lo, g = src_k.device, int(n_flush), self._n_quantized, self._group_size
        kb, vb = src_k[:, :, :n], src_v[:, :, :n]
        local = self._sink_pos - lo
        in_blk = (local >= 0) & (local < n)                                  # [B, n_sink]
        mask = torch.zeros((B, n + 1), dtype=torch.bool, device=dev)
        mask.scatter_(1, torch.where(in_blk, local, n), True)
        mask = mask[:, :n]                                                   # [B, n]: row is a sink of its batch element
        # nearest non-sink row: to the left first, else to the right (sink_cache.py:148-163)
        idx = torch.arange(n, device=dev).expand(B, n)
        left = torch.where(mask, -1, idx).cummax(dim=1).values
        right = torch.where(mask, n, idx).flip(1).cummin(dim=1).values.flip(1)
        src = torch.where(mask, torch.where(left >= 0, left, torch.where(right < n, right, idx)), idx)
        sel = src[:, None, :, None].expand(B, H, n, D)
        super()._quantize_rows(torch.gather(kb, 2, sel), torch.gather(vb, 2, sel), n)
        # the slots of the sinks add nothing to P.V
        live = (~mask).to(torch.float32)[:, None, :, None]
        self._v_scale[:, :, lo : lo + n] *= live
        self._v_zero[:, :, lo : lo + n] *= live
        # exact rows and the dequantized keys of the slots go to the side buffer
        need = self._fs_upper + min(self._n_sink, n)
        if need > self._fs_cap and self._fs_count is not None:
            # the bound counts every flush as if all candidates lay inside it: before growing the
            # buffer, replace it by the true count (the one read-back of the append path, once per
            # capacity / n_sink flushes)
            self._fs_upper = int(self._fs_count.max().item())
            need = self._fs_upper + min(self._n_sink, n)
        self._ensure_sink_rows(B, H, D, need, dev, kb.dtype)
        self._fs_upper = need
        k_hat = kernels.scalar_decode_once(self._k_codes[:, :, lo : lo + n].contiguous(),
                                           self._k_scale[:, :, lo // g : (lo + n) // g].contiguous(),
                                           self._k_zero[:, :, lo // g : (lo + n) // g].contiguous(), g, "K",
                                           store_bits=self._sb, out_dtype=torch.float32)
        rows = local.clamp(0, n - 1)[:, None, :, None].expand(B, H, self._n_sink, D)
        rank = in_blk.to(torch.int64).cumsum(dim=1) - 1
        dest = torch.where(in_blk, self._fs_count.to(torch.int64)[:, None] + rank, self._fs_cap)  # (spare row otherwise)
        dsel = dest[:, None, :, None].expand(B, H, self._n_sink, D)
        self._fs_k.scatter_(2, dsel, torch.gather(kb, 2, rows))
        self._fs_v.scatter_(2, dsel, torch.gather(vb, 2, rows))
        self._fs_kdead.scatter_(2, dsel, torch.gather(k_hat, 2, rows))
        self._fs_pos.scatter_(1, dest, self._sink_pos)
        per_b = in_blk.sum(dim=1)
        self._fs_count += per_b.to(torch.int32)
        self._blk_sinks = per_b.max()

    # -- protocol ------------------------------------------------------------------------
    def update_and_fetch(self, keys: torch.Tensor, values: torch.Tensor, *, overlap_previous: bool = False):
        """``KIVIKVCache.update_and_fetch`` after the block's key norms have been folded into the
        sink candidates (``sink_cache.py:112-190``). ``overlap_previous`` is accepted and ignored:
        the selection runs ordinary kernels in front of the append."""
        if self._n_sink and keys.ndim == 4:
            self._update_sinks(keys, self.offset)
        return super().update_and_fetch(keys, values)

    def _attend_sinks(self):
        if not self._n_sink or self._fs_k is None or self._n_quantized == 0:
            return None
        return (self._fs_k, self._fs_v, self._fs_kdead, self._fs_count)

    def fused_sdpa(self, q, scale, *, causal=True, sliding_window=0, out=None, overlap_previous=False, gather=None):
        if q.ndim == 4 and q.shape[2] > 1 and self._attend_sinks() is not None:
            raise ValueError("SinkProtectedKVCache.fused_sdpa: one query row per call once tokens have been quantized "
                             "(attend a longer block over update_and_fetch's dense view)")
        return super().fused_sdpa(q, scale, causal=causal, sliding_window=sliding_window, out=out,
                                  overlap_previous=overlap_previous, gather=gather)

    def _materialize(self):
        k, v = super()._materialize()
        if self._attend_sinks() is None:
            return k, v
        # exact rows back into the dense view (one spare row takes the unused entries)
        B, H, D = self._shape_bhd
        n = k.shape[2]
        cap = self._fs_cap
        valid = torch.arange(cap, device=k.device)[None, :] < self._fs_count[:, None]
        dest = torch.where(valid, self._fs_pos[:, :cap], n)[:, None, :, None].expand(B, H, cap, D)
        pad = k.new_zeros((B, H, 1, D))
        k = torch.cat([k, pad], dim=2).scatter_(2, dest, self._fs_k[:, :, :cap])[:, :, :n]
        v = torch.cat([v, pad], dim=2).scatter_(2, dest, self._fs_v[:, :, :cap])[:, :, :n]
        return k, v

    def trim(self, n: int) -> int:
        """``KIVIKVCache.trim`` plus the sinks (``sink_cache.py:192-218``): flushed sinks of the
        rolled-back groups leave the side buffer (those that survive the trim return to the
        residual window as their exact rows), candidates at discarded positions are dropped."""
        old_nq = self._n_quantized
        trimmed = super().trim(n)
        if not trimmed or not self._n_sink or self._sink_pos is None:
            return trimmed
        new_nq = self._n_quantized
        if new_nq < old_nq and self._fs_k is not None:
            B, H, D = self._shape_bhd
            cap = self._fs_cap
            pos = self._fs_pos[:, :cap]
            valid = torch.arange(cap, device=pos.device)[None, :] < self._fs_count[:, None]
            back = valid & (pos >= new_nq) & (pos < self.offset)
            if self._n_res:
                spare = self._k_res.shape[2] - 1  # (beyond the live rows: the window was moved to the front)
                dest = torch.where(back, pos - new_nq, spare)[:, None, :, None].expand(B, H, cap, D)
                self._k_res.scatter_(2, dest, self._fs_k[:, :, :cap])
                self._v_res.scatter_(2, dest, self._fs_v[:, :, :cap])
            leave = valid & (pos >= new_nq)
            gone = leave.sum(dim=1)
            # the rows that stay move to the front (a flush of several groups stores its sinks in
            # candidate order, not position order, so the rows that leave need not be the last)
            order = torch.sort((~valid | leave).to(torch.int8), dim=1, stable=True).indices
            osel = order[:, None, :, None].expand(B, H, cap, D)
            self._fs_k[:, :, :cap] = torch.gather(self._fs_k[:, :, :cap], 2, osel)
            self._fs_v[:, :, :cap] = torch.gather(self._fs_v[:, :, :cap], 2, osel)
            self._fs_kdead[:, :, :cap] = torch.gather(self._fs_kdead[:, :, :cap], 2, osel)
            self._fs_pos[:, :cap] = torch.gather(pos, 1, order)
            self._fs_count -= gone.to(torch.int32)
            B_, H_ = self._shape_bhd[0], self._shape_bhd[1]
            s = gone.max()
            n_rolled = old_nq - new_nq
            k0, v0 = self._quantized_bytes_dev(torch.full_like(s, n_rolled), B_, H_, D)
            k1, v1 = self._quantized_bytes_dev(n_rolled - s, B_, H_, D)
            self._acct += torch.stack([k0 - k1, v0 - v1, -s * D * 2 * 2 * H_ * B_])
        dropped = self._sink_pos >= self.offset
        self._sink_pos = torch.where(dropped, -1, self._sink_pos)
        self._sink_norm = torch.where(dropped, float("-inf"), self._sink_norm)
        return trimmed

    def _reset_tokens(self) -> None:
        super()._reset_tokens()
        self._clear_sinks()
        self._version += 1

    # -- state ---------------------------------------------------------------------------
    @property
    def state(self):
        base = KIVIKVCache.state.fget(self)
        if not base or not self._n_sink or self._sink_pos is None:
            return base
        B, H, D = self._shape_bhd
        if self._fs_k is None:
            self._ensure_sink_rows(B, H, D, 1, self._sink_pos.device, self._dtype)
        u = max(self._fs_upper, 1)
        return (*base, self._sink_pos, self._sink_norm, self._fs_pos[:, :u].contiguous(), self._fs_count,
                self._fs_k[:, :, :u].contiguous(), self._fs_v[:, :, :u].contiguous(), self._fs_kdead[:, :, :u].contiguous(),
                self._acct)

    @state.setter
    def state(self, st) -> None:
        if not st:
            return
        KIVIKVCache.state.fset(self, st[:9])
        self._clear_sinks()
        if len(st) > 9:
            sp, sn, fp, fc, fk, fv, fd, acct = st[9:]
            B, H, u, D = fk.shape
            self._sink_pos, self._sink_norm = sp.clone(), sn.clone()
            self._ensure_sink_rows(B, H, D, u, fk.device, fk.dtype)
            self._fs_pos[:, :u], self._fs_k[:, :, :u], self._fs_v[:, :, :u], self._fs_kdead[:, :, :u] = fp, fk, fv, fd
            self._fs_count = fc.clone()
            self._acct = acct.clone()
            self._fs_upper = u

    @property
    def meta_state(self):
        return (*KIVIKVCache.meta_state.fget(self), str(self._n_sink))

    @meta_state.setter
    def meta_state(self, v) -> None:
        KIVIKVCache.meta_state.fset(self, v[:7])
        if len(v) > 7:
            self._n_sink = int(v[7])

    @classmethod
    def from_state(cls, state, meta_state=None, config=None):
        if meta_state is None:
            raise TypeError("SinkProtectedKVCache.from_state() requires meta_state")
        hd, b, g, r = (int(x) for x in meta_state[:4])
        cfg = config if config is not None else KVCacheConfig(method="kivi_sink")
        obj = cls(dataclasses.replace(cfg, method="kivi_sink", head_dim=hd, bit_width_inlier=b, kivi_group_size=g,
                                      residual_length=r, n_sink_tokens=int(meta_state[7]) if len(meta_state) > 7 else 5))
        obj.meta_state = meta_state
        obj.state = state
        return obj

    # -- accounting (sink_cache.py:220-249): sinks are split out of the compressed pool ------
    def _quantized_bytes_dev(self, n, B, H, D):
        """``_quantized_bytes`` for a device scalar ``n`` (int64)."""
        gs = self._group_size
        code = torch.div(n * D * self._b + 7, 8, rounding_mode="floor") * H * B
        k = code + torch.div(n + gs - 1, gs, rounding_mode="floor") * D * 2 * 2 * H * B
        v = code + n * ((D + gs - 1) // gs) * 2 * 2 * H * B
        return k, v

    def _account_bytes(self, B, H, S, D, n_quant_now) -> None:
        super()._account_bytes(B, H, S, D, n_quant_now)
        if n_quant_now > 0 and self._blk_sinks is not None:
            # the host side counted all n_quant_now rows as compressed: move the block's sinks
            # (the largest count over the batch, as the reference does) to the sink pool
            s = self._blk_sinks
            k0, v0 = self._quantized_bytes_dev(torch.full_like(s, n_quant_now), B, H, D)
            k1, v1 = self._quantized_bytes_dev(n_quant_now - s, B, H, D)
            self._acct += torch.stack([k1 - k0, v1 - v0, s * D * 2 * 2 * H * B])
            self._blk_sinks = None

    def _acct_item(self, i: int) -> int:
        return 0 if self._acct is None else int(self._acct[i].item())

    @property
    def compressed_key_bytes(self) -> int:
        return max(0, self._key_bytes_compressed + self._acct_item(0))

    @property
    def compressed_value_bytes(self) -> int:
        return max(0, self._value_bytes_compressed + self._acct_item(1))

    @property
    def sink_fp16_bytes(self) -> int:
        """Bytes held exactly for protected tokens (keys + values)."""
        return max(0, self._acct_item(2))

    @property
    def sink_positions(self) -> list:
        """Protected absolute positions of batch element 0, highest norm first."""
        return self.sink_positions_for(0)

    def sink_positions_for(self, b: int) -> list:
        if self._sink_pos is None or b >= self._sink_pos.shape[0]:
            return []
        return [int(p) for p in self._sink_pos[b].tolist() if p >= 0]


_CACHE_CLASS_BY_METHOD["kivi_sink"] = SinkProtectedKVCache

__all__ = ["SinkProtectedKVCache"]
