"""TEST INFRASTRUCTURE ONLY -- CPU restatement (NumPy) of the reference's SKVQ path.

Follows ``veloxquant_mlx/quantizers/skvq.py`` (channel permutation :77-100, clipped group
quantization with per-group clip-factor search :103-165, dequantization :168-182, round trip
:185-209, byte helpers :212-226) and the cache policy of ``veloxquant_mlx/cache/skvq_cache.py``
(per-head permutations kept only where they help :137-175, window flush loop :199-254, byte
accounting :256-330).

Pinning: ``tests/golden/skvq.npz`` holds outputs of the reference's ``quantizers/skvq.py`` executed
unmodified with a NumPy stand-in for ``mlx.core`` (``tests/golden/make_golden.py``); this file
reproduces them bit for bit (``tests/test_oracle_golden.py``). What that cannot pin is MLX's own
order of the 1/group_size error mean and its rounding mode for ``round`` (taken as NumPy's: eight
strided partial sums and a tree; half to even). The cache model reproduces, bit for bit, what the
reference's ``SKVQKVCache`` class returns when it is executed over the same stand-in and a minimal
container for its ``mlx_lm`` base class (``tests/golden/cache_traces.npz``).

All arithmetic is float32 with every product and sum rounded separately.
"""

from __future__ import annotations

import math

import numpy as np

DEFAULT_ALPHA_GRID = (1.0, 0.97, 0.94, 0.90, 0.85)
_EPS = 1e-8
f32 = np.float32


def channel_permutation(x: np.ndarray) -> np.ndarray:
    """``[N, D]`` rows -> ``[D]`` int32: channels by ascending dynamic range, stable (skvq.py:77-91)."""
    x32 = np.asarray(x).astype(f32)
    rng = x32.max(axis=0) - x32.min(axis=0)
    return np.argsort(rng, kind="stable").astype(np.int32)


def invert_permutation(perm: np.ndarray) -> np.ndarray:
    return np.argsort(np.asarray(perm), kind="stable").astype(np.int32)


def apply_permutation(x: np.ndarray, perm: np.ndarray) -> np.ndarray:
    return np.take(x, perm, axis=-1)


def _group_error_sum(sq: np.ndarray) -> np.ndarray:
    """Sum over the last axis (length a multiple of 8, at most 128) in a fixed order: eight partial
    sums over the elements 8 apart, first to last, then ((r0+r1)+(r2+r3))+((r4+r5)+(r6+r7))."""
    gs = sq.shape[-1]
    if gs % 8 or gs > 128:
        raise ValueError("group_size must be a multiple of 8, at most 128, for the defined summation order")
    r = sq[..., 0:8].astype(f32).copy()
    for i in range(8, gs, 8):
        r = (r + sq[..., i:i + 8]).astype(f32)
    a = (r[..., 0::2] + r[..., 1::2]).astype(f32)      # r0+r1, r2+r3, r4+r5, r6+r7
    b = (a[..., 0::2] + a[..., 1::2]).astype(f32)
    return (b[..., 0] + b[..., 1]).astype(f32)


def clipped_group_quant(x: np.ndarray, bits: int, group_size: int, alphas=DEFAULT_ALPHA_GRID):
    """``[N, D]`` -> ``(codes u8 [N, D], lo f32 [N, G], scale f32 [N, G])`` (skvq.py:103-165).
    ``D`` must be a multiple of ``group_size`` here (the reference pads a ragged last group)."""
    n, d = x.shape
    gs = int(group_size)
    if d % gs:
        raise ValueError("D must be a multiple of group_size")
    G = d // gs
    xg = np.asarray(x).astype(f32).reshape(n, G, gs)
    gmin = xg.min(axis=-1, keepdims=True)
    gmax = xg.max(axis=-1, keepdims=True)
    mid = ((gmax + gmin).astype(f32) * f32(0.5)).astype(f32)
    rng = (gmax - gmin).astype(f32)
    levels = f32((1 << int(bits)) - 1)
    best_err = None
    for a in alphas:
        a = f32(a)
        ar = (a * rng).astype(f32)
        lo = (mid - (ar * f32(0.5)).astype(f32)).astype(f32)
        scale = np.maximum((ar / levels).astype(f32), f32(_EPS))
        codes = np.clip(np.round(((xg - lo).astype(f32) / scale).astype(f32)), 0, levels).astype(f32)
        recon = ((codes * scale).astype(f32) + lo).astype(f32)
        e = (recon - xg).astype(f32)
        err = _group_error_sum((e * e).astype(f32))      # the mean's 1/gs scaling does not change the argmin
        if best_err is None:
            best_err, best = err, (codes, lo, scale)
        else:
            take = err < best_err                        # first minimum wins
            best_err = np.where(take, err, best_err)
            best = tuple(np.where(take[..., None], new, old) for new, old in zip((codes, lo, scale), best))
    codes, lo, scale = best
    return codes.reshape(n, d).astype(np.uint8), lo[..., 0].astype(f32), scale[..., 0].astype(f32)


def clipped_group_dequant(codes: np.ndarray, lo: np.ndarray, scale: np.ndarray, group_size: int, d: int) -> np.ndarray:
    n = codes.shape[0]
    G = lo.shape[1]
    cg = codes.reshape(n, G, int(group_size)).astype(f32)
    recon = ((cg * scale[:, :, None]).astype(f32) + lo[:, :, None]).astype(f32)
    return recon.reshape(n, G * int(group_size))[:, :d]


def skvq_round_trip(x: np.ndarray, perm, bits: int, group_size: int, alphas=DEFAULT_ALPHA_GRID) -> np.ndarray:
    n, d = x.shape
    xp = apply_permutation(x, perm) if perm is not None else x
    codes, lo, scale = clipped_group_quant(xp, bits, group_size, alphas)
    recon = clipped_group_dequant(codes, lo, scale, group_size, d)
    if perm is not None:
        recon = apply_permutation(recon, invert_permutation(perm))
    return recon.astype(x.dtype)


def skvq_compressed_bytes(n_tokens: int, d: int, bits: int, group_size: int) -> int:
    n_groups = (d + group_size - 1) // group_size
    return math.ceil(n_tokens * d * bits / 8) + n_tokens * n_groups * 2 * 2


def skvq_fp16_bytes(n_tokens: int, d: int) -> int:
    return n_tokens * d * 2


# ---- cache policy (skvq_cache.py) ------------------------------------------------------------
def _round_trip_4d(x, perm, inv, bits, gs, alphas):
    """``[B,H,r,D]`` through per-head gather -> quantize -> dequantize -> inverse gather (skvq_cache.py:184-197)."""
    B, H, r, D = x.shape
    x32 = x.astype(f32)
    if perm is not None:
        x32 = np.take_along_axis(x32, np.broadcast_to(perm[None, :, None, :], x32.shape), axis=-1)
    codes, lo, scale = clipped_group_quant(x32.reshape(B * H * r, D), bits, gs, alphas)
    recon = clipped_group_dequant(codes, lo, scale, gs, D).reshape(B, H, r, D)
    if inv is not None:
        recon = np.take_along_axis(recon, np.broadcast_to(inv[None, :, None, :], recon.shape), axis=-1)
    return recon.astype(x.dtype)


def per_head_perms(chunk: np.ndarray, bits: int, n_sink: int, gs: int, alphas):
    """Candidate = channels of a head sorted by dynamic range over the chunk's non-sink rows; kept
    only where its round-trip error is strictly lower than the identity order's (skvq_cache.py:137-175).
    The per-head error is a float64 mean of the float32 squared errors."""
    B, H, r, D = chunk.shape
    x = chunk[:, :, n_sink:, :].astype(f32)
    xh = x.transpose(1, 0, 2, 3).reshape(H, -1, D)
    rng = xh.max(axis=1) - xh.min(axis=1)
    cand = np.argsort(rng, axis=-1, kind="stable").astype(np.int32)
    cand_inv = np.argsort(cand, axis=-1, kind="stable").astype(np.int32)

    def err(p, i):
        d = (_round_trip_4d(x, p, i, bits, gs, alphas) - x).astype(f32)
        return (d * d).astype(f32).astype(np.float64).mean(axis=(0, 2, 3))

    keep = (err(cand, cand_inv) < err(None, None))[:, None]
    identity = np.broadcast_to(np.arange(D, dtype=np.int32)[None, :], (H, D))
    return np.where(keep, cand, identity).astype(np.int32), np.where(keep, cand_inv, identity).astype(np.int32)


class SKVQCacheModel:
    """Dense model of the reference's cache: what ``update_and_fetch`` returns after every call."""

    def __init__(self, head_dim, bits_k=4, bits_v=4, group_size=32, window=128, n_sink=5, reorder=True,
                 clip_search=True, clip_alpha=1.0):
        self.D, self.bk, self.bv, self.gs, self.window, self.n_sink = head_dim, bits_k, bits_v, group_size, window, n_sink
        self.reorder = reorder
        self.alphas = DEFAULT_ALPHA_GRID if clip_search else (clip_alpha,)
        self.keys = self.values = None
        self.q_end = 0
        self.perm_k = self.inv_k = self.perm_v = self.inv_v = None
        self.compressed_key_bytes = self.compressed_value_bytes = 0

    @property
    def offset(self):
        return 0 if self.keys is None else self.keys.shape[2]

    def update_and_fetch(self, k, v):
        self.keys = k.copy() if self.keys is None else np.concatenate([self.keys, k], axis=2)
        self.values = v.copy() if self.values is None else np.concatenate([self.values, v], axis=2)
        B, H, _, D = self.keys.shape
        r = self.window
        while self.offset - self.q_end >= r:
            s, e = self.q_end, self.q_end + r
            kc, vc = self.keys[:, :, s:e].copy(), self.values[:, :, s:e].copy()
            if s == 0 and self.reorder:
                self.perm_k, self.inv_k = per_head_perms(kc, self.bk, self.n_sink, self.gs, self.alphas)
                self.perm_v, self.inv_v = per_head_perms(vc, self.bv, self.n_sink, self.gs, self.alphas)
            kq = _round_trip_4d(kc, self.perm_k, self.inv_k, self.bk, self.gs, self.alphas)
            vq = _round_trip_4d(vc, self.perm_v, self.inv_v, self.bv, self.gs, self.alphas)
            if s == 0 and self.n_sink > 0:
                kq[:, :, :self.n_sink] = kc[:, :, :self.n_sink]
                vq[:, :, :self.n_sink] = vc[:, :, :self.n_sink]
            self.keys[:, :, s:e], self.values[:, :, s:e] = kq, vq
            n_q = r - (self.n_sink if s == 0 else 0)
            self.compressed_key_bytes += skvq_compressed_bytes(n_q, D, self.bk, self.gs) * B * H
            self.compressed_value_bytes += skvq_compressed_bytes(n_q, D, self.bv, self.gs) * B * H
            self.q_end = e
        return self.keys, self.values
