"""Oracle: TurboQuant-RVQ quantize+pack and unpack+decode (test infrastructure only).

Restates, operation by operation:

* ``veloxquant_mlx/metal/src/rvq_quant_pack.metal`` (= ``ScalarCodebook.quantize``,
  ``codebooks/scalar_codebook.py:77-95``, for both stages with the residual rounded to fp16,
  ``quantizers/turboquant_rvq.py:176-180``, then ``_pack_indices``,
  ``cache/turboquant_rvq_cache.py:82-106``): integer results, bit-exact by construction.
* ``veloxquant_mlx/metal/src/rvq_unpack_decode.metal``: ``half(c1 + c2)``, float32 butterfly with
  strides 1, 2, 4, ... (lower = self + partner, upper = partner - self), ``/ sqrt(D)``,
  ``half(h * diag)``, ``half(clamp(x * norm, +-65504))``.

Pinned by ``tests/golden/rvq.npz`` (Lloyd-Max codebooks produced by executing the reference's
``math/lloyd_max.py`` and ``math/distributions.py``; the cache's packing and norm helpers) and by
``tests/golden/rvq_reference.npz``: the reference's ``TurboQuantRVQ.encode`` / ``decode``
(``quantizers/turboquant_rvq.py:163-194``) and its cache class (``cache/turboquant_rvq_cache.py``)
executed unmodified over a NumPy stand-in for ``mlx.core`` (``tests/golden/make_golden.py``). Given
the rotated input, both index streams, the packed words, the decoded vectors and everything the
cache class returns over a call script are reproduced bit for bit (``tests/test_oracle_golden.py``).
What that cannot pin is MLX's own ``hadamard_transform`` (order of its float32 sums; the stand-in
uses the butterfly of this file) and the Metal kernel's ``rsqrt`` (a correctly rounded
``1/sqrt(D)`` here).
"""

from __future__ import annotations

import numpy as np


def quantize_boundaries(y32: np.ndarray, boundaries) -> np.ndarray:
    """``#{k : y > b_k}`` for sorted boundaries (float comparisons of fp16-representable values)."""
    b = np.asarray(boundaries, dtype=np.float32)
    return (y32[..., None] > b).sum(-1).astype(np.uint8)


def pack_indices(idx: np.ndarray, bits: int) -> np.ndarray:
    epw = 32 // bits
    d = idx.shape[-1]
    pad = (-d) % epw
    x = idx.astype(np.uint64)
    if pad:
        x = np.concatenate([x, np.zeros(idx.shape[:-1] + (pad,), np.uint64)], axis=-1)
    x = x.reshape(idx.shape[:-1] + (-1, epw))
    shifts = (np.arange(epw, dtype=np.uint64) * np.uint64(bits))
    return (x << shifts).sum(-1).astype(np.uint32)


def unpack_indices(packed: np.ndarray, bits: int, d: int) -> np.ndarray:
    epw = 32 // bits
    shifts = np.arange(epw, dtype=np.uint32) * np.uint32(bits)
    codes = (packed[..., None] >> shifts) & np.uint32((1 << bits) - 1)
    return codes.reshape(packed.shape[:-1] + (-1,))[..., :d].astype(np.uint8)


def rvq_quant_pack(rotated16: np.ndarray, centroids1, boundaries1, boundaries2, bits: int):
    """``rotated16 [N, D]`` float16 -> ``(idx1, idx2, packed1, packed2)``."""
    y = rotated16.astype(np.float32)
    c1 = np.asarray(centroids1, dtype=np.float16).astype(np.float32)
    idx1 = quantize_boundaries(y, np.asarray(boundaries1, dtype=np.float16))
    r1 = (y - c1[idx1]).astype(np.float16).astype(np.float32)
    idx2 = quantize_boundaries(r1, np.asarray(boundaries2, dtype=np.float16))
    return idx1, idx2, pack_indices(idx1, bits), pack_indices(idx2, bits)


def wht_butterfly(v: np.ndarray) -> np.ndarray:
    """Unnormalised Walsh-Hadamard transform along the last axis in float32, strides ascending."""
    v = v.astype(np.float32).copy()
    D = v.shape[-1]
    s = 1
    while s < D:
        x = v.reshape(v.shape[:-1] + (D // (2 * s), 2, s))
        lo, hi = x[..., 0, :].copy(), x[..., 1, :].copy()
        x[..., 0, :] = lo + hi
        x[..., 1, :] = lo - hi
        v = x.reshape(v.shape)
        s *= 2
    return v


def rvq_unpack_decode(packed1, packed2, norms, centroids1, centroids2, diag, bits: int, d: int) -> np.ndarray:
    """``[N, n_words]`` streams + ``norms [N]`` -> float16 ``[N, d]``."""
    c1 = np.asarray(centroids1, dtype=np.float16)
    c2 = np.asarray(centroids2, dtype=np.float16)
    i1, i2 = unpack_indices(packed1, bits, d), unpack_indices(packed2, bits, d)
    y = (c1[i1].astype(np.float32) + c2[i2].astype(np.float32)).astype(np.float16)
    h = wht_butterfly(y.astype(np.float32)) * (np.float32(1.0) / np.sqrt(np.float32(d)))
    x_unit = (h * np.asarray(diag, dtype=np.float32)).astype(np.float16).astype(np.float32)
    k = x_unit * np.asarray(norms, dtype=np.float32).reshape(-1, 1)
    return np.clip(k, -65504.0, 65504.0).astype(np.float16)


# ---- cache pipeline (cache/turboquant_rvq_cache.py) -------------------------------------------
def unit_and_norm(k16: np.ndarray):
    """``[N, D]`` float16 -> ``(unit float16 [N, D], norm float32 [N, 1])``: float32 norm, floor 1e-4
    (turboquant_rvq_cache.py:66-72)."""
    k32 = k16.astype(np.float32)
    norms = np.sqrt(np.sum(k32 * k32, axis=-1, keepdims=True))
    return (k32 / np.maximum(norms, np.float32(1e-4))).astype(np.float16), norms


def rotate(unit16: np.ndarray, diag) -> np.ndarray:
    """Randomized Hadamard rotation ``H (diag * x) / sqrt(D)`` in float32, result in float16
    (preconditioners/rotation.py, ``HadamardPreconditioner.apply``)."""
    d = unit16.shape[-1]
    h = wht_butterfly(unit16.astype(np.float32) * np.asarray(diag, dtype=np.float32))
    return (h * (np.float32(1.0) / np.sqrt(np.float32(d)))).astype(np.float16)


def round_to_bfloat16(x: np.ndarray) -> np.ndarray:
    """float32 -> nearest bfloat16 (ties to even), returned as float32."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
    u = (u + ((u >> np.uint64(16)) & np.uint64(1)) + np.uint64(0x7FFF)) & np.uint64(0xFFFF0000)
    return u.astype(np.uint32).view(np.float32).reshape(np.shape(x))


class RVQCacheModel:
    """What the reference's ``TurboQuantRVQKVCache`` holds and returns (float16 keys): packed
    streams and bfloat16 norms in buffers that grow in steps of 256 rows, every live key decoded on
    each call (turboquant_rvq_cache.py:236-324), ``trim`` scaling the byte counters (:429-438)."""

    STEP = 256

    def __init__(self, head_dim, bits, diag, centroids1, boundaries1, centroids2, boundaries2):
        self.D, self.bits, self.diag = int(head_dim), int(bits), np.asarray(diag, dtype=np.float32)
        self.c1, self.b1, self.c2, self.b2 = centroids1, boundaries1, centroids2, boundaries2
        self.n_words = -(-self.D // (32 // self.bits))
        self.p1 = self.p2 = self.norms = self.values = None
        self.offset = 0
        self.compressed_key_bytes = self.fp16_key_bytes = 0

    def _grow(self, buf, prev, S, shape_tail, dtype, B, H):
        if buf is not None and prev + S <= buf.shape[2]:
            return buf
        rows = -(-(self.STEP + S - 1) // self.STEP) * self.STEP
        new = np.zeros((B, H, rows) + shape_tail, dtype)
        if buf is None:
            return new
        if prev % self.STEP:
            buf = buf[:, :, :prev]
        return np.concatenate([buf, new], axis=2)

    def update_and_fetch(self, keys, values):
        B, H, S, D = keys.shape
        prev = self.offset
        unit, norms = unit_and_norm(keys.reshape(-1, D))
        _, _, w1, w2 = rvq_quant_pack(rotate(unit, self.diag), self.c1, self.b1, self.b2, self.bits)
        self.p1 = self._grow(self.p1, prev, S, (self.n_words,), np.uint32, B, H)
        self.p2 = self._grow(self.p2, prev, S, (self.n_words,), np.uint32, B, H)
        self.norms = self._grow(self.norms, prev, S, (1,), np.float32, B, H)
        self.values = self._grow(self.values, prev, S, (values.shape[3],), values.dtype, B, H)
        self.offset = prev + S
        self.p1[:, :, prev:self.offset] = w1.reshape(B, H, S, self.n_words)
        self.p2[:, :, prev:self.offset] = w2.reshape(B, H, S, self.n_words)
        self.norms[:, :, prev:self.offset] = round_to_bfloat16(norms).reshape(B, H, S, 1)
        self.values[:, :, prev:self.offset] = values
        self.compressed_key_bytes += (2 * self.n_words * 4 + 2) * H * B * S
        self.fp16_key_bytes += H * B * S * D * 2
        n = self.offset
        k_hat = rvq_unpack_decode(self.p1[:, :, :n].reshape(-1, self.n_words), self.p2[:, :, :n].reshape(-1, self.n_words),
                                  self.norms[:, :, :n].reshape(-1), self.c1, self.c2, self.diag, self.bits, D)
        return k_hat.reshape(B, H, n, D), self.values[:, :, :n]

    def trim(self, n):
        old = self.offset
        n = min(old, n)
        self.offset -= n
        if n and old:
            keep = self.offset / old
            self.compressed_key_bytes = int(self.compressed_key_bytes * keep)
            self.fp16_key_bytes = int(self.fp16_key_bytes * keep)
        return n

    @property
    def nbytes(self):
        n = self.offset
        if n == 0 or self.p1 is None:
            return 0
        B, H = self.p1.shape[:2]
        return B * H * n * (2 * self.n_words * 4 + 2 + self.values.shape[3] * self.values.dtype.itemsize)
