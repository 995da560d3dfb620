"""Oracle: TurboQuant-RVQ quantize+pack and unpack+decode (test infrastructure only).

Restates, operation by operation:

* ``veloxquant_mlx/metal/src/rvq_quant_pack.metal`` (= ``ScalarCodebook.quantize``,
  ``codebooks/scalar_codebook.py:77-95``, for both stages with the residual rounded to fp16,
  ``quantizers/turboquant_rvq.py:176-180``, then ``_pack_indices``,
  ``cache/turboquant_rvq_cache.py:82-106``): integer results, bit-exact by construction.
* ``veloxquant_mlx/metal/src/rvq_unpack_decode.metal``: ``half(c1 + c2)``, float32 butterfly with
  strides 1, 2, 4, ... (lower = self + partner, upper = partner - self), ``/ sqrt(D)``,
  ``half(h * diag)``, ``half(clamp(x * norm, +-65504))``.

Pinned by ``tests/golden/rvq.npz``: Lloyd-Max codebooks produced by executing the reference's
``math/lloyd_max.py`` and ``math/distributions.py``. The kernels' outputs themselves have no
reference-held vectors (the reference's tests compare two MLX paths with each other), so the
arithmetic of this file is **parity unpinned** beyond the codebooks; the quantize side is pure
comparisons against fp16 tables and leaves no freedom, the decode side differs from the Metal
kernel at most by its ``rsqrt`` (a correctly rounded ``1/sqrt(D)`` here).
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
