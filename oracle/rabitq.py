"""Oracle: RaBitQ 1-bit key encode and popcount decode attention (test infrastructure only).

Follows:

* ``veloxquant_mlx/tests/metal/test_rabitq_encode.py:36-58`` (``_wht_butterfly``,
  ``_reference_encode``: the canonical Sylvester butterfly order)
* ``veloxquant_mlx/quantizers/rabitq.py:64-70`` (``_pack_signs``: ``>= 0`` is
  bit 1, ``np.packbits(bitorder="little")``)
* ``veloxquant_mlx/quantizers/rabitq.py:197-206`` (rotation: randomized
  Hadamard for power-of-two D, ``x*diag @ R.T`` otherwise)
* ``veloxquant_mlx/math/rotation.py:56-100`` (seeded diagonal / QR rotation)
* ``veloxquant_mlx/tests/metal/test_rabitq_attend.py:32-58`` (``_reference_attend``)
* ``veloxquant_mlx/metal/src/rabitq_hamming_score.metal`` (``ham*scale + Cx``)
"""

from __future__ import annotations

import numpy as np


def wht_butterfly(x: np.ndarray) -> np.ndarray:
    """Unscaled Sylvester-order Walsh-Hadamard transform along the last axis (fp32)."""
    y = np.array(x, dtype=np.float32, copy=True)
    d = y.shape[-1]
    if d & (d - 1):
        raise ValueError(f"wht_butterfly: D={d} must be a power of 2")
    stride = 1
    while stride < d:
        yv = y.reshape(y.shape[:-1] + (d // (2 * stride), 2, stride))
        a = yv[..., 0, :].copy()
        b = yv[..., 1, :].copy()
        yv[..., 0, :] = a + b
        yv[..., 1, :] = a - b
        stride <<= 1
    return y


def make_hadamard_diagonal(d: int, seed: int = 42) -> np.ndarray:
    rng = np.random.default_rng(seed)
    return rng.choice(np.array([-1.0, 1.0], dtype=np.float32), size=d)


def make_rotation_matrix(d: int, seed: int = 42) -> np.ndarray:
    rng = np.random.default_rng(seed)
    G = rng.standard_normal((d, d)).astype(np.float64)
    Q, _ = np.linalg.qr(G)
    return Q.astype(np.float64)


def pack_signs(y: np.ndarray) -> np.ndarray:
    """``[N, D] -> [N, D//8]`` uint8, element ``8*j+t`` at byte ``j`` bit ``t``."""
    signs = (y >= 0).astype(np.uint8)
    D = signs.shape[-1]
    packed = np.packbits(signs, axis=-1, bitorder="little")
    return packed[..., : D // 8]


def encode_hadamard(keys: np.ndarray, diag: np.ndarray):
    """``y = WHT(keys*diag)/sqrt(D)``; returns ``(bits u8 [N,D/8], mag f32 [N], y)``.

    ``mag = sum|y| / D`` (L1 magnitude per element).
    """
    keys = np.asarray(keys)
    D = keys.shape[-1]
    y = wht_butterfly(keys.astype(np.float32) * np.asarray(diag, dtype=np.float32)[None, :])
    y = y / np.sqrt(np.float32(D))
    bits = pack_signs(y)
    mag = (np.abs(y).sum(axis=1) / D).astype(np.float32)
    return bits, mag, y


def encode_rotation(keys: np.ndarray, rot: np.ndarray):
    """Dense-rotation variant (non power-of-two D, or a QR rotation by choice):
    ``y = keys @ rot.T`` in float32."""
    keys = np.asarray(keys)
    D = keys.shape[-1]
    y = keys.astype(np.float32) @ np.asarray(rot, dtype=np.float32).T
    bits = pack_signs(y)
    mag = (np.abs(y).sum(axis=1) / D).astype(np.float32)
    return bits, mag, y.astype(np.float32)


def hamming_score(q_bits: np.ndarray, bits: np.ndarray, scale: float, cx: np.ndarray) -> np.ndarray:
    """``score[i] = popcount(q ^ bits[i]) * scale + cx[i]`` (fp32)."""
    x = np.bitwise_xor(np.asarray(bits, np.uint8), np.asarray(q_bits, np.uint8)[None, :])
    ham = np.unpackbits(x, axis=1).sum(axis=1).astype(np.float32)
    return (ham * np.float32(scale) + np.asarray(cx, np.float32)).astype(np.float32)


def reference_attend(q, q_scale, k_bits, k_mag, k_const, v, v_cents=None) -> np.ndarray:
    """Popcount-scored attention.

    ``q [B,H_q,S_q,D]``; ``k_bits [B,H_kv,S,D/8]``; ``k_mag,k_const [B,H_kv,S]``;
    ``v`` is ``u8 [B,H_kv,S,D]`` indices into ``v_cents`` (reference form), or a
    dense float ``[B,H_kv,S,D]`` tensor when ``v_cents is None``. ``H_q`` may be
    a multiple of ``H_kv`` (contiguous GQA blocks). No attention scale is
    applied here: the caller folds it into ``q_scale``/``k_const``.
    """
    q = np.asarray(q)
    B, H_q, S_q, D = q.shape
    H_kv = k_bits.shape[1]
    rep = H_q // H_kv
    q_bits = q >= 0
    k_unp = np.unpackbits(np.asarray(k_bits, np.uint8), axis=-1, count=D, bitorder="little").astype(bool)
    k_mag = np.asarray(k_mag, np.float32)
    k_const = np.asarray(k_const, np.float32)
    if v_cents is not None:
        v_hat = np.asarray(v_cents, np.float32)[np.asarray(v)]
    else:
        v_hat = np.asarray(v).astype(np.float32)
    if rep > 1:
        k_unp = np.repeat(k_unp, rep, axis=1)
        k_mag = np.repeat(k_mag, rep, axis=1)
        k_const = np.repeat(k_const, rep, axis=1)
        v_hat = np.repeat(v_hat, rep, axis=1)
    out = np.empty((B, H_q, S_q, D), dtype=np.float32)
    for b in range(B):
        for h in range(H_q):
            ham = (q_bits[b, h][:, None, :] ^ k_unp[b, h][None, :, :]).sum(axis=-1).astype(np.float32)
            scores = (np.float32(D) - np.float32(2.0) * ham) * np.asarray(q_scale, np.float32)[b, h][:, None] \
                * k_mag[b, h][None, :] + k_const[b, h][None, :]
            scores = scores - scores.max(axis=-1, keepdims=True)
            w = np.exp(scores)
            w = w / w.sum(axis=-1, keepdims=True)
            out[b, h] = w @ v_hat[b, h]
    return out


def reference_prefill(q, scale, k_bits, k_mag, k_const, v, v_cents=None, causal: bool = False) -> np.ndarray:
    """Exact-dot attention of many query rows over sign-bit keys: a restatement of
    ``_reference_prefill`` (``tests/metal/test_rabitq_prefill.py:32-53``) with contiguous-block GQA
    and dense values added.

    ``k_hat = signs(k_bits) * k_mag``; ``score = (q . k_hat) * scale + k_const``; with ``causal``
    query row ``r`` of ``S_q`` sits at slot ``S_kv - S_q + r`` and slots after it are masked.
    ``v`` holds indices into ``v_cents`` (``u8 [B,H_kv,S,D]``, unpacked) or, with
    ``v_cents is None``, dense values.
    """
    q = np.asarray(q)
    D = q.shape[-1]
    S_q, S_kv = q.shape[2], k_bits.shape[2]
    signs = np.unpackbits(np.asarray(k_bits, np.uint8), axis=-1, count=D, bitorder="little").astype(np.float32) * 2.0 - 1.0
    k_hat = signs * np.asarray(k_mag, np.float32)[..., None]
    kc = np.zeros(k_hat.shape[:3], np.float32) if k_const is None else np.asarray(k_const, np.float32)
    v_hat = np.asarray(v_cents, np.float32)[np.asarray(v)] if v_cents is not None else np.asarray(v).astype(np.float32)
    rep = q.shape[1] // k_hat.shape[1]
    if rep > 1:
        k_hat, kc, v_hat = (np.repeat(t, rep, axis=1) for t in (k_hat, kc, v_hat))
    scores = np.einsum("bhqd,bhsd->bhqs", q.astype(np.float32), k_hat) * np.float32(scale) + kc[:, :, None, :]
    if causal:
        q_abs = (S_kv - S_q) + np.arange(S_q)
        scores = np.where(np.arange(S_kv)[None, :] > q_abs[:, None], -np.inf, scores)
    scores = scores - scores.max(axis=-1, keepdims=True)
    w = np.exp(scores)
    w = w / w.sum(axis=-1, keepdims=True)
    return np.einsum("bhqs,bhsd->bhqd", w, v_hat).astype(np.float32)
