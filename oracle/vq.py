"""Oracle: VecInfer product VQ and LUT decode attention (test infrastructure only).

Follows:

* ``veloxquant_mlx/allocators/vecinfer.py:281-318`` (``quantize_vq``) with the
  summation order of ``veloxquant_mlx/metal/src/vecinfer_quantize.metal:18-27``
* ``veloxquant_mlx/allocators/vecinfer.py:321-335`` (``dequantize_vq``)
* ``veloxquant_mlx/allocators/vecinfer.py:341-359`` (``compute_query_lut``)
* ``veloxquant_mlx/allocators/vecinfer.py:60-87`` (``walsh_hadamard_matrix``)
* ``veloxquant_mlx/allocators/vecinfer.py:93-184`` (dual transform)
* ``veloxquant_mlx/tests/cache/test_vecinfer_fused_sdpa.py:69-115`` (``_reference_sdpa``)

``quantize_vq``: the reference computes ``mx.sum(diff*diff, -1)`` / ``mx.argmin`` inside MLX, which
cannot be installed here, and its tests only check statistical agreement. The canonical order fixed
here: float32; ``d = x_i - c_i``; ``dist = dist + d*d`` with the product and the sum rounded
separately, for ``i = 0..sub_dim-1`` in order, starting from ``0.0``; the first (lowest-index)
minimum wins. Pinning: ``tests/golden/vq.npz`` holds the indices of the reference's own function
executed with NumPy answering ``mx`` (``tests/golden/make_golden.py``); NumPy sums a row of fewer than
8 float32 in exactly this order, so at sub-vector sizes 2 and 4 the pin is bit for bit by
construction; at size 8 NumPy adds as a tree and the recorded indices still all agree (a difference
could only be a near-tie). What stays open is MLX's own reduction order. ``reference_sdpa`` (with the
dual transform of the queries) equals the reference's ``_reference_sdpa``, executed the same way, to
2e-6 on causal / windowed / grouped-head / smoothed cases (same file). The fused encode / decode
kernels' arithmetic remains unpinned.
"""

from __future__ import annotations

import math

import numpy as np


def quantize_vq(x: np.ndarray, codebook: np.ndarray, sub_dim: int,
                chunk: int = 1 << 16) -> np.ndarray:
    """Nearest-centroid indices ``int32 [..., D//sub_dim]``.

    ``codebook`` is ``[n_c, sub_dim]`` shared by all sub-spaces (reference
    form) or ``[n_sub, n_c, sub_dim]`` (one codebook per sub-space).
    """
    x = np.asarray(x)
    *lead, D = x.shape
    if D % sub_dim:
        raise ValueError(f"quantize_vq: D={D} not divisible by sub_dim={sub_dim}")
    n_sub = D // sub_dim
    cb = np.asarray(codebook).astype(np.float32)
    flat = x.reshape(-1, n_sub, sub_dim).astype(np.float32)
    N = flat.shape[0]
    out = np.empty((N, n_sub), dtype=np.int32)
    for j in range(n_sub):
        cbj = cb if cb.ndim == 2 else cb[j]
        n_c = cbj.shape[0]
        for s in range(0, N, chunk):
            sub = flat[s:s + chunk, j, :]
            dist = np.zeros((sub.shape[0], n_c), dtype=np.float32)
            with np.errstate(invalid="ignore", over="ignore"):
                for i in range(sub_dim):
                    d = sub[:, i:i + 1] - cbj[None, :, i]
                    dist = dist + d * d
            # the kernel's scan is "if (dist < best)" from best = +inf: a NaN distance never
            # wins, and if nothing is finite the index stays 0 (vecinfer_quantize.metal:16-27)
            dist = np.where(np.isnan(dist), np.float32(np.inf), dist)
            out[s:s + chunk, j] = np.argmin(dist, axis=1).astype(np.int32)
    return out.reshape(*lead, n_sub)


def dequantize_vq(indices: np.ndarray, codebook: np.ndarray) -> np.ndarray:
    """Gather centroids: ``[..., n_sub] -> [..., n_sub*sub_dim]``.

    Out-of-range indices clamp to ``n_c-1`` as in ``vecinfer_dequant.metal``.
    """
    cb = np.asarray(codebook)
    idx = np.asarray(indices).astype(np.int64)
    *lead, n_sub = idx.shape
    if cb.ndim == 2:
        n_c, sub_dim = cb.shape
        g = cb[np.clip(idx, 0, n_c - 1)]
    else:
        _, n_c, sub_dim = cb.shape
        g = cb[np.arange(n_sub), np.clip(idx, 0, n_c - 1)]
    return g.reshape(*lead, n_sub * sub_dim)


def compute_query_lut(q_tilde: np.ndarray, codebook: np.ndarray, sub_dim: int) -> np.ndarray:
    """``lut[..., s, c] = q_sub[..., s, :] . codebook[c, :]``."""
    *lead, D = q_tilde.shape
    if D % sub_dim != 0:
        raise ValueError(f"compute_query_lut: D={D} not divisible by sub_dim={sub_dim}")
    n_sub = D // sub_dim
    q_sub = q_tilde.reshape(*lead, n_sub, sub_dim).astype(np.float32)
    cb = np.asarray(codebook).astype(np.float32)
    if cb.ndim == 2:
        return q_sub @ cb.T
    return np.einsum("...sd,scd->...sc", q_sub, cb)


def walsh_hadamard_matrix(d: int) -> np.ndarray:
    """Orthonormal Sylvester Walsh-Hadamard matrix, float32."""
    if d < 1 or (d & (d - 1)) != 0:
        raise ValueError(f"walsh_hadamard_matrix: d={d} must be a power of 2.")
    H = np.array([[1.0]], dtype=np.float32)
    inv_sqrt2 = 1.0 / math.sqrt(2.0)
    size = 1
    while size < d:
        top = np.concatenate([H, H], axis=1)
        bot = np.concatenate([H, -H], axis=1)
        H = np.concatenate([top, bot], axis=0) * inv_sqrt2
        size *= 2
    return H.astype(np.float32)


def _smooth_for(x: np.ndarray, smooth: np.ndarray, for_query: bool) -> np.ndarray:
    smooth = np.asarray(smooth)
    if smooth.ndim == 1:
        return smooth.astype(x.dtype)
    if smooth.ndim != 2:
        raise ValueError(f"smooth must be 1D or 2D, got {smooth.shape}")
    if x.ndim >= 3 and x.shape[-3] == smooth.shape[0]:
        return smooth[:, None, :].astype(x.dtype)
    if for_query and x.ndim >= 3 and smooth.shape[0] > 0 and x.shape[-3] % smooth.shape[0] == 0:
        rep = x.shape[-3] // smooth.shape[0]
        return np.repeat(smooth, rep, axis=0)[:, None, :].astype(x.dtype)
    if x.shape[-1] == smooth.shape[-1]:
        return smooth.mean(axis=0).astype(x.dtype)
    raise ValueError(f"cannot broadcast smooth {smooth.shape} to {x.shape}")


def apply_dual_transform_keys(K, smooth, H):
    """``(K / lambda) @ H``."""
    K = np.asarray(K)
    return (K / _smooth_for(K, smooth, False)) @ np.asarray(H).astype(K.dtype)


def apply_dual_transform_queries(q, smooth, H):
    """``(q * lambda) @ H``."""
    q = np.asarray(q)
    return (q * _smooth_for(q, smooth, True)) @ np.asarray(H).astype(q.dtype)


def _wht_fixed_order(x: np.ndarray, D: int) -> np.ndarray:
    """Unnormalised Sylvester butterfly over the last axis in float32 (pairs (lower + upper,
    lower - upper), strides 1, 2, 4, ...), then one multiplication by the common entry
    magnitude of ``walsh_hadamard_matrix(D)``."""
    y = np.ascontiguousarray(x, dtype=np.float32).reshape(-1, D).copy()
    h = 1
    while h < D:
        y = y.reshape(-1, D // (2 * h), 2, h)
        lo, up = y[:, :, 0, :].copy(), y[:, :, 1, :].copy()
        y[:, :, 0, :] = lo + up
        y[:, :, 1, :] = lo - up
        y = y.reshape(-1, D)
        h *= 2
    c = walsh_hadamard_matrix(D)[0, 0]
    return (y * c).astype(np.float32).reshape(x.shape)


def dual_transform_keys_wht(K, smooth=None):
    """``WHT(K / lambda)`` with the fixed summation order the native butterfly uses: the same
    mathematics as :func:`apply_dual_transform_keys` with the Walsh-Hadamard matrix, whose
    matrix-product order the reference leaves to its framework."""
    K = np.asarray(K).astype(np.float32)
    x = K if smooth is None else (K / _smooth_for(K, np.asarray(smooth, np.float32), False)).astype(np.float32)
    return _wht_fixed_order(x, K.shape[-1])


def dual_transform_queries_wht(q, smooth=None):
    """``WHT(q * lambda)``, the query side of :func:`dual_transform_keys_wht`."""
    q = np.asarray(q).astype(np.float32)
    x = q if smooth is None else (q * _smooth_for(q, np.asarray(smooth, np.float32), True)).astype(np.float32)
    return _wht_fixed_order(x, q.shape[-1])


def reference_sdpa(q_tilde, k_indices, k_codebook, v, scale, *, v_codebook=None,
                   causal=True, sliding_window=0) -> np.ndarray:
    """Dense fp32 attention over VQ keys in the transformed space.

    ``q_tilde [B,H_q,S_q,D]`` is already dual-transformed, so scores are
    ``q_tilde . dequant(k_indices)``. ``v`` is either value indices (with
    ``v_codebook``) or a dense ``[B,H_kv,S,D]`` value tensor. Masking follows
    ``_reference_sdpa``: tail-aligned causal, optional trailing window.
    """
    q32 = np.asarray(q_tilde).astype(np.float32)
    B, H_q, S_q, D = q32.shape
    k_hat = dequantize_vq(k_indices, k_codebook).astype(np.float32)
    if v_codebook is not None:
        v_hat = dequantize_vq(v, v_codebook).astype(np.float32)
    else:
        v_hat = np.asarray(v).astype(np.float32)
    H_kv, S_kv = k_hat.shape[1], k_hat.shape[2]
    rep = H_q // H_kv
    if rep > 1:
        k_hat = np.repeat(k_hat, rep, axis=1)
        v_hat = np.repeat(v_hat, rep, axis=1)
    scores = (q32 @ np.swapaxes(k_hat, -1, -2)) * np.float32(scale)
    if causal or sliding_window:
        q_pos = np.arange(S_q) + (S_kv - S_q)
        k_pos = np.arange(S_kv)
        if causal:
            scores = np.where(q_pos[:, None] < k_pos[None, :], np.float32(-1e9), scores)
        if sliding_window and sliding_window > 0:
            wm = k_pos[None, :] < (q_pos[:, None] - sliding_window + 1)
            scores = np.where(wm, np.float32(-1e9), scores)
    scores = scores - scores.max(axis=-1, keepdims=True)
    w = np.exp(scores)
    w = w / w.sum(axis=-1, keepdims=True)
    return (w @ v_hat).astype(np.float32)


def _seq_matvec(mat_rows: np.ndarray, vec: np.ndarray) -> np.ndarray:
    """``out[..., r] = sum_c mat_rows[r, c] * vec[..., c]`` accumulated for ``c = 0..D-1`` in
    order from ``0.0``, product and sum rounded separately (float32)."""
    D = vec.shape[-1]
    acc = np.zeros(vec.shape[:-1] + (mat_rows.shape[0],), dtype=np.float32)
    for c in range(D):
        acc = acc + mat_rows[:, c].astype(np.float32) * vec[..., c : c + 1].astype(np.float32)
    return acc


def encode_decode_keys(keys: np.ndarray, k_codebook: np.ndarray, sub_dim: int, H_mat: np.ndarray,
                       smooth: np.ndarray | None = None):
    """Fused key encode + decode of the reference's one-dispatch kernel
    (``veloxquant_mlx/metal/_vecinfer.py:225-293`` and
    ``veloxquant_mlx/metal/src/vecinfer_encode_decode_full.metal:8-110``):
    smooth divide (only where ``s > 1e-8``) -> ``H_mat @ x`` as a sequential matvec ->
    nearest centroid (sequential distance, first minimum) -> gather -> ``H_mat.T @ c`` ->
    smooth multiply -> float16. ``keys`` is ``[B, H, S, D]``; smooth rows are taken as
    ``h % rows`` after the wrapper's reduction (rows not in {1, H} are averaged to one row).
    Returns ``(k_hat float16 [B,H,S,D], indices int32 [B,H,S,n_sub])``. PARITY UNPINNED: whether
    the Metal compiler contracts ``dot += a*b`` into a fused multiply-add is not visible; the
    order fixed here rounds the product and the sum separately."""
    x = np.asarray(keys).astype(np.float32)
    if x.ndim != 4:
        raise ValueError(f"encode_decode_keys: keys must be 4D, got {x.shape}")
    B, Hn, S, D = x.shape
    Hm = np.asarray(H_mat).astype(np.float32)
    cb = np.asarray(k_codebook).astype(np.float32)
    sm = None
    if smooth is not None:
        sm = np.asarray(smooth).astype(np.float32)
        sm = sm.reshape(1, D) if sm.ndim == 1 else sm
        if sm.shape[0] not in (1, Hn):
            sm = sm.mean(axis=0, keepdims=True, dtype=np.float32)
        rows = sm[np.arange(Hn) % sm.shape[0]][None, :, None, :]  # [1,H,1,D]
        with np.errstate(divide="ignore", invalid="ignore"):
            x = np.where(rows > np.float32(1e-8), x / rows, x).astype(np.float32)
    y = _seq_matvec(Hm, x)
    idx = quantize_vq(y, cb, sub_dim)
    g = dequantize_vq(idx, cb).astype(np.float32)
    back = _seq_matvec(Hm.T, g)
    if sm is not None:
        back = back * rows
    return back.astype(np.float16), idx.astype(np.int32)


def encode_decode_values(values: np.ndarray, v_codebook: np.ndarray, sub_dim: int):
    """Fused value quantize + dequantize (``veloxquant_mlx/metal/_vecinfer.py:296-345``,
    ``veloxquant_mlx/metal/src/vecinfer_encode_decode_simple.metal:15-41``).
    Returns ``(v_hat float16, indices uint32)``."""
    cb = np.asarray(v_codebook).astype(np.float32)
    idx = quantize_vq(np.asarray(values).astype(np.float32), cb, sub_dim)
    return dequantize_vq(idx, cb).astype(np.float16), idx.astype(np.uint32)
