"""Oracle: KIVI asymmetric group quantization and decode attention (test infrastructure only).

Follows, line by line:

* ``veloxquant_mlx/quantizers/kivi.py:103-128`` (``KIVIQuantizer._quantize_groups``)
* ``veloxquant_mlx/tests/metal/test_scalar_attend.py:51-82`` (``_quant_keys`` /
  ``_quant_values``, the reference authors' NumPy statement of the same math)
* ``veloxquant_mlx/cache/kivi_cache.py:151-201`` (``_quant_dequant_along``)
* ``veloxquant_mlx/tests/metal/test_scalar_attend.py:85-115`` (``_reference_attend``)
* ``veloxquant_mlx/cache/kivi_cache.py:206-225`` (``_quantization_boundary``)

Pinning: ``tests/golden/kivi.npz`` (the test functions above, executed as they stand) and
``tests/golden/kivi_quantizer.npz`` (the ``KIVIQuantizer`` class executed unmodified over a NumPy
stand-in for ``mlx.core``), both reproduced bit for bit (``tests/test_oracle_golden.py``).

All arithmetic is float32 in the reference's operation order: ``min``, ``max``,
``(max-min)/levels``, ``maximum(eps)``, ``(x-min)/scale``, round-half-even,
``clip``. Reconstruction is a separately rounded multiply then add.
"""

from __future__ import annotations

import numpy as np

from . import bitpack

EPS = 1e-8


def _group_quant_last(x32: np.ndarray, g: int, levels: int, eps: float):
    """Quantize float32 ``x32`` in groups of ``g`` along its LAST axis.

    The ragged final group is padded with copies of the last live element
    (``quantizers/kivi.py:114-117``). Returns ``(codes u8 [..., L],
    scale f32 [..., G], zero f32 [..., G])``.
    """
    L = x32.shape[-1]
    G = (L + g - 1) // g
    pad = G * g - L
    x = x32
    if pad:
        tail = np.broadcast_to(x[..., -1:], x.shape[:-1] + (pad,))
        x = np.concatenate([x, tail], axis=-1)
    xg = x.reshape(x.shape[:-1] + (G, g))
    gmin = xg.min(axis=-1, keepdims=True)
    gmax = xg.max(axis=-1, keepdims=True)
    scale = np.maximum((gmax - gmin) / np.float32(levels), np.float32(eps))
    codes = np.clip(np.round((xg - gmin) / scale), 0, levels)
    codes = codes.reshape(x.shape)[..., :L].astype(np.uint8)
    return codes, scale[..., 0].astype(np.float32), gmin[..., 0].astype(np.float32)


def quant_keys(k: np.ndarray, g: int, levels: int, eps: float = EPS):
    """Per-CHANNEL group quant (groups along tokens). ``k: [B,H,S,D]``.

    Returns ``codes u8 [B,H,S,D]``, ``scale,zero f32 [B,H,ceil(S/g),D]``.
    """
    x = np.asarray(k).astype(np.float32)
    xt = np.swapaxes(x, -1, -2)  # [B,H,D,S] -> groups along last axis
    c, s, z = _group_quant_last(xt, g, levels, eps)
    return (
        np.ascontiguousarray(np.swapaxes(c, -1, -2)),
        np.ascontiguousarray(np.swapaxes(s, -1, -2)),
        np.ascontiguousarray(np.swapaxes(z, -1, -2)),
    )


def quant_values(v: np.ndarray, g: int, levels: int, eps: float = EPS):
    """Per-TOKEN group quant (groups along channels). ``v: [B,H,S,D]``.

    Returns ``codes u8 [B,H,S,D]``, ``scale,zero f32 [B,H,S,ceil(D/g)]``.
    """
    x = np.asarray(v).astype(np.float32)
    return _group_quant_last(x, g, levels, eps)


def dequant_keys(kc, ks, kz, g: int) -> np.ndarray:
    """``code*scale + zero`` with a separately rounded multiply and add (fp32)."""
    S = kc.shape[-2]
    kg = np.arange(S) // g
    prod = kc.astype(np.float32) * ks[..., kg, :]
    return (prod + kz[..., kg, :]).astype(np.float32)


def dequant_values(vc, vs, vz, g: int) -> np.ndarray:
    D = vc.shape[-1]
    vg = np.arange(D) // g
    prod = vc.astype(np.float32) * vs[..., vg]
    return (prod + vz[..., vg]).astype(np.float32)


def quant_dequant_along(x: np.ndarray, axis: int, g: int, levels: int, eps: float = EPS):
    """Round trip ``x`` through group quantization along ``axis`` (-2 keys, -1 values).

    Output keeps ``x``'s dtype (``cache/kivi_cache.py:151-201``).
    """
    if axis not in (-1, -2):
        raise ValueError("quant_dequant_along: axis must be -1 or -2")
    x = np.asarray(x)
    if axis == -2:
        c, s, z = quant_keys(x, g, levels, eps)
        rec = dequant_keys(c, s, z, g)
    else:
        c, s, z = quant_values(x, g, levels, eps)
        rec = dequant_values(c, s, z, g)
    return rec.astype(x.dtype)


def pack_codes(codes: np.ndarray, b: int) -> np.ndarray:
    """Pack codes along D, LSB first, using ``storage_bits(b)`` bits per code."""
    return bitpack.pack(codes, storage_bits(b))


def storage_bits(b: int) -> int:
    """Container width used for ``b``-bit codes in the packed store: 1, 2, 4 or 8."""
    if b < 1 or b > 8:
        raise ValueError(f"storage_bits: b={b} must be in 1..8")
    for sb in (1, 2, 4, 8):
        if b <= sb:
            return sb
    raise AssertionError


def quantization_boundary(offset: int, residual_length: int, g: int) -> int:
    """``((offset - R)//g)*g`` clamped at 0 (``cache/kivi_cache.py:206-225``)."""
    aged = max(0, offset - residual_length)
    return (aged // g) * g


def reference_attend(q, kc, ks, kz, vc, vs, vz, g: int, scale: float,
                     k_res=None, v_res=None, causal: bool = False) -> np.ndarray:
    """Dense fp32 softmax attention over dequantized K/V (+ optional fp16 tail).

    ``causal=True`` applies the tail-aligned causal mask the reference uses for attention
    over compressed caches (query row ``r`` of ``S_q`` sits at slot ``S_kv - S_q + r`` and
    sees slots up to its own: ``tests/cache/test_vecinfer_fused_sdpa.py:69-115``,
    ``metal/fused_sdpa.py:200-299``).

    ``q [B,H_q,S_q,D]``; quantized tensors carry ``H_kv`` heads; GQA uses
    contiguous blocks (``np.repeat`` along the head axis). No mask: every query
    row sees every slot, as in ``scalar_affine_attend.metal``. ``k_res/v_res``
    ``[B,H_kv,R,D]`` are the still-unquantized residual tokens that follow the
    quantized ones.
    """
    q = np.asarray(q)
    B, H, S_q, D = q.shape
    parts_k, parts_v = [], []
    if kc is not None and kc.shape[2] > 0:
        parts_k.append(dequant_keys(kc, ks, kz, g))
        parts_v.append(dequant_values(vc, vs, vz, g))
    if k_res is not None and k_res.shape[2] > 0:
        parts_k.append(np.asarray(k_res).astype(np.float32))
        parts_v.append(np.asarray(v_res).astype(np.float32))
    k_hat = np.concatenate(parts_k, axis=2)
    v_hat = np.concatenate(parts_v, axis=2)
    H_kv = k_hat.shape[1]
    if H_kv != H:
        assert H % H_kv == 0
        rep = H // H_kv
        k_hat = np.repeat(k_hat, rep, axis=1)
        v_hat = np.repeat(v_hat, rep, axis=1)
    scores = np.einsum("bhqd,bhsd->bhqs", q.astype(np.float32), k_hat) * np.float32(scale)
    if causal:
        S_kv = k_hat.shape[2]
        q_abs = S_kv - S_q + np.arange(S_q)[:, None]
        scores = np.where(np.arange(S_kv)[None, :] <= q_abs, scores, -np.inf)
    scores = scores - scores.max(axis=-1, keepdims=True)
    w = np.exp(scores)
    w = w / w.sum(axis=-1, keepdims=True)
    return np.einsum("bhqs,bhsd->bhqd", w, v_hat).astype(np.float32)


def make_inputs(B, H, S_kv, D, b, g, seed=0, H_kv=None):
    """Seeded inputs as in ``tests/metal/test_scalar_attend.py:118-129``."""
    if H_kv is None:
        H_kv = H
    rng = np.random.default_rng(seed)
    levels = (1 << b) - 1
    q = rng.standard_normal((B, H, 1, D)).astype(np.float16)
    kf = rng.standard_normal((B, H_kv, S_kv, D)).astype(np.float32)
    vf = rng.standard_normal((B, H_kv, S_kv, D)).astype(np.float32)
    kc, ks, kz = quant_keys(kf, g, levels)
    vc, vs, vz = quant_values(vf, g, levels)
    return q, kc, ks, kz, vc, vs, vz
