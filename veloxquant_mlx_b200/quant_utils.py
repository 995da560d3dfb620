"""The shared asymmetric min/max group-quantization core of the reference's sibling methods
(SKVQ, Kitty, AgeTiered, AdaKV, ZipCache, GEAR, ...): ``quantizers/_quant_utils.py:9-230``,
with the same function names and return conventions, on ``torch`` CUDA tensors.

Groups run along the token axis, one (scale, zero) per group and channel -- exactly the
per-channel key quantization of the KIVI path, so every function here is one call of
``vq_kivi_quantize`` (``axis = 0``, one code per byte): float32 min/max,
``scale = max((max-min)/levels, 1e-8)``, ``codes = clip(round((x-min)/scale), 0, levels)``
with round-half-even, a ragged final group padded with its last row. Results are bit-identical
to the oracle's ``quant_keys`` (and through it to the reference's NumPy twin).
"""

from __future__ import annotations

import torch

from . import kernels

_EPS = 1e-8


def _check(x: torch.Tensor, ndim: int, who: str, b: int, group_size: int) -> None:
    if x.ndim != ndim:
        raise ValueError(f"{who}: x must be {ndim}D, got {tuple(x.shape)}")
    if not 1 <= b <= 8:
        raise ValueError(f"{who}: b={b} must be in [1, 8]")
    if group_size < 1:
        raise ValueError(f"{who}: group_size={group_size} must be >= 1")
    if x.dtype not in (torch.float16, torch.bfloat16, torch.float32):
        raise ValueError(f"{who}: unsupported dtype {x.dtype}")


def _group_quant_codes_batched(x: torch.Tensor, b: int, group_size: int = 32):
    """``x [N, S, D]`` -> ``(codes f32 [N, n_groups, group_size, D], scale, zero f32
    [N, n_groups, 1, D])``; groups along axis 1, rows of the padded tail repeat the last row's
    codes (reference: ``_quant_utils.py:95-138``)."""
    _check(x, 3, "_group_quant_codes_batched", b, group_size)
    n, s, d = x.shape
    gs = group_size
    n_groups = (s + gs - 1) // gs
    if n == 0 or s == 0:
        z = torch.zeros((n, n_groups, gs, d), dtype=torch.float32, device=x.device)
        return z, torch.zeros((n, n_groups, 1, d), dtype=torch.float32, device=x.device), z[:, :, :1]
    codes, scale, zero = kernels.kivi_quantize(x.reshape(1, n, s, d), -2, gs, b, store_bits=8, eps=_EPS)
    codes = codes.reshape(n, s, d)
    pad = n_groups * gs - s
    if pad:
        codes = torch.cat([codes, codes[:, -1:].expand(n, pad, d)], dim=1)
    return (codes.to(torch.float32).reshape(n, n_groups, gs, d), scale.reshape(n, n_groups, 1, d),
            zero.reshape(n, n_groups, 1, d))


def _group_dequant_codes_batched(codes, scale, zero, s: int, group_size: int = 32) -> torch.Tensor:
    """Reconstruct ``[N, s, D]`` float32 from :func:`_group_quant_codes_batched`'s output
    (product and sum rounded separately; reference: ``_quant_utils.py:141-168``)."""
    n, d = codes.shape[0], codes.shape[-1]
    n_groups = scale.shape[1]
    codes = codes.reshape(n, n_groups, group_size, d)
    recon = codes * scale.reshape(n, n_groups, 1, d)
    recon = recon + zero.reshape(n, n_groups, 1, d)
    return recon.reshape(n, n_groups * group_size, d)[:, :s]


def _group_quant_dequant_batched(x: torch.Tensor, b: int, group_size: int = 32) -> torch.Tensor:
    """Round trip of ``x [N, S, D]``; float16 result (reference: ``_quant_utils.py:171-215``).
    One launch: the quantize kernel writes the reconstruction itself."""
    _check(x, 3, "_group_quant_dequant_batched", b, group_size)
    n, s, d = x.shape
    if n == 0 or s == 0:
        return x.to(torch.float16)
    # the reference casts to float32, reconstructs in float32 and rounds once to float16
    rec = kernels.kivi_group_quant_dequant(x.to(torch.float32).reshape(1, n, s, d), -2, group_size, (1 << b) - 1, eps=_EPS)
    return rec.reshape(n, s, d).to(torch.float16)


def _group_quant_codes(x: torch.Tensor, b: int, group_size: int = 32):
    """``x [N, D]`` -> ``(codes f32 [n_groups, group_size, D], scale, zero f32 [n_groups, 1, D])``
    (reference: ``_quant_utils.py:9-46``)."""
    _check(x, 2, "_group_quant_codes", b, group_size)
    codes, scale, zero = _group_quant_codes_batched(x[None], b, group_size)
    return codes[0], scale[0], zero[0]


def _group_dequant_codes(codes, scale, zero, n: int, group_size: int = 32) -> torch.Tensor:
    """Reconstruct ``[n, D]`` float32 (reference: ``_quant_utils.py:49-75``)."""
    d = codes.shape[-1]
    n_groups = scale.shape[0]
    return _group_dequant_codes_batched(codes.reshape(1, n_groups, group_size, d), scale.reshape(1, n_groups, 1, d),
                                        zero.reshape(1, n_groups, 1, d), n, group_size)[0]


def _group_quant_dequant(x: torch.Tensor, b: int, group_size: int = 32) -> torch.Tensor:
    """Round trip of ``x [N, D]``; float16 result (reference: ``_quant_utils.py:78-92``)."""
    _check(x, 2, "_group_quant_dequant", b, group_size)
    return _group_quant_dequant_batched(x[None], b, group_size)[0]


__all__ = ["_group_quant_codes", "_group_dequant_codes", "_group_quant_dequant", "_group_quant_codes_batched",
           "_group_dequant_codes_batched", "_group_quant_dequant_batched"]
