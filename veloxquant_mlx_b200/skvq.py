"""SKVQ primitives: channel reordering and clipped group quantization with clip-factor search.

Same functions, arguments and results as ``veloxquant_mlx/quantizers/skvq.py``
(``channel_permutation`` :77-91, ``invert_permutation`` :94-95, ``apply_permutation`` :98-100,
``clipped_group_quant`` :103-165, ``clipped_group_dequant`` :168-182, ``skvq_round_trip`` :185-209,
byte helpers :212-226) on CUDA tensors. The quantizer and its inverse are the native kernels
``vq_skvq_quantize_pack`` / ``vq_skvq_unpack_dequant``, which keep the codes bit-packed;
``clipped_group_quant`` unpacks them to the reference's one-code-per-byte form.

Not offered natively: group sizes other than 8, 16, 32, 64 and a ragged last group (the
reference pads it by repeating the last channel).
"""

from __future__ import annotations

import ctypes as C
import math
from typing import Sequence

import torch

from . import _lib
from ._lib import check, dtype_code, lib, require_cuda, stream_ptr

DEFAULT_ALPHA_GRID: tuple = (1.0, 0.97, 0.94, 0.90, 0.85)


def _validate(bits: int, group_size: int, alphas: Sequence[float]) -> None:
    if not (1 <= int(bits) <= 8):
        raise ValueError(f"skvq: bits={bits} must be in [1, 8] (uint8 codes)")
    if int(group_size) < 1:
        raise ValueError(f"skvq: group_size={group_size} must be >= 1")
    if len(alphas) == 0:
        raise ValueError("skvq: alphas must be non-empty")
    for a in alphas:
        if not (0.0 < float(a) <= 1.0):
            raise ValueError(f"skvq: alpha={a} must be in (0, 1]")
    if len(alphas) > 8:
        raise ValueError("skvq: at most 8 clip factors are searched natively")


def channel_permutation(x: torch.Tensor) -> torch.Tensor:
    """``[N, D]`` observed rows -> ``[D]`` int32: channels by ascending dynamic range (stable)."""
    x32 = x.float()
    rng = x32.amax(dim=0) - x32.amin(dim=0)
    return torch.argsort(rng, stable=True).to(torch.int32)


def invert_permutation(perm: torch.Tensor) -> torch.Tensor:
    return torch.argsort(perm.long(), stable=True).to(torch.int32)


def apply_permutation(x: torch.Tensor, perm: torch.Tensor) -> torch.Tensor:
    return torch.index_select(x, -1, perm.long())


def quantize_pack(x: torch.Tensor, bits: int, group_size: int, alphas: Sequence[float] = DEFAULT_ALPHA_GRID, *,
                  perm: torch.Tensor | None = None, out=None, tok_offset: int = 0):
    """Quantize ``x [n_bh, n_tok, D]`` (a view whose (batch, head) blocks may be strided; rows
    contiguous) into packed codes ``[n_bh, cap, D*bits/8]`` uint8 and ``lo`` / ``scale``
    ``[n_bh, cap, D/group_size]`` float32. ``perm [n_heads, D]`` int32 gathers the channels first
    (block ``i`` uses row ``i % n_heads``). ``out=(codes, lo, scale)`` writes rows
    ``tok_offset .. tok_offset+n_tok`` of existing buffers; otherwise new ones are returned."""
    _validate(bits, group_size, alphas)
    require_cuda(x, "skvq.quantize_pack")
    if x.ndim != 3 or x.stride(2) != 1 or x.stride(1) != x.shape[2]:
        raise ValueError(f"skvq.quantize_pack: x must be [n_bh, n_tok, D] with contiguous rows, got {tuple(x.shape)} / {x.stride()}")
    n_bh, n_tok, D = x.shape
    if D % group_size or (D * bits) % 8:
        raise ValueError(f"skvq: D={D} must be a multiple of group_size={group_size} (a ragged last group is not offered natively)")
    G = D // group_size
    if out is None:
        codes = torch.empty((n_bh, n_tok, D * bits // 8), dtype=torch.uint8, device=x.device)
        lo = torch.empty((n_bh, n_tok, G), dtype=torch.float32, device=x.device)
        scale = torch.empty_like(lo)
        tok_offset = 0
    else:
        codes, lo, scale = out
        if codes.shape[2] != D * bits // 8 or lo.shape[2] != G or not (codes.shape[:2] == lo.shape[:2] == scale.shape[:2]):
            raise ValueError("skvq.quantize_pack: output buffers do not match")
        if tok_offset + n_tok > codes.shape[1] or not (codes.is_contiguous() and lo.is_contiguous() and scale.is_contiguous()):
            raise ValueError("skvq.quantize_pack: output buffers too small or not contiguous")
    a = _lib.SkvqQuantArgs()
    a.x, a.x_stride_bh, a.x_dtype = x.data_ptr(), x.stride(0) if n_bh > 1 else n_tok * D, dtype_code(x.dtype)
    n_heads = 1
    if perm is not None:
        if perm.dtype != torch.int32 or perm.ndim != 2 or perm.shape[1] != D or not perm.is_contiguous() or perm.device != x.device:
            raise ValueError("skvq.quantize_pack: perm must be a contiguous int32 [n_heads, D] tensor on x's device")
        n_heads, a.perm = perm.shape[0], perm.data_ptr()
    cap = codes.shape[1]
    a.codes = codes.data_ptr() + tok_offset * codes.shape[2]
    a.lo, a.scale = lo.data_ptr() + tok_offset * G * 4, scale.data_ptr() + tok_offset * G * 4
    a.q_stride_bh = cap
    for i, al in enumerate(alphas):
        a.alphas[i] = float(al)
    a.n_alphas, a.n_bh, a.n_heads, a.n_tok, a.D, a.bits, a.group_size = len(alphas), n_bh, n_heads, n_tok, D, bits, group_size
    with _lib.on_device(x.device):
        check(lib().vq_skvq_quantize_pack(C.byref(a), stream_ptr(x.device)), "skvq.quantize_pack")
    return codes, lo, scale


def unpack_dequant(codes: torch.Tensor, lo: torch.Tensor, scale: torch.Tensor, bits: int, group_size: int, n_tok: int,
                   dtype: torch.dtype, *, inv_perm: torch.Tensor | None = None, out: torch.Tensor | None = None) -> torch.Tensor:
    """The first ``n_tok`` rows of packed buffers ``[n_bh, cap, D*bits/8]`` back to ``[n_bh, n_tok, D]``
    in ``dtype``; ``inv_perm [n_heads, D]`` undoes the channel gather. ``out`` may be a strided view
    ``[n_bh, n_tok, D]`` with contiguous rows."""
    require_cuda(codes, "skvq.unpack_dequant")
    n_bh, cap, row_bytes = codes.shape
    D = row_bytes * 8 // bits
    if out is None:
        out = torch.empty((n_bh, n_tok, D), dtype=dtype, device=codes.device)
    elif out.shape != (n_bh, n_tok, D) or out.stride(2) != 1 or out.stride(1) != D or out.dtype != dtype:
        raise ValueError("skvq.unpack_dequant: out must be [n_bh, n_tok, D] with contiguous rows")
    if n_tok > cap or not (codes.is_contiguous() and lo.is_contiguous() and scale.is_contiguous()):
        raise ValueError("skvq.unpack_dequant: bad buffers")
    a = _lib.SkvqDequantArgs()
    a.codes, a.lo, a.scale, a.q_stride_bh = codes.data_ptr(), lo.data_ptr(), scale.data_ptr(), cap
    n_heads = 1
    if inv_perm is not None:
        if inv_perm.dtype != torch.int32 or inv_perm.ndim != 2 or inv_perm.shape[1] != D or not inv_perm.is_contiguous():
            raise ValueError("skvq.unpack_dequant: inv_perm must be a contiguous int32 [n_heads, D] tensor")
        n_heads, a.inv_perm = inv_perm.shape[0], inv_perm.data_ptr()
    a.out, a.out_stride_bh, a.out_dtype = out.data_ptr(), out.stride(0) if n_bh > 1 else n_tok * D, dtype_code(dtype)
    a.n_bh, a.n_heads, a.n_tok, a.D, a.bits, a.group_size = n_bh, n_heads, n_tok, D, bits, group_size
    with _lib.on_device(codes.device):
        check(lib().vq_skvq_unpack_dequant(C.byref(a), stream_ptr(codes.device)), "skvq.unpack_dequant")
    return out


def clipped_group_quant(x: torch.Tensor, bits: int, group_size: int, alphas: Sequence[float] = DEFAULT_ALPHA_GRID):
    """``[N, D]`` -> ``(codes uint8 [N, D], lo float32 [N, G], scale float32 [N, G])``."""
    _validate(bits, group_size, alphas)
    if x.ndim != 2:
        raise ValueError(f"skvq.clipped_group_quant: x must be [N, D], got {tuple(x.shape)}")
    n, d = x.shape
    packed, lo, scale = quantize_pack(x.contiguous().reshape(1, n, d), bits, group_size, alphas)
    if bits == 8:
        return packed.reshape(n, d), lo[0], scale[0]
    # one code per byte: the packed codes "dequantized" with scale 1 and offset 0
    codes = unpack_dequant(packed, torch.zeros_like(lo), torch.ones_like(scale), bits, group_size, n, torch.float32)
    return codes[0].to(torch.uint8), lo[0], scale[0]


def clipped_group_dequant(codes: torch.Tensor, lo: torch.Tensor, scale: torch.Tensor, group_size: int, d: int) -> torch.Tensor:
    """Reconstruct ``[N, d]`` float32 rows from one-code-per-byte codes (8-bit packed form)."""
    n = codes.shape[0]
    return unpack_dequant(codes.contiguous().reshape(1, n, -1), lo.contiguous().reshape(1, n, -1), scale.contiguous().reshape(1, n, -1),
                          8, group_size, n, torch.float32)[0][:, :d]


def skvq_round_trip(x: torch.Tensor, perm, bits: int, group_size: int, alphas: Sequence[float] = DEFAULT_ALPHA_GRID) -> torch.Tensor:
    """Permute -> clipped group quant -> dequant -> inverse permute, in ``x``'s dtype (one quantize and
    one dequantize launch; the gathers are folded into them)."""
    n, d = x.shape
    p = None if perm is None else perm.reshape(1, d).to(torch.int32).contiguous()
    packed, lo, scale = quantize_pack(x.contiguous().reshape(1, n, d), bits, group_size, alphas, perm=p)
    inv = None if perm is None else invert_permutation(perm).reshape(1, d).contiguous()
    return unpack_dequant(packed, lo, scale, bits, group_size, n, x.dtype, inv_perm=inv)[0]


def skvq_compressed_bytes(n_tokens: int, d: int, bits: int, group_size: int) -> int:
    n_groups = (d + group_size - 1) // group_size
    return math.ceil(n_tokens * d * bits / 8) + n_tokens * n_groups * 2 * 2


def skvq_fp16_bytes(n_tokens: int, d: int) -> int:
    return n_tokens * d * 2


__all__ = ["DEFAULT_ALPHA_GRID", "channel_permutation", "invert_permutation", "apply_permutation", "clipped_group_quant",
           "clipped_group_dequant", "skvq_round_trip", "skvq_compressed_bytes", "skvq_fp16_bytes", "quantize_pack", "unpack_dequant"]
