"""VecInfer product-VQ wrappers on ``torch.Tensor`` (reference: ``allocators/vecinfer.py``,
``metal/_vecinfer.py``, ``metal/fused_sdpa.py``). The nearest-centroid search, the gather and
the LUT attention run in ``libvqb200.so``. The dual transform exists twice: as the reference
writes it (an elementwise scale and a D x D matrix product with any matrix ``H``), and, for the
Walsh-Hadamard matrix itself, as a native butterfly with a fixed summation order
(``dual_transform_*_wht``), which is what the caches use.
"""

from __future__ import annotations

import ctypes as C
import functools
import math

import numpy as np
import torch

from . import _lib
from ._lib import VqAttendArgs, VqEncodeArgs, check, dtype_code, lib, require_cuda, stream_ptr
from .kernels import _FLOAT_DTYPES, _workspace

_INDEX_DTYPES = {torch.uint8: 1, torch.int16: 2, torch.uint16: 2, torch.int32: 4, torch.uint32: 4}


def walsh_hadamard_matrix(d: int, dtype=torch.float32, device=None) -> torch.Tensor:
    """Orthonormal Sylvester Walsh-Hadamard matrix ``[d, d]`` (``allocators/vecinfer.py:60-87``)."""
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
    return torch.from_numpy(H).to(dtype=dtype, device=device)


def _smooth_for(x: torch.Tensor, smooth: torch.Tensor, for_query: bool, who: str) -> torch.Tensor:
    if smooth.ndim in (1, 2) and smooth.shape[-1] not in (1, x.shape[-1]):
        # (the reference's array library answers an impossible broadcast with a ValueError)
        raise ValueError(f"{who}: cannot broadcast smooth {tuple(smooth.shape)} to {tuple(x.shape)}")
    if smooth.ndim == 1:
        return smooth.to(x.dtype)
    if smooth.ndim != 2:
        raise ValueError(f"smooth must be 1D or 2D, got {tuple(smooth.shape)}")
    if x.ndim >= 3 and x.shape[-3] == smooth.shape[0]:
        return smooth[:, None, :].to(x.dtype)
    if for_query and x.ndim >= 3 and smooth.shape[0] > 0 and x.shape[-3] % smooth.shape[0] == 0:
        rep = x.shape[-3] // smooth.shape[0]
        return smooth.repeat_interleave(rep, dim=0)[:, None, :].to(x.dtype)
    if x.shape[-1] == smooth.shape[-1]:
        return smooth.mean(dim=0).to(x.dtype)
    raise ValueError(f"{who}: cannot broadcast smooth {tuple(smooth.shape)} to {tuple(x.shape)}")


def apply_dual_transform_keys(K: torch.Tensor, smooth: torch.Tensor, H: torch.Tensor) -> torch.Tensor:
    """``K_tilde = (K / lambda) @ H`` (``allocators/vecinfer.py:93-134``)."""
    return (K / _smooth_for(K, smooth, False, "apply_dual_transform_keys")) @ H.to(K.dtype)


def apply_dual_transform_queries(q: torch.Tensor, smooth: torch.Tensor, H: torch.Tensor) -> torch.Tensor:
    """``q_tilde = (q * lambda) @ H``; per-KV-head factors repeat over their query group
    (``allocators/vecinfer.py:137-184``)."""
    return (q * _smooth_for(q, smooth, True, "apply_dual_transform_queries")) @ H.to(q.dtype)


@functools.lru_cache(maxsize=None)
def wht_entry(d: int) -> float:
    """The common entry magnitude of :func:`walsh_hadamard_matrix` ``(d)``, computed by the same
    float32 recurrence (one multiplication by ``1/sqrt(2)`` per doubling)."""
    if d < 1 or (d & (d - 1)) != 0:
        raise ValueError(f"wht_entry: d={d} must be a power of 2.")
    c = np.array([[1.0]], dtype=np.float32)
    inv_sqrt2 = 1.0 / math.sqrt(2.0)
    size = 1
    while size < d:
        c = c * inv_sqrt2
        size *= 2
    return float(c[0, 0])


def _dual_transform_wht(x: torch.Tensor, smooth, for_query: bool, who: str) -> torch.Tensor:
    if x.ndim < 1 or x.shape[-1] not in (32, 64, 128, 256):
        raise ValueError(f"{who}: head_dim={x.shape[-1] if x.ndim else None} must be 32, 64, 128 or 256")
    if x.dtype not in _FLOAT_DTYPES:
        raise ValueError(f"{who}: unsupported dtype {x.dtype}")
    require_cuda(x, f"{who}: x")
    D = x.shape[-1]
    x = x.contiguous()
    n_rows = x.numel() // D
    sm_ptr, rows, n_heads, tph = None, 0, 1, max(n_rows, 1)
    if smooth is not None:
        # (the broadcasting rule only looks at the shape: a storage-less stand-in of x's shape)
        sm = _smooth_for(torch.empty(x.shape, dtype=torch.float32, device="meta"), smooth.to(torch.float32), for_query, who)
        sm = sm.to(device=x.device, dtype=torch.float32)
        if sm.ndim == 1:
            sm2, n_heads, tph = sm.reshape(1, D).contiguous(), 1, max(n_rows, 1)
        else:  # [heads, 1, D]: one row per head of x's axis -3
            sm2, n_heads, tph = sm.reshape(-1, D).contiguous(), x.shape[-3], x.shape[-2]
        sm_ptr, rows = sm2.data_ptr(), sm2.shape[0]
    out = torch.empty(x.shape, dtype=torch.float32, device=x.device)
    with _lib.on_device(x.device):
        check(lib().vq_vq_dual_transform(x.data_ptr(), dtype_code(x.dtype), n_rows, D, tph, n_heads, sm_ptr, rows,
                                         0 if for_query else 1, wht_entry(D), out.data_ptr(), stream_ptr(x.device)), who)
    return out


def dual_transform_keys_wht(K: torch.Tensor, smooth=None) -> torch.Tensor:
    """``K_tilde = WHT(K / lambda)``: :func:`apply_dual_transform_keys` for the Walsh-Hadamard
    matrix itself, as a butterfly with a fixed float32 summation order (so that the VQ indices
    of the transformed keys are reproducible bit for bit) instead of a matrix product. float32
    result; ``smooth`` as in :func:`apply_dual_transform_keys` or ``None``."""
    return _dual_transform_wht(K, smooth, False, "dual_transform_keys_wht")


def dual_transform_queries_wht(q: torch.Tensor, smooth=None) -> torch.Tensor:
    """``q_tilde = WHT(q * lambda)``, the query side of :func:`dual_transform_keys_wht`."""
    return _dual_transform_wht(q, smooth, True, "dual_transform_queries_wht")


def _codebook_f32(codebook: torch.Tensor, who: str):
    if codebook.ndim not in (2, 3):
        raise ValueError(f"{who}: codebook must be [n_c, sub_dim] or [n_sub, n_c, sub_dim], got {tuple(codebook.shape)}")
    cb = codebook.to(torch.float32).contiguous()
    stacked = cb.shape[0] if cb.ndim == 3 else 0
    return cb, stacked, cb.shape[-2], cb.shape[-1]


def quantize_vq(x: torch.Tensor, codebook: torch.Tensor, sub_dim: int, *,
                index_dtype: torch.dtype = torch.int32) -> torch.Tensor:
    """Nearest-centroid indices ``[..., D // sub_dim]`` (``allocators/vecinfer.py:281-318``).

    float32 distances in the order of ``vecinfer_quantize.metal``; lowest index on ties.
    ``index_dtype=torch.uint8`` stores one byte per index (<= 256 centroids).
    """
    *lead, D = x.shape
    if D % sub_dim != 0:
        raise ValueError(f"quantize_vq: D={D} not divisible by sub_dim={sub_dim}")
    if x.dtype not in _FLOAT_DTYPES:
        raise ValueError(f"quantize_vq: unsupported dtype {x.dtype}")
    require_cuda(x, "quantize_vq: x")
    cb, stacked, n_c, sd = _codebook_f32(codebook.to(x.device), "quantize_vq")
    if sd != sub_dim:
        raise ValueError(f"quantize_vq: codebook width {sd} != sub_dim={sub_dim}")
    n_sub = D // sub_dim
    if stacked and stacked != n_sub:
        raise ValueError(f"quantize_vq: {stacked} stacked codebooks for {n_sub} sub-spaces")
    if index_dtype not in _INDEX_DTYPES:
        raise ValueError(f"quantize_vq: unsupported index dtype {index_dtype}")
    xs = x.contiguous()
    out = torch.empty((*lead, n_sub), dtype=index_dtype, device=x.device)
    n = xs.numel() // sub_dim
    with _lib.on_device(x.device):
        check(lib().vq_vq_quantize(xs.data_ptr(), dtype_code(x.dtype), n, sub_dim, cb.data_ptr(), n_c, stacked,
                                   out.data_ptr(), _INDEX_DTYPES[index_dtype], stream_ptr(x.device)), "quantize_vq")
    return out


def vecinfer_quantize(x: torch.Tensor, codebook: torch.Tensor) -> torch.Tensor:
    """Flat form ``x [N, sub_dim] -> int32 [N]`` (``metal/_vecinfer.py:181-222``)."""
    if x.ndim != 2 or codebook.ndim != 2 or x.shape[1] != codebook.shape[1]:
        raise ValueError(f"vecinfer_quantize: x [N, sub_dim] and codebook [n_c, sub_dim] expected, got "
                         f"{tuple(x.shape)} / {tuple(codebook.shape)}")
    return quantize_vq(x, codebook, x.shape[1]).reshape(-1)


def dequantize_vq(indices: torch.Tensor, codebook: torch.Tensor, *, out_dtype=None) -> torch.Tensor:
    """``[..., n_sub] -> [..., n_sub*sub_dim]`` gather; out-of-range indices clamp to the last
    centroid (``allocators/vecinfer.py:321-335``, ``metal/src/vecinfer_dequant.metal``)."""
    require_cuda(indices, "dequantize_vq: indices")
    if indices.dtype not in _INDEX_DTYPES:
        indices = indices.to(torch.int32)
    cb, stacked, n_c, sd = _codebook_f32(codebook.to(indices.device), "dequantize_vq")
    *lead, n_sub = indices.shape
    out_dtype = out_dtype or (codebook.dtype if codebook.dtype in _FLOAT_DTYPES else torch.float32)
    idx = indices.contiguous()
    out = torch.empty((*lead, n_sub * sd), dtype=out_dtype, device=indices.device)
    with _lib.on_device(indices.device):
        check(lib().vq_vq_dequant(idx.data_ptr(), _INDEX_DTYPES[idx.dtype], idx.numel(), cb.data_ptr(), n_c, sd,
                                  stacked, out.data_ptr(), dtype_code(out_dtype), stream_ptr(indices.device)),
              "dequantize_vq")
    return out


def vecinfer_quantize_metal(x: torch.Tensor, codebook: torch.Tensor, sub_dim: int) -> torch.Tensor:
    """``x [..., D] -> int32 [..., D // sub_dim]`` under the reference's kernel-wrapper name
    (``metal/_vecinfer.py:181-222``)."""
    D = x.shape[-1]
    if D % sub_dim != 0:
        raise ValueError(f"vecinfer_quantize_metal: D={D} not divisible by sub_dim={sub_dim}")
    if codebook.ndim != 2 or codebook.shape[1] != sub_dim:
        raise ValueError(f"vecinfer_quantize_metal: codebook must be [n_centroids, {sub_dim}], got {tuple(codebook.shape)}")
    return quantize_vq(x, codebook, sub_dim)


def vecinfer_dequant_metal(indices: torch.Tensor, codebook: torch.Tensor, out_dtype=None) -> torch.Tensor:
    """Codebook gather under the reference's kernel-wrapper name (``metal/_vecinfer.py:144-178``)."""
    return dequantize_vq(indices, codebook, out_dtype=out_dtype)


def _encode_decode(who: str, x: torch.Tensor, codebook: torch.Tensor, sub_dim: int, H_mat, smooth, keys: bool,
                   index_dtype, want_hat: bool = True, hat_dtype=torch.float16):
    if x.ndim != 4:
        raise ValueError(f"{who}: {'keys' if keys else 'values'} must be 4D, got {tuple(x.shape)}")
    B, Hn, S, D = x.shape
    if D % sub_dim != 0:
        raise ValueError(f"{who}: D={D} not divisible by sub_dim={sub_dim}")
    if D > 512:
        raise ValueError(f"{who}: D={D} > 512 (threadgroup limit)")
    if x.dtype not in _FLOAT_DTYPES:
        raise ValueError(f"{who}: unsupported dtype {x.dtype}")
    require_cuda(x, f"{who}: input")
    cb, stacked, n_c, sd = _codebook_f32(codebook.to(x.device), who)
    if n_c == 0 or sd != sub_dim:
        raise ValueError(f"{who}: codebook must be non-empty [n_centroids, {sub_dim}], got {tuple(codebook.shape)}")
    n_sub = D // sub_dim
    if stacked and stacked != n_sub:
        raise ValueError(f"{who}: {stacked} stacked codebooks for {n_sub} sub-spaces")
    Hf = sm = None
    rows = 1
    if keys and H_mat is not None:
        Hf = H_mat.to(device=x.device, dtype=torch.float32).contiguous()
        if tuple(Hf.shape) != (D, D):
            raise ValueError(f"{who}: H_mat must be [{D}, {D}], got {tuple(Hf.shape)}")
    if keys and smooth is not None:
        sm = smooth.to(device=x.device, dtype=torch.float32)
        sm = sm.reshape(1, D) if sm.ndim == 1 else sm
        if sm.shape[0] not in (1, Hn):
            acc = sm[0].clone()  # rows added in order, then one divide: a fixed summation order
            for r in range(1, sm.shape[0]):
                acc += sm[r]
            # tensor / tensor is a true IEEE divide (a Python-scalar divisor becomes a reciprocal multiply)
            sm = torch.div(acc, torch.full_like(acc, float(sm.shape[0]))).reshape(1, D)
        sm = sm.contiguous()
        rows = sm.shape[0]
    xs = x.contiguous()
    idx = torch.empty((B, Hn, S, n_sub), dtype=index_dtype, device=x.device)
    hat = torch.empty((B, Hn, S, D), dtype=hat_dtype, device=x.device) if want_hat else None
    a = VqEncodeArgs(
        x=xs.data_ptr(), x_dtype=dtype_code(x.dtype), n_tok=B * Hn * S, D=D, sub_dim=sub_dim,
        tok_per_head=max(S, 1), n_heads=Hn, codebook=cb.data_ptr(), n_centroids=n_c,
        stacked_codebooks=1 if stacked else 0, H=Hf.data_ptr() if Hf is not None else None,
        smooth=sm.data_ptr() if sm is not None else None, smooth_rows=rows,
        x_hat=hat.data_ptr() if hat is not None else None, hat_dtype=dtype_code(hat_dtype),
        indices=idx.data_ptr(), index_bytes=_INDEX_DTYPES[index_dtype])
    fn = lib().vq_vq_encode_decode_keys if keys else lib().vq_vq_encode_decode_values
    with _lib.on_device(x.device):
        check(fn(C.byref(a), stream_ptr(x.device)), who)
    return hat, idx


def vecinfer_encode_decode_metal(keys: torch.Tensor, k_codebook: torch.Tensor, sub_dim: int, H_mat: torch.Tensor,
                                 smooth: torch.Tensor | None = None):
    """Fused key encode + decode in one launch: smooth -> WHT -> VQ -> dequant -> inverse WHT ->
    smooth. Returns ``(k_hat float16 [B,H,S,D], k_indices int32 [B,H,S,n_sub])``
    (``metal/_vecinfer.py:225-293``). Smooth rows other than 1 or H are averaged to one row."""
    return _encode_decode("vecinfer_encode_decode_metal", keys, k_codebook, sub_dim, H_mat, smooth, True,
                          torch.int32)


def vecinfer_encode_decode_simple_metal(values: torch.Tensor, v_codebook: torch.Tensor, sub_dim: int):
    """Fused value quantize + dequantize. Returns ``(v_hat float16, v_indices uint32)``
    (``metal/_vecinfer.py:296-345``)."""
    return _encode_decode("vecinfer_encode_decode_simple_metal", values, v_codebook, sub_dim, None, None, False,
                          torch.uint32)


def vecinfer_encode_keys(keys: torch.Tensor, k_codebook: torch.Tensor, sub_dim: int, H_mat, smooth=None, *,
                         index_dtype=torch.uint8) -> torch.Tensor:
    """Indices only (the form a memory-bound cache stores): the same launch without the decode
    half. No counterpart under this name in the reference."""
    return _encode_decode("vecinfer_encode_keys", keys, k_codebook, sub_dim, H_mat, smooth, True, index_dtype,
                          want_hat=False)[1]


def compute_query_lut(q_tilde: torch.Tensor, codebook: torch.Tensor, sub_dim: int) -> torch.Tensor:
    """``lut[..., s, c] = q_sub[..., s, :] . codebook[c]`` (``allocators/vecinfer.py:341-359``)."""
    *lead, D = q_tilde.shape
    if D % sub_dim != 0:
        raise ValueError(f"compute_query_lut: D={D} not divisible by sub_dim={sub_dim}")
    q_sub = q_tilde.reshape(*lead, D // sub_dim, sub_dim)
    return q_sub @ codebook.to(q_sub.dtype).T


def fused_sdpa_vq(q_tilde: torch.Tensor, k_indices: torch.Tensor, k_codebook: torch.Tensor,
                  v, v_codebook, scale: float, *, causal: bool = True, sliding_window: int = 0,
                  out_dtype=None, s_kv: int | None = None, n_splits: int = 0) -> torch.Tensor:
    """Attention over VQ-coded keys through a per-query lookup table.

    Same arguments as ``metal_fused_sdpa`` (``metal/fused_sdpa.py:200-299``): ``q_tilde
    [B,H_q,S_q,D]`` already dual-transformed, ``k_indices [B,H_kv,S_kv,n_sub]``, key codebook
    ``[n_c, sub_dim]`` (or stacked per sub-space). Values are VQ-coded (``v`` = indices
    ``[B,H_kv,S_kv,n_sub_v]`` with ``v_codebook``) or, with ``v_codebook=None``, a dense
    ``[B,H_kv,S_kv,D]`` tensor. ``s_kv`` limits attention to the first rows of larger buffers.
    """
    if q_tilde.ndim != 4 or k_indices.ndim != 4:
        raise ValueError("fused_sdpa: q_tilde and k_indices must be 4D")
    B, H_q, S_q, D = q_tilde.shape
    _, H_kv, cap, n_sub = k_indices.shape
    S_kv = cap if s_kv is None else int(s_kv)
    if k_codebook.ndim in (2, 3) and n_sub * k_codebook.shape[-1] != D:
        raise ValueError(f"fused_sdpa: D={D} must equal n_sub*sub_dim={n_sub * k_codebook.shape[-1]}.")
    if H_q % H_kv != 0:
        raise ValueError(f"fused_sdpa: H_q={H_q} must be a multiple of H_kv={H_kv}.")
    require_cuda(q_tilde, "fused_sdpa: q_tilde")
    kcb, k_stacked, n_c, sub_dim = _codebook_f32(k_codebook.to(q_tilde.device), "fused_sdpa")
    if k_indices.dtype not in _INDEX_DTYPES:
        k_indices = k_indices.to(torch.int32)
    k_indices = k_indices.contiguous()
    q = q_tilde.contiguous()
    if q.dtype not in _FLOAT_DTYPES:
        q = q.to(torch.float32)
    out_dtype = out_dtype or q_tilde.dtype
    out = torch.empty((B, H_q, S_q, D), dtype=out_dtype, device=q.device)
    a = VqAttendArgs(q=q.data_ptr(), out=out.data_ptr(), q_dtype=dtype_code(q.dtype), out_dtype=dtype_code(out_dtype),
                     B=B, H_q=H_q, H_kv=H_kv, S_q=S_q, S_kv=S_kv, D=D, kv_stride_tok=cap, scale=float(scale),
                     causal=int(bool(causal)), sliding_window=int(sliding_window or 0),
                     k_indices=k_indices.data_ptr(), k_index_bytes=_INDEX_DTYPES[k_indices.dtype],
                     k_codebook=kcb.data_ptr(), k_n_centroids=n_c, k_sub_dim=sub_dim, k_stacked=k_stacked,
                     n_splits=int(n_splits))
    keep = [kcb]
    if v_codebook is not None:
        vcb, v_stacked, n_c_v, sub_dim_v = _codebook_f32(v_codebook.to(q.device), "fused_sdpa")
        if v_stacked:
            raise ValueError("fused_sdpa: stacked value codebooks are not supported")
        n_sub_v = v.shape[-1]
        if n_sub_v * sub_dim_v != D:
            raise ValueError(f"fused_sdpa: D={D} must equal n_sub_v*sub_dim_v={n_sub_v * sub_dim_v}.")
        if v.shape[2] != cap:
            raise ValueError("fused_sdpa: k_indices and v_indices must share their token capacity")
        if v.dtype not in _INDEX_DTYPES:
            v = v.to(torch.int32)
        v = v.contiguous()
        a.v_mode, a.v, a.v_index_bytes = 1, v.data_ptr(), _INDEX_DTYPES[v.dtype]
        a.v_codebook, a.v_n_centroids, a.v_sub_dim = vcb.data_ptr(), n_c_v, sub_dim_v
        keep.append(vcb)
    else:
        if v.ndim != 4 or v.shape[-1] != D or v.shape[2] != cap or v.dtype not in _FLOAT_DTYPES:
            raise ValueError(f"fused_sdpa: dense values must be float [B,H_kv,{cap},{D}], got {tuple(v.shape)}")
        v = v.contiguous()
        a.v_mode, a.v, a.v_dtype = 0, v.data_ptr(), dtype_code(v.dtype)
    with _lib.on_device(q.device):
        ws = _workspace(q.device, lib().vq_vq_attend_workspace_bytes(C.byref(a)))
        a.workspace, a.workspace_bytes = ws.data_ptr(), ws.numel()
        check(lib().vq_vq_decode_attend(C.byref(a), stream_ptr(q.device)), "fused_sdpa")
    return out


def supports_shape(n_centroids: int, n_sub: int, head_dim: int) -> bool:
    """Whether the lookup-table attention of this package takes a configuration (the reference's
    check of its own kernel's caps, ``metal/fused_sdpa.py:141-147``: 256 centroids, 16 sub-spaces,
    head_dim 256). Here: head_dim a multiple of 32 up to 256, and one query head's table
    (``n_sub * n_centroids`` float32) within 200 KiB of shared memory; the query heads of one KV head
    share a thread block, up to eight of them, and their tables must fit together."""
    return (n_centroids >= 1 and n_sub >= 1 and 1 <= head_dim <= 256 and head_dim % 32 == 0
            and n_sub * n_centroids * 4 <= 200 * 1024)


def metal_fused_sdpa(q_tilde, k_indices, k_codebook, v_indices, v_codebook, scale, *, causal=True,
                     sliding_window=0, out_dtype=None):
    """The reference's name for :func:`fused_sdpa_vq` (``metal/fused_sdpa.py:200``)."""
    return fused_sdpa_vq(q_tilde, k_indices, k_codebook, v_indices, v_codebook, scale, causal=causal,
                         sliding_window=sliding_window, out_dtype=out_dtype)


__all__ = ["walsh_hadamard_matrix", "apply_dual_transform_keys", "apply_dual_transform_queries", "quantize_vq",
           "vecinfer_quantize", "dequantize_vq", "compute_query_lut", "fused_sdpa_vq", "metal_fused_sdpa",
           "vecinfer_quantize_metal", "vecinfer_dequant_metal", "vecinfer_encode_decode_metal",
           "vecinfer_encode_decode_simple_metal", "vecinfer_encode_keys", "supports_shape"]
