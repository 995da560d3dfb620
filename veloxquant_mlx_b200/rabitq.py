"""RaBitQ 1-bit key wrappers on ``torch.Tensor`` (reference: ``metal/_rabitq_encode.py``,
``metal/_rabitq_attend.py``, ``metal/_rabitq_values.py``, ``metal/_rabitq.py``,
``quantizers/rabitq.py:64-70,197-206``, ``math/rotation.py:56-100``).
"""

from __future__ import annotations

import ctypes as C

import numpy as np
import torch

from . import _lib
from ._lib import RabitqAttendArgs, RabitqPrefillArgs, check, dtype_code, lib, require_cuda, stream_ptr
from .kernels import _FLOAT_DTYPES, _workspace


def make_hadamard_diagonal(d: int, seed: int = 42) -> np.ndarray:
    """Seeded +-1 diagonal of the randomized Hadamard rotation (``math/rotation.py:56-77``)."""
    if d < 1:
        raise ValueError(f"make_hadamard_diagonal: d must be >= 1, got {d}")
    rng = np.random.default_rng(seed)
    return rng.choice(np.array([-1.0, 1.0], dtype=np.float32), size=d)


def make_rotation_matrix(d: int, seed: int = 42) -> np.ndarray:
    """Haar-distributed rotation: Q of the QR factorisation of a seeded Gaussian matrix
    (``math/rotation.py:80-100``)."""
    if d < 1:
        raise ValueError(f"make_rotation_matrix: d must be >= 1, got {d}")
    rng = np.random.default_rng(seed)
    G = rng.standard_normal((d, d)).astype(np.float64)
    Q, _ = np.linalg.qr(G)
    return Q.astype(np.float64)


def _encode(keys: torch.Tensor, diag, rotate: int, who: str):
    if keys.ndim != 2:
        raise ValueError(f"{who}: keys must be 2D [N, D], got {tuple(keys.shape)}")
    N, D = keys.shape
    if D % 8 != 0:
        raise ValueError(f"{who}: D={D} must be divisible by 8")
    if rotate and D & (D - 1) != 0:
        raise ValueError(f"{who}: D={D} must be a power of two")
    if D > 1024:
        raise ValueError(f"{who}: D={D} exceeds the 1024 limit")
    if keys.dtype not in _FLOAT_DTYPES:
        raise ValueError(f"{who}: unsupported dtype {keys.dtype}")
    if rotate and tuple(diag.shape) != (D,):
        raise ValueError(f"{who}: diag must be [{D}], got {tuple(diag.shape)}")
    require_cuda(keys, f"{who}: keys")
    dptr = None
    if rotate:
        diag = diag.to(device=keys.device, dtype=torch.float32).contiguous()
        dptr = diag.data_ptr()
    keys = keys.contiguous()
    bits = torch.empty((N, D // 8), dtype=torch.uint8, device=keys.device)
    mag = torch.empty((N,), dtype=torch.float32, device=keys.device)
    with _lib.on_device(keys.device):
        check(lib().vq_rabitq_encode(keys.data_ptr(), dtype_code(keys.dtype), N, D, dptr, rotate,
                                     bits.data_ptr(), mag.data_ptr(), stream_ptr(keys.device)), who)
    return bits, mag


def rabitq_encode(keys: torch.Tensor, diag: torch.Tensor):
    """``y = WHT(keys*diag)/sqrt(D)`` -> ``(k_bits u8 [N,D/8], k_mag f32 [N])``
    (``metal/_rabitq_encode.py:83-128``)."""
    return _encode(keys, diag, 1, "rabitq_encode")


def rabitq_encode_rotated(y: torch.Tensor):
    """Sign bits and L1 magnitude of already-rotated rows, e.g. ``keys @ R.T`` with a dense
    QR rotation (``quantizers/rabitq.py:64-70`` ``_pack_signs``)."""
    return _encode(y, None, 0, "rabitq_encode_rotated")


def rabitq_pack_values(v_idx: torch.Tensor) -> torch.Tensor:
    """Two 4-bit indices per byte, low nibble = even element (``metal/_rabitq_values.py:64-95``)."""
    if v_idx.shape[-1] % 2 != 0:
        raise ValueError(f"rabitq_pack_values: last dimension must be even, got {v_idx.shape[-1]}")
    require_cuda(v_idx, "rabitq_pack_values: v_idx")
    v = v_idx.to(torch.uint8).contiguous()
    out = torch.empty((*v.shape[:-1], v.shape[-1] // 2), dtype=torch.uint8, device=v.device)
    with _lib.on_device(v.device):
        check(lib().vq_rabitq_pack_values(v.data_ptr(), out.numel(), out.data_ptr(), stream_ptr(v.device)),
              "rabitq_pack_values")
    return out


def rabitq_hamming_score(qbits: torch.Tensor, bits: torch.Tensor, Cx: torch.Tensor, scale) -> torch.Tensor:
    """``score[i] = popcount(qbits ^ bits[i]) * scale + Cx[i]`` (``metal/_rabitq.py:63-103``, same argument
    order): ``qbits [D//8]`` and ``bits [N, D//8]`` uint8, ``Cx [N]``, ``scale`` a number or a one-element
    tensor. Returns float32 ``[N]``."""
    if qbits.ndim != 1:
        raise ValueError(f"rabitq_hamming_score: qbits must be 1D, got {tuple(qbits.shape)}")
    if bits.ndim != 2:
        raise ValueError(f"rabitq_hamming_score: bits must be 2D [N, D//8], got {tuple(bits.shape)}")
    N, n_bytes = bits.shape
    if qbits.shape[0] != n_bytes:
        raise ValueError(f"rabitq_hamming_score: qbits length {qbits.shape[0]} != bits cols {n_bytes}")
    if not isinstance(Cx, torch.Tensor) or Cx.numel() != N:
        raise ValueError(f"rabitq_hamming_score: Cx must hold one constant per candidate ({N}), got "
                         f"{tuple(Cx.shape) if isinstance(Cx, torch.Tensor) else type(Cx).__name__}")
    if isinstance(scale, torch.Tensor):
        if scale.numel() != 1:
            raise ValueError(f"rabitq_hamming_score: scale must be a single value, got {tuple(scale.shape)}")
        scale = scale.reshape(()).item()
    require_cuda(bits, "rabitq_hamming_score: bits")
    qb = qbits.to(device=bits.device, dtype=torch.uint8).contiguous()
    bb = bits.to(torch.uint8).contiguous()
    cxf = Cx.reshape(N).to(device=bits.device, dtype=torch.float32).contiguous()
    out = torch.empty((N,), dtype=torch.float32, device=bits.device)
    with _lib.on_device(bits.device):
        check(lib().vq_rabitq_hamming_score(qb.data_ptr(), bb.data_ptr(), N, n_bytes, float(scale), cxf.data_ptr(),
                                            out.data_ptr(), stream_ptr(bits.device)), "rabitq_hamming_score")
    return out


def rabitq_fused_attend(q, q_scale, k_bits, k_mag, k_const, v_idx, v_cents=None, *, s_kv=None,
                        out_dtype=torch.float16, n_splits: int = 0) -> torch.Tensor:
    """Popcount-scored attention over sign-bit keys (``metal/_rabitq_attend.py:112-216``).

    ``q [B,H_q,S_q,D]``, ``q_scale [B,H_q,S_q]``, ``k_bits [B,H_kv,S,D/8]``, ``k_mag``/``k_const
    [B,H_kv,S]`` (``k_const`` may be ``None``). Values: codebook indices ``u8 [..,D]`` or
    nibble-packed ``[..,D/2]`` with ``v_cents [<=16]`` (reference form), or, with
    ``v_cents=None``, a dense float ``[B,H_kv,S,D]`` tensor. ``H_q`` may be a multiple of
    ``H_kv`` (contiguous GQA blocks; the reference kernel has ``H_q == H_kv``).
    """
    fn = "rabitq_fused_attend"
    if q.ndim != 4:
        raise ValueError(f"{fn}: q must be 4D, got {tuple(q.shape)}")
    require_cuda(q, f"{fn}: q")
    B, H, S_q, D = q.shape
    if D % 8 != 0:
        raise ValueError(f"{fn}: D={D} must be divisible by 8")
    if D > 256:
        raise ValueError(f"{fn}: D={D} exceeds the 256 limit")
    n_bytes = D // 8
    if k_bits.ndim != 4 or k_bits.shape[0] != B or k_bits.shape[3] != n_bytes or H % k_bits.shape[1] != 0:
        raise ValueError(f"{fn}: k_bits must be [B, H_kv, S_kv, {n_bytes}] with H_kv dividing {H}, got {tuple(k_bits.shape)}")
    H_kv, cap = k_bits.shape[1], k_bits.shape[2]
    S_kv = cap if s_kv is None else int(s_kv)
    if tuple(k_mag.shape) != (B, H_kv, cap):
        raise ValueError(f"{fn}: k_mag must be {(B, H_kv, cap)}, got {tuple(k_mag.shape)}")
    if k_const is not None and tuple(k_const.shape) != (B, H_kv, cap):
        raise ValueError(f"{fn}: k_const must be {(B, H_kv, cap)}, got {tuple(k_const.shape)}")
    if tuple(q_scale.shape) != (B, H, S_q):
        raise ValueError(f"{fn}: q_scale must be {(B, H, S_q)}, got {tuple(q_scale.shape)}")
    q = q.contiguous()
    out = torch.empty((B, H, S_q, D), dtype=out_dtype, device=q.device)
    qs = q_scale.to(torch.float32).contiguous()
    kb = k_bits.to(torch.uint8).contiguous()
    km = k_mag.to(torch.float32).contiguous()
    kc = None if k_const is None else k_const.to(torch.float32).contiguous()
    a = RabitqAttendArgs(q=q.data_ptr(), out=out.data_ptr(), q_dtype=dtype_code(q.dtype), out_dtype=dtype_code(out_dtype),
                         B=B, H_q=H, H_kv=H_kv, S_q=S_q, S_kv=S_kv, D=D, kv_stride_tok=cap,
                         q_scale=qs.data_ptr(), k_bits=kb.data_ptr(), k_mag=km.data_ptr(),
                         k_const=None if kc is None else kc.data_ptr(), n_splits=int(n_splits))
    if v_cents is None:
        if tuple(v_idx.shape) != (B, H_kv, cap, D) or v_idx.dtype not in _FLOAT_DTYPES:
            raise ValueError(f"{fn}: dense values must be float {(B, H_kv, cap, D)}, got {tuple(v_idx.shape)}")
        v = v_idx.contiguous()
        a.v_mode, a.v, a.v_dtype = 0, v.data_ptr(), dtype_code(v.dtype)
        cents = None
    else:
        if tuple(v_idx.shape) == (B, H_kv, cap, D):
            a.v_mode = 2
        elif tuple(v_idx.shape) == (B, H_kv, cap, D // 2):
            a.v_mode = 3
        else:
            raise ValueError(f"{fn}: v_idx must be {(B, H_kv, cap, D)} (one index per byte) or "
                             f"{(B, H_kv, cap, D // 2)} (nibble-packed), got {tuple(v_idx.shape)}")
        if v_cents.ndim != 1:
            raise ValueError(f"{fn}: v_cents must be 1D, got {tuple(v_cents.shape)}")
        if v_cents.shape[0] > 16:
            raise ValueError(f"{fn}: v_cents holds {v_cents.shape[0]} entries; at most 16 are supported")
        v = v_idx.to(torch.uint8).contiguous()
        cents = v_cents.to(device=q.device, dtype=torch.float32).contiguous()
        a.v, a.v_cents, a.n_cents = v.data_ptr(), cents.data_ptr(), cents.shape[0]
    with _lib.on_device(q.device):
        ws = _workspace(q.device, lib().vq_rabitq_attend_workspace_bytes(C.byref(a)))
        a.workspace, a.workspace_bytes = ws.data_ptr(), ws.numel()
        check(lib().vq_rabitq_decode_attend(C.byref(a), stream_ptr(q.device)), fn)
    return out


def rabitq_prefill_attend(q, scale, k_bits, k_mag, k_const, v_idx, v_cents=None, *, causal: bool = False,
                          s_kv=None, out_dtype=torch.float16) -> torch.Tensor:
    """Tiled attention of many query rows over sign-bit keys (``metal/_rabitq_prefill.py:116-196``).

    ``q [B,H_q,S_q,D]``; ``scale`` a float (or one-element tensor); ``k_bits [B,H_kv,S,D/8]``;
    ``k_mag`` / ``k_const [B,H_kv,S]`` (``k_const`` may be ``None``); values nibble-packed
    ``u8 [B,H_kv,S,D/2]`` with ``v_cents [<=16]`` (the reference form) or, with ``v_cents=None``,
    a dense f16 / bf16 ``[B,H_kv,S,D]`` tensor. Scores are exact dots with the decoded keys
    ``signs * k_mag`` (not the popcount estimator of :func:`rabitq_fused_attend`). ``causal=True``
    aligns the queries to the tail of the cache (``q_abs = S_kv - S_q + q_pos``).
    """
    fn = "rabitq_prefill_attend"
    if q.ndim != 4:
        raise ValueError(f"{fn}: q must be 4D, got {tuple(q.shape)}")
    B, H, S_q, D = q.shape
    if D % 8 != 0:
        raise ValueError(f"{fn}: D={D} must be divisible by 8")
    if D not in (64, 128):
        raise ValueError(f"{fn}: D={D} must be 64 or 128")
    n_bytes = D // 8
    if k_bits.ndim != 4 or k_bits.shape[0] != B or k_bits.shape[3] != n_bytes or H % k_bits.shape[1] != 0:
        raise ValueError(f"{fn}: k_bits must be [B, H_kv, S_kv, {n_bytes}] with H_kv dividing {H}, got {tuple(k_bits.shape)}")
    H_kv, cap = k_bits.shape[1], k_bits.shape[2]
    S_kv = cap if s_kv is None else int(s_kv)
    if tuple(k_mag.shape) != (B, H_kv, cap):
        raise ValueError(f"{fn}: k_mag must be {(B, H_kv, cap)}, got {tuple(k_mag.shape)}")
    if k_const is not None and tuple(k_const.shape) != (B, H_kv, cap):
        raise ValueError(f"{fn}: k_const must be {(B, H_kv, cap)}, got {tuple(k_const.shape)}")
    if causal and S_q > S_kv:
        raise ValueError(f"{fn}: causal attention of {S_q} query rows over {S_kv} slots")
    if q.dtype not in _FLOAT_DTYPES:
        raise ValueError(f"{fn}: unsupported q dtype {q.dtype}")
    if isinstance(scale, torch.Tensor):
        scale = float(scale.reshape(-1)[0])
    require_cuda(q, f"{fn}: q")
    q = q.contiguous()
    out = torch.empty((B, H, S_q, D), dtype=out_dtype, device=q.device)
    kb = k_bits.to(torch.uint8).contiguous()
    km = k_mag.to(torch.float32).contiguous()
    kc = None if k_const is None else k_const.to(torch.float32).contiguous()
    a = RabitqPrefillArgs(q=q.data_ptr(), out=out.data_ptr(), q_dtype=dtype_code(q.dtype), out_dtype=dtype_code(out_dtype),
                          B=B, H_q=H, H_kv=H_kv, S_q=S_q, S_kv=S_kv, D=D, kv_stride_tok=cap, scale=float(scale),
                          causal=1 if causal else 0, k_bits=kb.data_ptr(), k_mag=km.data_ptr(),
                          k_const=None if kc is None else kc.data_ptr())
    if v_cents is None:
        if tuple(v_idx.shape) != (B, H_kv, cap, D) or v_idx.dtype not in (torch.float16, torch.bfloat16):
            raise ValueError(f"{fn}: dense values must be f16 / bf16 {(B, H_kv, cap, D)}, got {tuple(v_idx.shape)} {v_idx.dtype}")
        v = v_idx.contiguous()
        a.v_mode, a.v, a.v_dtype = 0, v.data_ptr(), dtype_code(v.dtype)
        cents = None
    else:
        if tuple(v_idx.shape) != (B, H_kv, cap, D // 2):
            raise ValueError(f"{fn}: v_idx must be nibble-packed {(B, H_kv, cap, D // 2)} (see rabitq_pack_values), "
                             f"got {tuple(v_idx.shape)}")
        if v_cents.ndim != 1 or v_cents.shape[0] > 16:
            raise ValueError(f"{fn}: v_cents must be 1D with <= 16 entries, got {tuple(v_cents.shape)}")
        v = v_idx.to(torch.uint8).contiguous()
        cents = v_cents.to(device=q.device, dtype=torch.float32).contiguous()
        a.v_mode, a.v, a.v_cents, a.n_cents = 3, v.data_ptr(), cents.data_ptr(), cents.shape[0]
    with _lib.on_device(q.device):
        check(lib().vq_rabitq_prefill_attend(C.byref(a), stream_ptr(q.device)), fn)
    return out


__all__ = ["rabitq_prefill_attend", "make_hadamard_diagonal", "make_rotation_matrix", "rabitq_encode", "rabitq_encode_rotated",
           "rabitq_pack_values", "rabitq_hamming_score", "rabitq_fused_attend"]
