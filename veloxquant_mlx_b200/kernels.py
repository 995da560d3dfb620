"""Kernel wrappers with the reference's names and argument meaning, on ``torch.Tensor``.

Mirrors the reference's ``veloxquant_mlx/metal/kernels.py`` facade for the compressed-KV
hot path. Every function validates like its reference counterpart (same exception types,
function name prefixed in the message) and then calls the C ABI in ``libvqb200.so``;
nothing here computes on the CPU.
"""

from __future__ import annotations

import ctypes as C
import math

import torch

from . import _lib
from ._lib import KiviAttendArgs, KiviDequantArgs, KiviQuantArgs, check, dtype_code, lib, require_cuda, stream_ptr

_FLOAT_DTYPES = (torch.float16, torch.bfloat16, torch.float32)
_MAX_HEADS_PER_KV = 16


def kivi_available() -> bool:
    """True when the native library is built and a CUDA device is visible."""
    import os

    return os.path.exists(_lib.LIB_PATH) and torch.cuda.is_available()


def metal_available() -> bool:
    """The reference's name for the backend probe (``metal/__init__.py:26-31``): here, whether the
    native kernels can run."""
    return kivi_available()


_KNOBS = {"attend_stages": _lib.VQ_KNOB_ATTEND_STAGES, "attend_waves": _lib.VQ_KNOB_ATTEND_WAVES,
          "vq_search": _lib.VQ_KNOB_VQ_SEARCH, "attend_wait_test": _lib.VQ_KNOB_ATTEND_WAIT_TEST,
          "vq_wait_test": _lib.VQ_KNOB_VQ_WAIT_TEST}


def tune(knob: str, value: int) -> int:
    """Set a process-wide tuning / self-test knob of the native library (``vq_tune``) and return
    its previous value. Knobs: ``attend_stages`` (2..4), ``attend_waves`` (1..32), ``vq_search``
    (0 choose, 1 tcgen05, 2 mma.sync, 3 exact, 4 tcgen05 with the two-pass epilogue), and the one-shot self-tests ``attend_wait_test`` / ``vq_wait_test`` that
    make the next launch's bounded device wait run out."""
    if knob not in _KNOBS:
        raise ValueError(f"tune: unknown knob {knob!r}; choices: {sorted(_KNOBS)}")
    prev = lib().vq_tune(_KNOBS[knob], int(value))
    if prev == -(1 << 31):
        raise ValueError(f"tune: value {value} is out of range for {knob!r}")
    return prev


def attend_status() -> None:
    """Synchronise the device and raise :class:`VQLibraryError` (``VQ_ERR_TIMEOUT``) if a decode
    attention or peer-arrival kernel launched since the last check gave up a bounded device-side
    wait; its output is then invalid. The flag is cleared by the check. Poll this where a wrong
    result must not go unnoticed, e.g. once per decode step or per request."""
    check(lib().vq_kivi_attend_status(), "attend_status")


def quantize_status() -> None:
    """The same check for the tensor-memory nearest-centroid search (``vq_vq_quantize_status``)."""
    check(lib().vq_vq_quantize_status(), "quantize_status")


def storage_bits(b: int) -> int:
    """Container width (1, 2, 4 or 8) used to store ``b``-bit codes."""
    if b < 1 or b > 8:
        raise ValueError(f"storage_bits: b={b} must be in 1..8")
    for sb in (1, 2, 4, 8):
        if b <= sb:
            return sb
    raise AssertionError


def _slab_view(x: torch.Tensor, name: str):
    """Return (tensor with contiguous [S, D] rows, n_bh, stride_bh_in_elements).

    Accepts ``[..., S, D]`` tensors whose leading axes collapse to one uniform stride (a
    contiguous tensor, or a slice ``buf[:, :, lo:hi, :]`` of one); anything else is copied.
    """
    S, D = x.shape[-2], x.shape[-1]
    n_bh = 1
    for v in x.shape[:-2]:
        n_bh *= v
    ok = x.stride(-1) == 1 and x.stride(-2) == D
    stride_bh = S * D
    lead = [(x.shape[i], x.stride(i)) for i in range(x.ndim - 2) if x.shape[i] > 1]
    if ok and lead:
        stride_bh = lead[-1][1]
        expect = stride_bh
        for size, st in reversed(lead):
            if st != expect:
                ok = False
                break
            expect = st * size
    if not ok:
        x = x.contiguous()
        stride_bh = S * D
    return x, n_bh, stride_bh


# ----------------------------------------------------------------------------------------
# KIVI quantization
# ----------------------------------------------------------------------------------------

def kivi_append(keys: torch.Tensor, values: torch.Tensor, k_res: torch.Tensor, v_res: torch.Tensor,
                tok_offset: int, overlap_previous: bool = False) -> bool:
    """Copy the block ``keys/values [B,H,S,D]`` behind row ``tok_offset`` of the residual buffers
    ``k_res/v_res [B,H,cap,D]``, both in one launch (the store of the incoming block in the
    reference's ``KIVIKVCache.update_and_fetch``, ``cache/kivi_cache.py:250``). Returns ``False``
    without doing anything when the layout is not one the kernel takes (rows, strides and
    pointers must be multiples of 16 bytes, slabs evenly spaced); the caller then copies with
    torch. ``overlap_previous``: see ``vq_kivi_append`` (the copy may start under the preceding
    work; ``keys`` / ``values`` must not be produced by that work)."""
    B, H, S, D = keys.shape
    es = keys.element_size()
    if keys.dtype not in _FLOAT_DTYPES or not (keys.dtype == values.dtype == k_res.dtype == v_res.dtype):
        return False
    if not (keys.is_cuda and values.is_cuda and k_res.is_cuda and v_res.is_cuda) or S == 0:
        return False
    if tok_offset + S > k_res.shape[2] or k_res.shape != v_res.shape or values.shape != keys.shape:
        return False

    def slabs(t):  # elements between (batch, head) slabs if they are evenly spaced, else None
        if t.stride(3) != 1 or t.stride(2) != D:
            return None
        if t.shape[0] > 1 and t.stride(0) != t.shape[1] * t.stride(1):
            return None
        return t.stride(1) if t.shape[1] > 1 else (t.stride(0) if t.shape[0] > 1 else t.shape[2] * D)

    sn, sv, rk, rv = slabs(keys), slabs(values), slabs(k_res), slabs(v_res)
    if None in (sn, sv, rk, rv) or sn != sv or rk != rv:
        return False
    if (D * es) % 16 or (sn * es) % 16 or (rk * es) % 16:
        return False
    if any(t.data_ptr() % 16 for t in (keys, values, k_res, v_res)):
        return False
    check(lib().vq_kivi_append(keys.data_ptr(), values.data_ptr(), sn, k_res.data_ptr(), v_res.data_ptr(), rk, B * H, S,
                               int(tok_offset), D, dtype_code(keys.dtype),
                               _lib.VQ_ATTEND_OVERLAP_PREVIOUS if overlap_previous else 0, stream_ptr(keys.device)), "kivi_append")
    return True


def kivi_group_quant_dequant(x: torch.Tensor, axis: int, group_size: int, levels: int,
                             eps: float = 1e-8) -> torch.Tensor:
    """Round-trip ``x [..., S, D]`` through KIVI asymmetric group quantization.

    ``axis=-2``: per-channel (keys, groups along tokens); ``axis=-1``: per-token (values,
    groups along channels). Output has ``x``'s shape and dtype and is bit-identical to the
    reference's ``KIVIKVCache._quant_dequant_along`` (``cache/kivi_cache.py:151-201``,
    ``metal/_kivi_quant.py:138-207``).
    """
    if axis not in (-1, -2):
        raise ValueError(f"kivi_group_quant_dequant: axis must be -1 or -2, got {axis}")
    if x.ndim < 2:
        raise ValueError(f"kivi_group_quant_dequant: x must be at least 2D, got {tuple(x.shape)}")
    if group_size < 1:
        raise ValueError(f"kivi_group_quant_dequant: group_size must be >= 1, got {group_size}")
    if levels < 1:
        raise ValueError(f"kivi_group_quant_dequant: levels must be >= 1, got {levels}")
    if x.dtype not in _FLOAT_DTYPES:
        raise ValueError(
            f"kivi_group_quant_dequant: unsupported dtype {x.dtype}; expected one of "
            f"{sorted(str(d) for d in _FLOAT_DTYPES)}"
        )
    if x.numel() == 0:
        return x
    require_cuda(x, "kivi_group_quant_dequant: x")
    xs, n_bh, stride = _slab_view(x, "x")
    S, D = x.shape[-2], x.shape[-1]
    out = torch.empty(x.shape, dtype=x.dtype, device=x.device)
    a = KiviQuantArgs(
        x=xs.data_ptr(), dtype=dtype_code(x.dtype), axis=0 if axis == -2 else 1,
        n_bh=n_bh, n_tok=S, head_dim=D, x_stride_bh=stride,
        levels=int(levels), store_bits=8, group=int(group_size), eps=float(eps),
        codes=None, codes_stride_bh=0, scale=None, zero=None, param_stride_bh=0,
        recon=out.data_ptr(), recon_stride_bh=S * D,
    )
    with _lib.on_device(x.device):
        check(lib().vq_kivi_quant_dequant(C.byref(a), stream_ptr(x.device)), "kivi_group_quant_dequant")
    return out


def kivi_quantize_into(x: torch.Tensor, axis: int, group_size: int, bits: int, *,
                       codes: torch.Tensor, scale: torch.Tensor, zero: torch.Tensor,
                       tok_offset: int = 0, store_bits: int | None = None, eps: float = 1e-8) -> None:
    """Quantize ``x [B,H,S,D]`` and write packed codes / params into cache buffers in place.

    ``codes [B,H,cap,D*sb/8] u8``; keys (``axis=-2``): ``scale,zero [B,H,cap/g,D] f32`` and
    ``tok_offset`` must be a multiple of ``group_size``; values (``axis=-1``):
    ``scale,zero [B,H,cap,ceil(D/g)] f32``. Rows ``[tok_offset, tok_offset+S)`` are written.
    Code-emitting twin of ``KIVIQuantizer._quantize_groups`` (``quantizers/kivi.py:103-128``)
    fused with LSB-first packing (``dsa/bit_pack.py``).
    """
    if axis not in (-1, -2):
        raise ValueError(f"kivi_quantize: axis must be -1 or -2, got {axis}")
    if x.ndim != 4:
        raise ValueError(f"kivi_quantize: x must be 4D [B,H,S,D], got {tuple(x.shape)}")
    if bits < 1 or bits > 8:
        raise ValueError(f"kivi_quantize: bits={bits} must be in [1, 8] (uint8 codes).")
    if group_size < 1:
        raise ValueError(f"kivi_quantize: group_size={group_size} must be >= 1.")
    if x.dtype not in _FLOAT_DTYPES:
        raise ValueError(f"kivi_quantize: unsupported dtype {x.dtype}")
    sb = storage_bits(bits) if store_bits is None else int(store_bits)
    B, H, S, D = x.shape
    if S == 0:
        return
    row_bytes = D * sb // 8
    if codes.dtype != torch.uint8 or codes.shape[-1] != row_bytes or not codes.is_contiguous():
        raise ValueError(f"kivi_quantize: codes must be contiguous uint8 [B,H,cap,{row_bytes}]")
    if scale.dtype != torch.float32 or zero.dtype != torch.float32 or scale.shape != zero.shape:
        raise ValueError("kivi_quantize: scale/zero must be float32 tensors of equal shape")
    if not (scale.is_contiguous() and zero.is_contiguous()):
        raise ValueError("kivi_quantize: scale/zero must be contiguous")
    if codes.ndim != 4 or scale.ndim != 4 or tuple(codes.shape[:2]) != (B, H) or tuple(scale.shape[:2]) != (B, H):
        raise ValueError(f"kivi_quantize: codes and scale/zero must be 4D with leading [B={B}, H={H}] like x, got "
                         f"codes {tuple(codes.shape)}, scale {tuple(scale.shape)}")
    if codes.device != x.device or scale.device != x.device or zero.device != x.device:
        raise ValueError("kivi_quantize: codes, scale and zero must live on x's device")
    cap = codes.shape[2]
    if tok_offset < 0 or tok_offset + S > cap:
        raise RuntimeError(f"kivi_quantize: rows [{tok_offset}, {tok_offset + S}) exceed capacity {cap}")
    require_cuda(x, "kivi_quantize: x")
    xs, n_bh, stride = _slab_view(x, "x")
    if axis == -2:
        if tok_offset % group_size:
            raise ValueError("kivi_quantize: tok_offset must be a multiple of group_size for keys")
        g_off = tok_offset // group_size
        n_g = (S + group_size - 1) // group_size
        if scale.shape[-1] != D or g_off + n_g > scale.shape[2]:
            raise RuntimeError("kivi_quantize: key scale/zero buffer too small")
        p_stride = scale.shape[2] * D
        p_off = g_off * D
    else:
        gv = (D + group_size - 1) // group_size
        if scale.shape[-1] != gv or tok_offset + S > scale.shape[2]:
            raise RuntimeError("kivi_quantize: value scale/zero buffer too small")
        p_stride = scale.shape[2] * gv
        p_off = tok_offset * gv
    a = KiviQuantArgs(
        x=xs.data_ptr(), dtype=dtype_code(x.dtype), axis=0 if axis == -2 else 1,
        n_bh=n_bh, n_tok=S, head_dim=D, x_stride_bh=stride,
        levels=(1 << bits) - 1, store_bits=sb, group=int(group_size), eps=float(eps),
        codes=codes.data_ptr() + tok_offset * row_bytes, codes_stride_bh=cap * row_bytes,
        scale=scale.data_ptr() + 4 * p_off, zero=zero.data_ptr() + 4 * p_off, param_stride_bh=p_stride,
        recon=None, recon_stride_bh=0,
    )
    with _lib.on_device(x.device):
        check(lib().vq_kivi_quantize_pack(C.byref(a), stream_ptr(x.device)), "kivi_quantize")


def kivi_quantize(x: torch.Tensor, axis: int, group_size: int, bits: int, *,
                  store_bits: int | None = None, eps: float = 1e-8):
    """Quantize ``x [B,H,S,D]``; returns ``(packed codes u8, scale f32, zero f32)``.

    Freshly allocated outputs; see :func:`kivi_quantize_into` for layouts. With
    ``store_bits=8`` the codes are one per byte, the reference's own layout.
    """
    if x.ndim != 4:
        raise ValueError(f"kivi_quantize: x must be 4D [B,H,S,D], got {tuple(x.shape)}")
    B, H, S, D = x.shape
    sb = storage_bits(bits) if store_bits is None else int(store_bits)
    codes = torch.empty((B, H, S, D * sb // 8), dtype=torch.uint8, device=x.device)
    if axis == -2:
        pshape = (B, H, (S + group_size - 1) // max(group_size, 1), D)
    else:
        pshape = (B, H, S, (D + group_size - 1) // max(group_size, 1))
    scale = torch.empty(pshape, dtype=torch.float32, device=x.device)
    zero = torch.empty(pshape, dtype=torch.float32, device=x.device)
    kivi_quantize_into(x, axis, group_size, bits, codes=codes, scale=scale, zero=zero,
                       store_bits=sb, eps=eps)
    return codes, scale, zero


def scalar_decode_once(codes: torch.Tensor, scale: torch.Tensor, zero: torch.Tensor,
                       group_size: int, mode: str, *, store_bits: int = 8,
                       out_dtype: torch.dtype = torch.float16) -> torch.Tensor:
    """Decode a group-affine K (``mode="K"``) or V (``"V"``) tensor to ``out_dtype`` once.

    ``codes [B,H_kv,S,D*store_bits/8] u8``. Mirrors ``scalar_decode_once``
    (``metal/_scalar_attend.py:650-699``).
    """
    if mode not in ("K", "V"):
        raise ValueError(f"scalar_decode_once: mode must be 'K' or 'V', got {mode!r}")
    if codes.ndim != 4:
        raise ValueError(f"scalar_decode_once: codes must be 4D, got {tuple(codes.shape)}")
    require_cuda(codes, "scalar_decode_once: codes")
    B, H, S, rb = codes.shape
    D = rb * 8 // store_bits
    codes = codes.contiguous()
    scale = scale.to(torch.float32).contiguous()
    zero = zero.to(torch.float32).contiguous()
    out = torch.empty((B, H, S, D), dtype=out_dtype, device=codes.device)
    if out.numel() == 0:
        return out
    a = KiviDequantArgs(
        codes=codes.data_ptr(), codes_stride_bh=S * rb, scale=scale.data_ptr(), zero=zero.data_ptr(),
        param_stride_bh=scale.shape[2] * scale.shape[3], axis=0 if mode == "K" else 1,
        store_bits=store_bits, group=int(group_size), n_bh=B * H, n_tok=S, head_dim=D,
        out=out.data_ptr(), out_dtype=dtype_code(out_dtype), out_stride_bh=S * D,
    )
    with _lib.on_device(codes.device):
        check(lib().vq_kivi_dequant(C.byref(a), stream_ptr(codes.device)), "scalar_decode_once")
    return out


# ----------------------------------------------------------------------------------------
# KIVI decode attention
# ----------------------------------------------------------------------------------------

_workspaces: dict = {}


def _workspace(device: torch.device, nbytes: int) -> torch.Tensor:
    """Per-(device, stream) scratch buffer, grown geometrically and reused."""
    key = (device.index, stream_ptr(device))
    buf = _workspaces.get(key)
    if buf is None or buf.numel() < nbytes:
        buf = torch.empty(max(nbytes, 1 << 20), dtype=torch.uint8, device=device)
        _workspaces[key] = buf
    return buf


def kivi_decode_attend(q, k_codes, k_scale, k_zero, v_codes, v_scale, v_zero, group_size, scale, *,
                       store_bits=8, n_quant=None, k_res=None, v_res=None, n_res=None,
                       out=None, out_dtype=None, n_splits=0, variant=0, static_scratch=False,
                       overlap_previous=False, gather=None, res_offset=0, causal=False, sinks=None,
                       _plan_batch=None, _keep_args=None, _plain_launch=False, _fn="kivi_decode_attend"):
    """Fused dequant + attention over packed codes and an optional unquantized tail.

    ``k_codes/v_codes [B,H_kv,cap,D*store_bits/8]`` (first ``n_quant`` rows used),
    ``k_scale/k_zero [B,H_kv,capG,D]``, ``v_scale/v_zero [B,H_kv,cap,ceil(D/g)]``,
    ``k_res/v_res [B,H_kv,capR,D]`` float (first ``n_res`` rows used), ``q [B,H_q,S_q,D]``.
    Returns ``[B,H_q,S_q,D]`` in ``out_dtype`` (default: ``q.dtype``).

    ``static_scratch=True`` routes to ``vq_kivi_decode_attend_static``: no workspace is
    taken from torch's allocator, the split partials live in an 8 MiB array inside the
    library. For callers that must not allocate (pass ``out=`` too, so that nothing is
    allocated here either); such calls must not overlap on the GPU.

    ``overlap_previous=True`` (``VQ_ATTEND_OVERLAP_PREVIOUS``) lets the kernel start while the
    preceding work on the stream is still running; only pass it when ``q`` and the packed store
    were complete before that preceding work was launched (true for a decode loop over per-layer
    caches whose queries do not come from the kernel right before; the residual rows may come
    from a ``kivi_append`` issued right before). ``gather`` is a
    ``_lib.PeerGather`` (see ``sharding.PeerExchange``): the output rows are also stored into
    every rank's gathered tensor. ``causal=True`` (several query rows) applies the tail-aligned
    causal mask: row ``r`` sees slots ``<= n_quant + n_res - S_q + r``. ``res_offset`` is the
    first live row of ``k_res/v_res``.
    """
    fn = _fn
    if q.ndim != 4:
        raise ValueError(f"{fn}: q must be 4D, got {tuple(q.shape)}")
    B, H, S_q, D = q.shape
    if D > 256:
        raise ValueError(f"{fn}: D={D} must be <= 256")
    has_q = k_codes is not None
    if has_q:
        if k_codes.ndim != 4 or v_codes.ndim != 4:
            raise ValueError(
                f"{fn}: k_codes and v_codes must be 4D, got k_codes={tuple(k_codes.shape)}, "
                f"v_codes={tuple(v_codes.shape)}"
            )
        Bk, H_kv, cap, rb = k_codes.shape
        Dk = rb * 8 // store_bits
        if Bk != B:
            raise ValueError(f"{fn}: batch mismatch: q B={B} vs k_codes B={Bk}")
        if Dk != D:
            raise ValueError(f"{fn}: head_dim mismatch: q D={D} vs k_codes D={Dk}")
        if v_codes.shape[1] != H_kv:
            raise ValueError(f"{fn}: k_codes H_kv={H_kv} vs v_codes H_kv={v_codes.shape[1]} mismatch")
        if n_quant is None:
            n_quant = cap
        if n_quant > cap or n_quant > v_codes.shape[2]:
            raise ValueError(f"{fn}: n_quant={n_quant} exceeds the code buffers")
        if v_codes.shape[0] != B or v_codes.shape[3] != rb:
            raise ValueError(f"{fn}: v_codes shape={tuple(v_codes.shape)} must have batch {B} and rows of {rb} bytes "
                             "like k_codes")
        g = int(group_size)
        if g < 1:
            raise ValueError(f"{fn}: group_size={group_size} must be >= 1")
        gv = (D + g - 1) // g
        for nm, t in (("k_scale", k_scale), ("k_zero", k_zero), ("v_scale", v_scale), ("v_zero", v_zero)):
            if t is None or t.ndim != 4 or t.dtype != torch.float32 or tuple(t.shape[:2]) != (B, H_kv):
                raise ValueError(f"{fn}: {nm} must be a float32 tensor [B={B}, H_kv={H_kv}, ...], got "
                                 f"{None if t is None else (tuple(t.shape), t.dtype)}")
        if k_scale.shape != k_zero.shape or k_scale.shape[3] != D or k_scale.shape[2] * g < n_quant:
            raise ValueError(f"{fn}: k_scale/k_zero must be equal shapes [B,H_kv,>={-(-n_quant // g)},{D}], got "
                             f"{tuple(k_scale.shape)} / {tuple(k_zero.shape)}")
        if v_scale.shape != v_zero.shape or v_scale.shape[3] != gv or v_scale.shape[2] < n_quant:
            raise ValueError(f"{fn}: v_scale/v_zero must be equal shapes [B,H_kv,>={n_quant},{gv}], got "
                             f"{tuple(v_scale.shape)} / {tuple(v_zero.shape)}")
        for nm, t in (("k_codes", k_codes), ("v_codes", v_codes), ("k_scale", k_scale), ("k_zero", k_zero),
                      ("v_scale", v_scale), ("v_zero", v_zero)):
            if t.device != q.device:
                raise ValueError(f"{fn}: {nm} is on {t.device}, q on {q.device}")
        if k_codes.dtype != torch.uint8 or v_codes.dtype != torch.uint8:
            raise ValueError(f"{fn}: k_codes / v_codes must be uint8")
    else:
        if k_res is None:
            raise ValueError(f"{fn}: no keys given")
        H_kv = k_res.shape[1]
        n_quant = 0
    if H % H_kv != 0:
        raise ValueError(
            f"{fn}: H_q={H} must be a multiple of H_kv={H_kv} (k_codes.shape[1]) for GQA head-packing"
        )
    if H // H_kv > _MAX_HEADS_PER_KV:
        raise ValueError(
            f"{fn}: heads_per_kv={H // H_kv} exceeds the supported maximum of {_MAX_HEADS_PER_KV}"
        )
    if k_res is not None:
        if n_res is None:
            n_res = k_res.shape[2]
        if k_res.shape != v_res.shape or k_res.dtype != v_res.dtype:
            raise ValueError(f"{fn}: k_res and v_res must match in shape and dtype")
        if not (k_res.is_contiguous() and v_res.is_contiguous()):
            raise ValueError(f"{fn}: k_res / v_res must be contiguous")
        if res_offset < 0 or res_offset + n_res > k_res.shape[2]:
            raise ValueError(f"{fn}: rows [{res_offset}, {res_offset + n_res}) exceed the residual buffers "
                             f"({k_res.shape[2]} rows)")
        if k_res.ndim != 4 or tuple(k_res.shape[:2]) != (B, H_kv) or k_res.shape[3] != D or k_res.device != q.device:
            raise ValueError(f"{fn}: k_res / v_res must be [B={B}, H_kv={H_kv}, rows, D={D}] on q's device, got "
                             f"{tuple(k_res.shape)} on {k_res.device}")
        if k_res.dtype not in _FLOAT_DTYPES:
            raise ValueError(f"{fn}: unsupported residual dtype {k_res.dtype}")
    else:
        n_res = 0
    if q.dtype not in _FLOAT_DTYPES:
        raise ValueError(f"{fn}: unsupported q dtype {q.dtype}")
    q = q.contiguous()
    out_dtype = out_dtype or q.dtype
    if out is None:
        out = torch.empty((B, H, S_q, D), dtype=out_dtype, device=q.device)
    else:
        # a caller-owned output is written through its raw pointer: a wrong shape would be an
        # out-of-bounds device write
        if tuple(out.shape) != (B, H, S_q, D) or not out.is_contiguous() or out.device != q.device:
            raise ValueError(f"{fn}: out must be a contiguous [{B}, {H}, {S_q}, {D}] tensor on {q.device}, got "
                             f"{tuple(out.shape)} (contiguous={out.is_contiguous()}) on {out.device}")
        if out.dtype not in _FLOAT_DTYPES:
            raise ValueError(f"{fn}: unsupported out dtype {out.dtype}")
    if gather is not None and not isinstance(gather, _lib.PeerGather):
        raise ValueError(f"{fn}: gather must be a PeerGather structure (sharding.PeerExchange.layer)")
    sink_struct = None
    if sinks is not None:
        # (exact keys, exact values, dequantized keys of the slots left behind, rows in use per batch element)
        sk, sv, sd, cnt = sinks
        for t, nm in ((sk, "sinks[0]"), (sv, "sinks[1]"), (sd, "sinks[2]")):
            if t.ndim != 4 or t.shape[0] != B or t.shape[1] != H_kv or t.shape[3] != D or not t.is_contiguous() or t.shape != sk.shape:
                raise ValueError(f"{fn}: {nm} must be a contiguous [{B}, {H_kv}, rows, {D}] tensor, got {tuple(t.shape)}")
            if t.device != q.device:
                raise ValueError(f"{fn}: {nm} must be on {q.device}")
        if sv.dtype != sk.dtype or sd.dtype != torch.float32:
            raise ValueError(f"{fn}: sinks[0] and sinks[1] must share one dtype and sinks[2] must be float32, got "
                             f"{sk.dtype}, {sv.dtype}, {sd.dtype}")
        if k_res is not None and sk.dtype != k_res.dtype:
            raise ValueError(f"{fn}: sink rows must have the residual's dtype {k_res.dtype}, got {sk.dtype}")
        if sk.dtype not in _FLOAT_DTYPES:
            raise ValueError(f"{fn}: unsupported sink row dtype {sk.dtype}")
        if cnt.dtype != torch.int32 or tuple(cnt.shape) != (B,) or cnt.device != q.device or not cnt.is_contiguous():
            raise ValueError(f"{fn}: sinks[3] must be an int32 [{B}] tensor on {q.device}, got {cnt.dtype} {tuple(cnt.shape)}")
        if not has_q or S_q != 1:
            raise ValueError(f"{fn}: protected tokens need a packed store and one query row")
        sink_struct = _lib.KiviSinks(k=sk.data_ptr(), v=sv.data_ptr(), k_dead=sd.data_ptr(), count=cnt.data_ptr(),
                                     stride_bh=sk.shape[2] * D, max_rows=sk.shape[2])
    require_cuda(q, f"{fn}: q")  # (after the shape checks, so that those can be exercised without a GPU)
    a = KiviAttendArgs(
        q=q.data_ptr(), out=out.data_ptr(), q_dtype=dtype_code(q.dtype), out_dtype=dtype_code(out.dtype),
        B=B, H_q=H, H_kv=H_kv, S_q=S_q, D=D, store_bits=int(store_bits), group=int(group_size),
        n_quant=int(n_quant), n_res=int(n_res), scale=float(scale),
        n_splits=int(n_splits), variant=int(variant),
        flags=(_lib.VQ_ATTEND_OVERLAP_PREVIOUS if overlap_previous else 0) | (_lib.VQ_ATTEND_CAUSAL if causal else 0),
        gather=C.addressof(gather) if gather is not None else None,
        sinks=C.addressof(sink_struct) if sink_struct is not None else None,
    )
    if sink_struct is not None:
        a.res_dtype = dtype_code(sinks[0].dtype)
        a._sink_struct = sink_struct  # (keeps the structure alive as long as the arguments)
    if has_q:
        for t, nm in ((k_codes, "k_codes"), (v_codes, "v_codes"), (k_scale, "k_scale"), (k_zero, "k_zero"),
                      (v_scale, "v_scale"), (v_zero, "v_zero")):
            if not t.is_contiguous():
                raise ValueError(f"{fn}: {nm} must be contiguous")
        a.k_codes, a.k_codes_stride_bh = k_codes.data_ptr(), k_codes.shape[2] * k_codes.shape[3]
        a.v_codes, a.v_codes_stride_bh = v_codes.data_ptr(), v_codes.shape[2] * v_codes.shape[3]
        a.k_scale, a.k_zero = k_scale.data_ptr(), k_zero.data_ptr()
        a.k_param_stride_bh = k_scale.shape[2] * k_scale.shape[3]
        a.v_scale, a.v_zero = v_scale.data_ptr(), v_zero.data_ptr()
        a.v_param_stride_bh = v_scale.shape[2] * v_scale.shape[3]
    if n_res:
        row_bytes = D * k_res.element_size()
        a.k_res, a.v_res = k_res.data_ptr() + res_offset * row_bytes, v_res.data_ptr() + res_offset * row_bytes
        a.res_dtype = dtype_code(k_res.dtype)
        a.res_stride_bh = k_res.shape[2] * k_res.shape[3]
    with _lib.on_device(q.device):
        if _plain_launch and a.flags & _lib.VQ_ATTEND_OVERLAP_PREVIOUS and not n_splits:
            # the split plan (= summation order) of an overlapped call, launched plainly: for a call
            # whose packed store was written by the kernels right before it
            a.n_splits = int(lib().vq_kivi_attend_splits(C.byref(a)))
            a.flags &= ~_lib.VQ_ATTEND_OVERLAP_PREVIOUS
        if _plan_batch is not None and not n_splits:
            # layers folded into the batch axis: take the split count of one layer's shape
            a.B = int(_plan_batch)
            a.n_splits = int(lib().vq_kivi_attend_splits(C.byref(a)))
            a.B = B
        if static_scratch:
            check(lib().vq_kivi_decode_attend_static(C.byref(a), stream_ptr(q.device)), fn)
            return out
        need = lib().vq_kivi_attend_workspace_bytes(C.byref(a))
        ws = _workspace(q.device, need)
        a.workspace, a.workspace_bytes = ws.data_ptr(), ws.numel()
        entry = lib().vq_kivi_decode_attend if has_q else lib().vq_predecoded_attend
        check(entry(C.byref(a), stream_ptr(q.device)), fn)
    if _keep_args is not None and has_q:
        _keep_args.append(a)  # (for a caller that repeats the call with the same buffers)
    return out


def scalar_fused_decode_attend(q, k_codes, k_scale, k_zero, v_codes, v_scale, v_zero,
                               group_size: int, scale: float, nsg: int | None = None, *,
                               store_bits: int = 8) -> torch.Tensor:
    """Reference-shaped entry: one code per byte by default, fp16 output.

    Same arguments as ``scalar_fused_decode_attend`` (``metal/_scalar_attend.py:370-493``);
    ``nsg`` (1..32) pins the number of context splits. Codes are ``uint8 [B,H_kv,S_kv,D]``
    (or packed rows with ``store_bits`` < 8).
    """
    fn = "scalar_fused_decode_attend"
    if nsg is not None and not (1 <= nsg <= 32):
        raise ValueError(f"{fn}: nsg={nsg} must be in 1..32")
    return kivi_decode_attend(
        q, k_codes.to(torch.uint8), k_scale.to(torch.float32), k_zero.to(torch.float32),
        v_codes.to(torch.uint8), v_scale.to(torch.float32), v_zero.to(torch.float32),
        group_size, scale, store_bits=store_bits, out_dtype=torch.float16,
        n_splits=0 if nsg is None else nsg, _fn=fn,
    )


def scalar_fused_decode_attend_batched(q, k_codes, k_scale, k_zero, v_codes, v_scale, v_zero,
                                       group_size: int, scale: float, nsg: int | None = None, *,
                                       store_bits: int = 8) -> torch.Tensor:
    """Every layer of a decode step in one launch: all inputs carry a leading ``NL`` axis
    (``q [NL,B,H_q,S_q,D]``, codes ``[NL,B,H_kv,S_kv,D*store_bits/8]``, ...); uniform ``S_kv``.

    Mirrors ``scalar_fused_decode_attend_batched`` (``metal/_scalar_attend.py:496-647``). The
    layer axis is folded into the batch axis of the same kernel (layers are just more
    independent (batch, kv head) units), so stacked contiguous inputs cost no copy. The context
    split count is the one a single layer's call would use, so each layer's result is bit-identical
    to the per-layer call, as the reference pins it (``tests/metal/test_scalar_attend.py:660-707``).
    """
    fn = "scalar_fused_decode_attend_batched"
    if q.ndim != 5:
        raise ValueError(f"{fn}: q must be 5D [NL,B,H,S_q,D], got {tuple(q.shape)}")
    if k_codes.ndim != 5 or v_codes.ndim != 5:
        raise ValueError(f"{fn}: k_codes and v_codes must be 5D, got k_codes={tuple(k_codes.shape)}, "
                         f"v_codes={tuple(v_codes.shape)}")
    NL, B, H, S_q, D = q.shape
    if NL < 1:
        raise ValueError(f"{fn}: NL={NL} must be >= 1")
    if D > 256:
        raise ValueError(f"{fn}: D={D} must be <= 256")
    if nsg is not None and not (1 <= nsg <= 32):
        raise ValueError(f"{fn}: nsg={nsg} must be in 1..32")
    if k_codes.shape[0] != NL:
        raise ValueError(f"{fn}: NL mismatch: q NL={NL} vs k_codes NL={k_codes.shape[0]}")
    if k_codes.shape[1] != B:
        raise ValueError(f"{fn}: batch mismatch: q B={B} vs k_codes B={k_codes.shape[1]}")
    if v_codes.shape != k_codes.shape:
        raise ValueError(f"{fn}: k_codes shape={tuple(k_codes.shape)} vs v_codes shape={tuple(v_codes.shape)} mismatch")
    H_kv = k_codes.shape[2]
    for name, arr in (("k_scale", k_scale), ("k_zero", k_zero), ("v_scale", v_scale), ("v_zero", v_zero)):
        if arr.ndim != 5 or arr.shape[0] != NL or arr.shape[1] != B or arr.shape[2] != H_kv:
            raise ValueError(f"{fn}: {name} shape={tuple(arr.shape)} must be 5D with leading "
                             f"[NL={NL}, B={B}, H_kv={H_kv}, ...]")
    if H % H_kv != 0:
        raise ValueError(f"{fn}: H_q={H} must be a multiple of H_kv={H_kv} (k_codes.shape[2]) for GQA head-packing")

    def fold(t):
        return t.reshape(NL * B, *t.shape[2:])

    out = kivi_decode_attend(
        fold(q), fold(k_codes.to(torch.uint8)), fold(k_scale.to(torch.float32)), fold(k_zero.to(torch.float32)),
        fold(v_codes.to(torch.uint8)), fold(v_scale.to(torch.float32)), fold(v_zero.to(torch.float32)),
        group_size, scale, store_bits=store_bits, out_dtype=torch.float16,
        n_splits=0 if nsg is None else nsg, _plan_batch=B, _fn=fn,
    )
    return out.reshape(NL, B, H, S_q, D)


def lse_merge(part_o: torch.Tensor, part_ml: torch.Tensor, out_dtype=torch.float16) -> torch.Tensor:
    """Combine split softmax partials ``part_o f32 [rows, n_splits, D]`` (unnormalised,
    relative to each split's own maximum) and ``part_ml f32 [rows, n_splits, 2]`` (max, sum)
    into ``[rows, D]``. No counterpart in the reference (its kernels merge internally)."""
    fn = "lse_merge"
    if part_o.ndim != 3 or part_ml.ndim != 3 or part_ml.shape != (part_o.shape[0], part_o.shape[1], 2):
        raise ValueError(f"{fn}: part_o [rows,n_splits,D] and part_ml [rows,n_splits,2] expected, got "
                         f"{tuple(part_o.shape)} / {tuple(part_ml.shape)}")
    require_cuda(part_o, f"{fn}: part_o")
    if part_o.dtype != torch.float32 or part_ml.dtype != torch.float32:
        raise ValueError(f"{fn}: partials must be float32")
    rows, n_splits, D = part_o.shape
    po, pm = part_o.contiguous(), part_ml.contiguous()
    out = torch.empty((rows, D), dtype=out_dtype, device=part_o.device)
    with _lib.on_device(part_o.device):
        check(lib().vq_lse_merge(po.data_ptr(), pm.data_ptr(), rows, n_splits, D, out.data_ptr(),
                                 dtype_code(out_dtype), stream_ptr(part_o.device)), fn)
    return out


def scalar_predecoded_attend(q, k_hat, v_hat, scale: float, nsg: int | None = None) -> torch.Tensor:
    """Attention over already-decoded ``k_hat/v_hat [B,H_kv,S,D]``; fp16 output.

    Mirrors ``scalar_predecoded_attend`` (``metal/_scalar_attend.py:702-779``).
    """
    fn = "scalar_predecoded_attend"
    if q.ndim != 4:
        raise ValueError(f"{fn}: q must be 4D, got {tuple(q.shape)}")
    if k_hat.ndim != 4 or v_hat.ndim != 4:
        raise ValueError(f"{fn}: k_hat and v_hat must be 4D, got k_hat={tuple(k_hat.shape)}, v_hat={tuple(v_hat.shape)}")
    if nsg is not None and not (1 <= nsg <= 32):
        raise ValueError(f"{fn}: nsg={nsg} must be in 1..32")
    if k_hat.shape[0] != q.shape[0]:
        raise ValueError(f"{fn}: batch mismatch: q B={q.shape[0]} vs k_hat B={k_hat.shape[0]}")
    if k_hat.shape[3] != q.shape[3]:
        raise ValueError(f"{fn}: head_dim mismatch: q D={q.shape[3]} vs k_hat D={k_hat.shape[3]}")
    if v_hat.shape != k_hat.shape:
        raise ValueError(f"{fn}: k_hat shape={tuple(k_hat.shape)} vs v_hat shape={tuple(v_hat.shape)} mismatch")
    return kivi_decode_attend(
        q, None, None, None, None, None, None, 1, scale,
        k_res=k_hat.contiguous(), v_res=v_hat.contiguous().to(k_hat.dtype),
        out_dtype=torch.float16, n_splits=0 if nsg is None else nsg, _fn=fn,
    )


# ----------------------------------------------------------------------------------------
# Bit packing
# ----------------------------------------------------------------------------------------

def turboquant_bit_pack(indices: torch.Tensor, b: int) -> torch.Tensor:
    """Pack uint8 indices (values < 2**b) LSB first; ``b`` in {1, 2, 4}.

    Mirrors ``turboquant_bit_pack`` (``metal/_bit_packing.py:87-116``).
    """
    if b not in (1, 2, 4):
        raise ValueError(f"turboquant_bit_pack: b must be 1, 2, or 4, got {b}")
    N = indices.numel()
    per = 8 // b
    if N % per != 0:
        raise ValueError(f"turboquant_bit_pack: N={N} not divisible by {per} (= 8/b)")
    require_cuda(indices, "turboquant_bit_pack: indices")
    flat = indices.reshape(-1).to(torch.uint8).contiguous()
    out = torch.empty(N * b // 8, dtype=torch.uint8, device=indices.device)
    with _lib.on_device(indices.device):
        check(lib().vq_bit_pack(flat.data_ptr(), N, b, out.data_ptr(), stream_ptr(indices.device)),
              "turboquant_bit_pack")
    return out


def turboquant_bit_unpack(packed: torch.Tensor, N: int, b: int) -> torch.Tensor:
    """Inverse of :func:`turboquant_bit_pack` (``metal/_bit_packing.py:119-148``)."""
    if b not in (1, 2, 4):
        raise ValueError(f"turboquant_bit_unpack: b must be 1, 2, or 4, got {b}")
    if N < 0:
        raise ValueError(f"turboquant_bit_unpack: N must be >= 0, got {N}")
    need = -(-N * b // 8)
    if packed.numel() < need:
        raise ValueError(
            f"turboquant_bit_unpack: packed has {packed.numel()} byte(s) but N={N} at b={b} needs {need}"
        )
    require_cuda(packed, "turboquant_bit_unpack: packed")
    flat = packed.reshape(-1).to(torch.uint8).contiguous()
    out = torch.empty(N, dtype=torch.uint8, device=packed.device)
    with _lib.on_device(packed.device):
        check(lib().vq_bit_unpack(flat.data_ptr(), N, b, out.data_ptr(), stream_ptr(packed.device)),
              "turboquant_bit_unpack")
    return out


# The reference gathers every kernel wrapper in one module (``metal/kernels.py:19-146``), so that
# ``from ...kernels import rvq_quant_pack`` works whatever file defines it. The wrappers of the other
# code families live in their own modules here (which import this one), and are resolved on first use.
_DEFINED_ELSEWHERE = {
    "rabitq_encode": "rabitq", "rabitq_fused_attend": "rabitq", "rabitq_hamming_score": "rabitq",
    "rabitq_pack_values": "rabitq", "rabitq_prefill_attend": "rabitq",
    "rvq_quant_pack": "rvq", "rvq_unpack_decode": "rvq",
    "vecinfer_quantize_metal": "vecinfer", "vecinfer_dequant_metal": "vecinfer",
    "vecinfer_encode_decode_metal": "vecinfer", "vecinfer_encode_decode_simple_metal": "vecinfer",
    "metal_fused_sdpa": "vecinfer",
}


def __getattr__(name: str):
    module = _DEFINED_ELSEWHERE.get(name)
    if module is None:
        raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
    import importlib

    return getattr(importlib.import_module("." + module, __package__), name)


__all__ = [
    "kivi_available", "metal_available", "tune", "attend_status", "quantize_status", "storage_bits", "kivi_group_quant_dequant", "kivi_quantize", "kivi_quantize_into",
    "scalar_decode_once", "kivi_decode_attend", "scalar_fused_decode_attend", "scalar_predecoded_attend",
    "scalar_fused_decode_attend_batched", "lse_merge",
    "turboquant_bit_pack", "turboquant_bit_unpack", *_DEFINED_ELSEWHERE,
]
