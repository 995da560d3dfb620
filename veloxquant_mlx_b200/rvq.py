"""TurboQuant-RVQ: two-stage scalar residual quantization of rotated keys, bit-packed.

Mirrors the reference's packed RVQ path: ``rvq_quant_pack`` (``metal/_rvq_quant_pack.py:83-149``),
``rvq_unpack_decode`` (``metal/_rvq_unpack_decode.py:78-183``), ``_pack_indices`` /
``_unpack_indices`` (``cache/turboquant_rvq_cache.py:82-126``), ``ScalarCodebook``
(``codebooks/scalar_codebook.py``), the Lloyd-Max codebooks (``math/lloyd_max.py``,
``codebooks/strategies.py:26-56``) and the quantizer ``TurboQuantRVQ``
(``quantizers/turboquant_rvq.py``): stage 1 quantizes each rotated coordinate against an
``N(0, 1/d)`` Lloyd-Max codebook, stage 2 quantizes the fp16 residual against a Laplacian-fit
one; both code streams are stored as uint32 words. The two kernels run on the device
(``csrc/rvq.cu``); the codebooks are a handful of numbers computed once on the host.
"""

from __future__ import annotations

import ctypes as C
import math
from functools import lru_cache

import numpy as np
import torch

from . import _lib
from ._lib import check, dtype_code, lib, require_cuda, stream_ptr
from .rabitq import make_hadamard_diagonal, make_rotation_matrix

_WORD_BITS = 32
LLOYD_MAX_N_ITER, LLOYD_MAX_TOL, LLOYD_MAX_N_QUAD = 5000, 1e-9, 10_000


# ----------------------------------------------------------------------------------------
# Lloyd-Max codebooks (host)
# ----------------------------------------------------------------------------------------
def lloyd_max(pdf_fn, support, n_levels: int, n_iter: int = LLOYD_MAX_N_ITER, tol: float = LLOYD_MAX_TOL,
              n_quad_points: int = LLOYD_MAX_N_QUAD):
    """MSE-optimal scalar quantizer of a density on ``support`` (``math/lloyd_max.py:19-127``).

    The density is tabulated on a uniform grid; the running trapezoid integrals of ``f`` and
    ``x f`` are interpolated at the cell edges (midpoints of neighbouring centroids), so that a
    cell's mass and first moment include the partial grid intervals at its edges. Centroids
    start at the equal-mass quantiles and move to their cells' means until the largest shift is
    below ``tol``. Returns ``(centroids, boundaries)`` in float64, boundaries with infinite ends.
    """
    lo, hi = float(support[0]), float(support[1])
    if lo >= hi:
        raise ValueError(f"lloyd_max: support must have lo < hi, got ({lo}, {hi})")
    if n_levels < 1:
        raise ValueError(f"lloyd_max: n_levels must be >= 1, got {n_levels}")
    x = np.linspace(lo, hi, n_quad_points)
    p = pdf_fn(x)
    step = np.diff(x)

    def running(y):
        return np.concatenate([[0.0], np.cumsum((y[1:] + y[:-1]) / 2.0 * step)])

    mass_to, moment_to = running(p), running(x * p)
    if mass_to[-1] > 0.0:
        cents = np.interp((np.arange(n_levels) + 0.5) / n_levels * mass_to[-1], mass_to, x)
    else:
        cents = np.linspace(lo, hi, n_levels)
    for _ in range(n_iter):
        edges = np.concatenate([[lo], np.clip((cents[:-1] + cents[1:]) / 2.0, lo, hi), [hi]])
        mass = np.diff(np.interp(edges, x, mass_to))
        moment = np.diff(np.interp(edges, x, moment_to))
        ok = mass >= 1e-12
        new = np.where(ok, moment / np.where(ok, mass, 1.0), cents)
        shift = np.max(np.abs(new - cents))
        cents = new
        if shift < tol:
            break
    bounds = np.concatenate([[-np.inf], (cents[:-1] + cents[1:]) / 2.0, [np.inf]])
    return cents.astype(np.float64), bounds.astype(np.float64)


def _gaussian_pdf(sigma: float):
    coeff = 1.0 / (sigma * math.sqrt(2.0 * math.pi))
    return lambda x: coeff * np.exp(-0.5 * (np.asarray(x, dtype=np.float64) / sigma) ** 2)


def _laplacian_pdf(scale: float):
    return lambda x: (1.0 / (2.0 * scale)) * np.exp(-np.abs(x) * (1.0 / scale))


def _beta_pdf(d: int):
    """Density of one coordinate of a uniform point on the unit sphere in ``d`` dimensions
    (``math/distributions.py:19-47``)."""
    log_norm = math.lgamma(d / 2.0) - 0.5 * math.log(math.pi) - math.lgamma((d - 1) / 2.0)
    alpha = (d - 3) / 2.0

    def pdf(x):
        x = np.asarray(x, dtype=np.float64)
        out = np.zeros_like(x)
        m = (x > -1.0) & (x < 1.0)
        out[m] = np.exp(log_norm + alpha * np.log1p(-(x[m] ** 2)))
        return out

    return pdf


class ScalarCodebook:
    """Sorted scalar centroids with their Voronoi boundaries, held as the reference holds them
    (``codebooks/scalar_codebook.py:37-60``): centroids float32 -> float16, boundaries the float32
    midpoints rounded to float16. ``quantize`` counts the boundaries below a value."""

    def __init__(self, centroids) -> None:
        c = np.sort(np.asarray(centroids, dtype=np.float32))
        if c.ndim != 1 or len(c) & (len(c) - 1) or len(c) < 2:
            raise ValueError(f"ScalarCodebook: the number of centroids must be a power of 2 >= 2, got shape {c.shape}")
        self.k, self.b = len(c), int(math.log2(len(c)))
        self.centroids32 = c
        self.centroids = c.astype(np.float16)
        self.boundaries = ((c[:-1] + c[1:]) / np.float32(2.0)).astype(np.float16)
        self._dev: dict = {}

    def _on(self, device):
        t = self._dev.get(str(device))
        if t is None:
            t = (torch.from_numpy(self.centroids).to(device), torch.from_numpy(self.boundaries).to(device))
            self._dev[str(device)] = t
        return t

    def quantize(self, y: torch.Tensor) -> torch.Tensor:
        """``#{k : y > boundary_k}`` as uint8 (``scalar_codebook.py:77-95``)."""
        _, bounds = self._on(y.device)
        return torch.searchsorted(bounds.to(y.dtype), y.contiguous(), right=False).to(torch.uint8)

    def dequantize(self, idx: torch.Tensor) -> torch.Tensor:
        cents, _ = self._on(idx.device)
        return cents[idx.long()]


@lru_cache(maxsize=None)
def gaussian_codebook(b: int, d: int) -> ScalarCodebook:
    """Stage-1 codebook: Lloyd-Max for ``N(0, 1/d)`` on +-6 sigma (``codebooks/strategies.py:38-56``)."""
    if not 1 <= b <= 8 or d < 1:
        raise ValueError(f"gaussian_codebook: b={b} must be in 1..8 and d={d} >= 1")
    sigma = 1.0 / math.sqrt(d)
    cents, _ = lloyd_max(_gaussian_pdf(sigma), (-6.0 * sigma, 6.0 * sigma), 2 ** b)
    return ScalarCodebook(cents.astype(np.float32))


@lru_cache(maxsize=None)
def beta_codebook(b: int, d: int) -> ScalarCodebook:
    """Stage-1 codebook for small ``d`` (< 64): the exact coordinate density on (-1, 1)
    (``codebooks/strategies.py:63-94``)."""
    cents, _ = lloyd_max(_beta_pdf(d), (-1.0 + 1e-6, 1.0 - 1e-6), 2 ** b)
    return ScalarCodebook(cents.astype(np.float32))


@lru_cache(maxsize=None)
def laplacian_codebook(b: int, residual_scale: float) -> ScalarCodebook:
    """Stage-2 codebook: Lloyd-Max for a zero-mean Laplacian on +-8 scales
    (``quantizers/turboquant_rvq.py:52-72``)."""
    hi = 8.0 * residual_scale
    cents, _ = lloyd_max(_laplacian_pdf(residual_scale), (-hi, hi), 2 ** b)
    return ScalarCodebook(cents.astype(np.float32))


# ----------------------------------------------------------------------------------------
# packing (torch) and the two kernels
# ----------------------------------------------------------------------------------------
def n_words_for(d: int, bits: int) -> int:
    return -(-d // (_WORD_BITS // bits))


def pack_indices(idx: torch.Tensor, bits: int) -> torch.Tensor:
    """Codes ``[..., d]`` -> uint32 words ``[..., ceil(d / (32 // bits))]`` (held as int32 bit
    patterns), code i of a word in bits ``[i*bits, (i+1)*bits)`` (``turboquant_rvq_cache.py:82-106``)."""
    epw = _WORD_BITS // bits
    d = idx.shape[-1]
    pad = (-d) % epw
    x = idx.to(torch.int64)
    if pad:
        x = torch.nn.functional.pad(x, (0, pad))
    x = x.reshape(*idx.shape[:-1], -1, epw)
    shifts = torch.arange(epw, device=idx.device, dtype=torch.int64) * bits
    words = (x << shifts).sum(dim=-1)
    return (words & 0xFFFFFFFF).to(torch.uint32)


def unpack_indices(packed: torch.Tensor, bits: int, d: int) -> torch.Tensor:
    """Inverse of :func:`pack_indices` (``turboquant_rvq_cache.py:109-126``): uint8 ``[..., d]``."""
    epw = _WORD_BITS // bits
    w = packed.view(torch.int32).to(torch.int64) & 0xFFFFFFFF
    shifts = torch.arange(epw, device=packed.device, dtype=torch.int64) * bits
    codes = (w[..., None] >> shifts) & ((1 << bits) - 1)
    return codes.reshape(*packed.shape[:-1], -1)[..., :d].to(torch.uint8)


def _count(t) -> int:
    return int(t.numel()) if isinstance(t, torch.Tensor) else int(np.asarray(t).size)


def _host_f32(t, n: int, name: str, who: str):
    a = t.detach().float().cpu().numpy() if isinstance(t, torch.Tensor) else np.asarray(t, dtype=np.float32)
    a = np.ascontiguousarray(a.reshape(-1), dtype=np.float32)
    if a.size != n:
        raise ValueError(f"{who}: expected {n} {name}, got {a.size}")
    return a


_TABLES: dict = {}


def rvq_code_table(centroids1, boundaries1, boundaries2, bits: int, device) -> torch.Tensor:
    """The two-stage quantizer as a table over all float16 bit patterns: ``uint8 [65536]`` with
    ``idx1 | idx2 << 4`` (both codes depend on the coordinate's 16 bits only). Built on the device
    once per (codebooks, device) and kept."""
    who = "rvq_code_table"
    c1 = _host_f32(centroids1, 1 << bits, "stage-1 centroids", who)
    b1 = _host_f32(boundaries1, (1 << bits) - 1, "stage-1 boundaries", who)
    b2 = _host_f32(boundaries2, (1 << bits) - 1, "stage-2 boundaries", who)
    device = torch.device(device)
    key = (c1.tobytes(), b1.tobytes(), b2.tobytes(), bits, str(device))
    t = _TABLES.get(key)
    if t is None:
        t = torch.empty(65536, dtype=torch.uint8, device=device)
        require_cuda(t, f"{who}: device")
        with _lib.on_device(device):
            check(lib().vq_rvq_build_table(c1.ctypes.data_as(C.c_void_p), b1.ctypes.data_as(C.c_void_p),
                                           b2.ctypes.data_as(C.c_void_p), bits, t.data_ptr(), stream_ptr(device)), who)
        if len(_TABLES) > 64:
            _TABLES.clear()
        _TABLES[key] = t
    return t


def rvq_quant_pack(rotated: torch.Tensor, centroids1, boundaries1, boundaries2, bits: int, *, use_table: bool | None = None):
    """Stage-1 + stage-2 quantize of rotated fp16 vectors, packed (``metal/_rvq_quant_pack.py:83-149``).

    ``rotated [N, D]`` float16; ``centroids1 [2**bits]``, ``boundaries1/2 [2**bits - 1]`` sorted
    (host arrays or tensors). Returns ``(packed1, packed2)``, each uint32 ``[N, ceil(D/(32//bits))]``,
    bit-identical to packing ``ScalarCodebook.quantize`` of both stages. ``use_table``: go through
    the 64 KiB code table (default: for inputs of at least 65 536 words)."""
    who = "rvq_quant_pack"
    if rotated.ndim != 2:
        raise ValueError(f"{who}: rotated must be 2D [N, D], got {tuple(rotated.shape)}")
    if not 1 <= bits <= 4:
        raise ValueError(f"{who}: bits must be 1-4, got {bits}")
    N, D = rotated.shape
    if D > 1024:
        raise ValueError(f"{who}: D={D} exceeds the 1024 limit")
    if rotated.dtype != torch.float16:
        raise ValueError(f"{who}: rotated must be float16, got {rotated.dtype}")
    n_levels = 1 << bits
    if _count(centroids1) != n_levels:
        raise ValueError(f"{who}: expected {n_levels} stage-1 centroids for bits={bits}, got {_count(centroids1)}")
    if _count(boundaries1) != n_levels - 1 or _count(boundaries2) != n_levels - 1:
        raise ValueError(f"{who}: expected {n_levels - 1} boundaries per stage for bits={bits}, "
                         f"got {_count(boundaries1)} (stage 1), {_count(boundaries2)} (stage 2)")
    c1 = _host_f32(centroids1, n_levels, "stage-1 centroids", who)
    b1 = _host_f32(boundaries1, n_levels - 1, "stage-1 boundaries", who)
    b2 = _host_f32(boundaries2, n_levels - 1, "stage-2 boundaries", who)
    require_cuda(rotated, f"{who}: rotated")
    y = rotated.contiguous()
    nw = n_words_for(D, bits)
    if use_table is None:
        use_table = N * nw >= 65536
    table = rvq_code_table(c1, b1, b2, bits, y.device) if use_table else None
    p1 = torch.empty((N, nw), dtype=torch.uint32, device=y.device)
    p2 = torch.empty((N, nw), dtype=torch.uint32, device=y.device)
    with _lib.on_device(y.device):
        check(lib().vq_rvq_quant_pack(y.data_ptr(), N, D, c1.ctypes.data_as(C.c_void_p), b1.ctypes.data_as(C.c_void_p),
                                      b2.ctypes.data_as(C.c_void_p), table.data_ptr() if table is not None else None, bits,
                                      p1.data_ptr(), p2.data_ptr(), stream_ptr(y.device)), who)
    return p1, p2


def rvq_unpack_decode(packed1: torch.Tensor, packed2: torch.Tensor, norms: torch.Tensor, centroids1, centroids2, diag,
                      bits: int, d: int, seq_len: int | None = None) -> torch.Tensor:
    """Packed RVQ keys -> fp16 vectors in one launch (``metal/_rvq_unpack_decode.py:78-183``):
    unpack, ``half(c1 + c2)``, inverse randomized Hadamard, norm rescale with fp16 saturation.
    ``packed1/2 [N, n_words]`` or a cache buffer ``[BH, cap, n_words]`` read in place with
    ``seq_len`` live rows per ``BH``; returns ``[N, d]`` (``N = BH * seq_len``) float16."""
    who = "rvq_unpack_decode"
    if d <= 0 or d & (d - 1):
        raise ValueError(f"{who}: d={d} must be a power of two")
    if d > 1024:
        raise ValueError(f"{who}: d={d} exceeds the 1024 limit")
    if not 1 <= bits <= 4:
        raise ValueError(f"{who}: bits must be 1-4, got {bits}")
    nw = n_words_for(d, bits)
    if packed1.ndim == 2 and packed2.ndim == 2:
        if seq_len is not None:
            raise ValueError(f"{who}: seq_len requires 3D [BH, cap, n_words] streams")
        bh, cap = 1, packed1.shape[0]
        seq = cap
    elif packed1.ndim == 3 and packed2.ndim == 3:
        bh, cap = packed1.shape[0], packed1.shape[1]
        seq = cap if seq_len is None else int(seq_len)
        if not 0 <= seq <= cap:
            raise ValueError(f"{who}: seq_len={seq} must be in [0, {cap}]")
    else:
        raise ValueError(f"{who}: packed streams must be 2D [N, n_words] or 3D [BH, cap, n_words], got "
                         f"{tuple(packed1.shape)} and {tuple(packed2.shape)}")
    if packed1.shape[-1] != nw:
        raise ValueError(f"{who}: expected {nw} words per row for d={d}, bits={bits}, got packed shape {tuple(packed1.shape)}")
    if packed2.shape != packed1.shape:
        raise ValueError(f"{who}: packed shape mismatch {tuple(packed1.shape)} vs {tuple(packed2.shape)}")
    if packed1.dtype != torch.uint32 or packed2.dtype != torch.uint32:
        raise ValueError(f"{who}: packed streams must be uint32")
    if norms.numel() != bh * cap:
        raise ValueError(f"{who}: expected {bh * cap} norms, got {norms.numel()}")
    c1 = _host_f32(centroids1, 1 << bits, "stage-1 centroids", who)
    c2 = _host_f32(centroids2, 1 << bits, "stage-2 centroids", who)
    if (diag.numel() if isinstance(diag, torch.Tensor) else np.size(diag)) != d:
        raise ValueError(f"{who}: expected diag of size {d}")
    N = bh * seq
    if N == 0:
        return torch.zeros((0, d), dtype=torch.float16, device=packed1.device)
    require_cuda(packed1, f"{who}: packed1")
    dev = packed1.device
    dg = (diag if isinstance(diag, torch.Tensor) else torch.from_numpy(np.asarray(diag))).to(device=dev, dtype=torch.float32).contiguous()
    nr = norms.contiguous()
    if nr.dtype not in (torch.float16, torch.bfloat16, torch.float32):
        nr = nr.float()
    p1, p2 = packed1.contiguous(), packed2.contiguous()
    out = torch.empty((N, d), dtype=torch.float16, device=dev)
    with _lib.on_device(dev):
        check(lib().vq_rvq_unpack_decode(p1.data_ptr(), p2.data_ptr(), nr.data_ptr(), dtype_code(nr.dtype),
                                         c1.ctypes.data_as(C.c_void_p), c2.ctypes.data_as(C.c_void_p), dg.data_ptr(), bits, d,
                                         bh, seq, cap, out.data_ptr(), stream_ptr(dev)), who)
    return out


# ----------------------------------------------------------------------------------------
# the quantizer
# ----------------------------------------------------------------------------------------
class TurboQuantRVQ:
    """Two-pass residual quantizer on rotated coordinates (``quantizers/turboquant_rvq.py:76-326``):
    ``2 * b`` bits per coordinate. ``use_hadamard=True`` (power-of-two ``d``) rotates by the seeded
    randomized Hadamard transform, otherwise by a seeded Haar rotation matrix."""

    def __init__(self, d: int, b: int = 2, seed: int = 42, use_hadamard: bool = False, residual_scale: float | None = None) -> None:
        if not 1 <= b <= 4:
            raise ValueError(f"TurboQuantRVQ: b={b} must be in 1..4 for the packed path")
        self._d, self._b, self._seed = int(d), int(b), int(seed)
        self._hadamard = bool(use_hadamard) and d > 0 and d & (d - 1) == 0
        if self._hadamard:
            self._diag_np = make_hadamard_diagonal(d, seed=seed).astype(np.float32)
            self._pi_np = None
        else:
            self._diag_np = None
            self._pi_np = make_rotation_matrix(d, seed=seed).astype(np.float16)
        self._codebook1 = gaussian_codebook(b, d) if d >= 64 else beta_codebook(b, d)
        if residual_scale is None:
            sigma_q = math.sqrt((math.sqrt(3.0 * math.pi) / 2.0) * (4.0 ** -b) / d)
            residual_scale = max(sigma_q / math.sqrt(2.0), 1e-6)
        self._residual_scale = float(residual_scale)
        self._codebook2 = laplacian_codebook(b, self._residual_scale)
        self._dev: dict = {}

    @property
    def supports_fused_decode(self) -> bool:
        return self._hadamard and self._d <= 1024

    def _rot(self, device):
        t = self._dev.get(str(device))
        if t is None:
            src = self._diag_np if self._hadamard else self._pi_np
            t = torch.from_numpy(src).to(device)
            self._dev[str(device)] = t
        return t

    def rotate(self, x: torch.Tensor) -> torch.Tensor:
        """``y = H (D x)`` (normalized Walsh-Hadamard, float32 arithmetic) or ``x @ Pi^T``, in ``x``'s dtype
        (``preconditioners/rotation.py:44-62``, ``:120-140``)."""
        r = self._rot(x.device)
        if not self._hadamard:
            return (x.float() @ r.float().T).to(x.dtype)
        if self._d in (32, 64, 128, 256) and x.is_cuda:
            from . import vecinfer as vi

            return vi.dual_transform_queries_wht(x, r).to(x.dtype)
        from .vecinfer import walsh_hadamard_matrix

        H = walsh_hadamard_matrix(self._d, device=x.device)
        return ((x.float() * r) @ H).to(x.dtype)

    def rotate_inverse(self, y: torch.Tensor) -> torch.Tensor:
        r = self._rot(y.device)
        if not self._hadamard:
            return (y.float() @ r.float()).to(y.dtype)
        from .vecinfer import walsh_hadamard_matrix

        H = walsh_hadamard_matrix(self._d, device=y.device)
        return ((y.float() @ H) * r).to(y.dtype)

    def encode(self, x: torch.Tensor):
        """``(idx1, idx2)`` uint8 ``[batch, d]``: the unpacked codes of both stages."""
        if x.ndim == 1:
            x = x[None]
        y = self.rotate(x)
        idx1 = self._codebook1.quantize(y)
        r1 = y - self._codebook1.dequantize(idx1).to(y.dtype)
        return idx1, self._codebook2.quantize(r1)

    def encode_pack(self, x: torch.Tensor):
        """Rotate, then quantize both stages and pack in one launch: ``(packed1, packed2)``."""
        if x.ndim == 1:
            x = x[None]
        y = self.rotate(x.to(torch.float16))
        return rvq_quant_pack(y, self._codebook1.centroids, self._codebook1.boundaries, self._codebook2.boundaries, self._b)

    def decode(self, idx1: torch.Tensor, idx2: torch.Tensor) -> torch.Tensor:
        """``unrotate(c1[idx1] + c2[idx2])`` in float16."""
        y = self._codebook1.dequantize(idx1) + self._codebook2.dequantize(idx2)
        return self.rotate_inverse(y)

    def decode_packed(self, packed1, packed2, norms, seq_len: int | None = None) -> torch.Tensor:
        if not self.supports_fused_decode:
            raise ValueError("TurboQuantRVQ.decode_packed requires use_hadamard=True with a power-of-two d <= 1024.")
        return rvq_unpack_decode(packed1, packed2, norms, self._codebook1.centroids, self._codebook2.centroids,
                                 self._rot(packed1.device), self._b, self._d, seq_len=seq_len)


__all__ = ["lloyd_max", "ScalarCodebook", "gaussian_codebook", "beta_codebook", "laplacian_codebook", "pack_indices",
           "unpack_indices", "n_words_for", "rvq_code_table", "rvq_quant_pack", "rvq_unpack_decode", "TurboQuantRVQ"]
