"""Oracle: LSB-first sub-byte packing (test infrastructure only).

Follows ``veloxquant_mlx/dsa/bit_pack.py:44-69`` (``BitPackBuffer.pack``),
``:120-139`` (2-bit), ``:141-196`` (3-bit), ``:198-220`` (4-bit) and
``veloxquant_mlx/metal/src/bit_pack.metal:8-19``: element ``i`` of a row
occupies bits ``[i*b, (i+1)*b)`` of the row's little-endian bit stream.
All four reference layouts (1/2/3/4 bit) are that same rule; this module
states it once for any ``b`` in 1..8.
"""

from __future__ import annotations

import numpy as np


def packed_row_bytes(n: int, b: int) -> int:
    """Bytes needed for ``n`` codes of ``b`` bits: ``ceil(n*b/8)``; the 3-bit
    layout pads to whole 8-value / 3-byte groups as ``_pack_3bit`` does."""
    if b == 3:
        return ((n + 7) // 8) * 3
    return (n * b + 7) // 8


def pack(codes: np.ndarray, b: int) -> np.ndarray:
    """Pack the LAST axis of ``codes`` (uint8, values < 2**b) LSB-first.

    Returns uint8 with last axis ``ceil(n*b/8)``. Values are masked to ``b``
    bits the way ``bit_pack.metal`` and ``_pack_2bit``/``_pack_4bit`` do.
    """
    if not 1 <= b <= 8:
        raise ValueError(f"bitpack.pack: b={b} must be in 1..8")
    codes = np.asarray(codes, dtype=np.uint8)
    n = codes.shape[-1]
    lead = codes.shape[:-1]
    flat = codes.reshape(-1, n) & np.uint8((1 << b) - 1)
    # bit matrix [rows, n, b] -> little-endian stream
    bits = ((flat[:, :, None] >> np.arange(b, dtype=np.uint8)) & 1).astype(np.uint8)
    stream = bits.reshape(flat.shape[0], n * b)
    packed = np.packbits(stream, axis=1, bitorder="little")
    nb = packed_row_bytes(n, b)
    if packed.shape[1] < nb:
        packed = np.concatenate([packed, np.zeros((packed.shape[0], nb - packed.shape[1]), np.uint8)], axis=1)
    return packed.reshape(*lead, nb)


def unpack(packed: np.ndarray, b: int, n: int) -> np.ndarray:
    """Inverse of :func:`pack` along the last axis; returns ``n`` codes."""
    if not 1 <= b <= 8:
        raise ValueError(f"bitpack.unpack: b={b} must be in 1..8")
    packed = np.asarray(packed, dtype=np.uint8)
    lead = packed.shape[:-1]
    flat = packed.reshape(-1, packed.shape[-1])
    stream = np.unpackbits(flat, axis=1, count=n * b, bitorder="little")
    bits = stream.reshape(flat.shape[0], n, b).astype(np.uint16)
    vals = (bits << np.arange(b, dtype=np.uint16)).sum(axis=2).astype(np.uint8)
    return vals.reshape(*lead, n)


def pack_nibbles(v_idx: np.ndarray) -> np.ndarray:
    """Two 4-bit indices per byte, low nibble = even element.

    Follows ``veloxquant_mlx/metal/src/rabitq_pack_values.metal`` and the
    NumPy statement in ``veloxquant_mlx/tests/metal/test_rabitq_values.py:30-34``.
    Out-of-range inputs are masked to 4 bits.
    """
    v_idx = np.asarray(v_idx, dtype=np.uint8)
    if v_idx.shape[-1] % 2:
        raise ValueError("pack_nibbles: last dim must be even")
    lo = v_idx[..., 0::2] & 0xF
    hi = v_idx[..., 1::2] & 0xF
    return (lo | (hi << 4)).astype(np.uint8)
