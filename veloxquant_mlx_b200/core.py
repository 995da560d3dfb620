"""Standalone cache protocol and the typed quantizer output of the reference's ``core`` package.

``KVCache`` mirrors the abstract base class ``veloxquant_mlx/core/abstractions.py:120-189``
(``append_key`` / ``append_value`` / ``attend`` / ``memory_bytes`` / ``reset`` / ``append`` /
``__len__``): one key and one value vector of one head per call, ``attend(q)`` returning
``softmax(q.K^T / sqrt(d)) V`` as the reference's standalone caches compute it
(``cache/turboquant_cache.py:250-330``). ``EncodedVector`` mirrors ``core/context.py:72-138``.

``StandaloneProtocol`` implements that interface on top of the batched
``update_and_fetch`` / ``fused_sdpa`` protocol, so every cache of this package (KIVI, VecInfer,
RaBitQ) is also a ``KVCache``: a single-head cache is the batched one with ``B = H = 1``.
"""

from __future__ import annotations

import math
from abc import ABC, abstractmethod
from dataclasses import dataclass
from typing import Any

import numpy as np
import torch


class KVCache(ABC):
    """Abstract base class of the standalone (one vector per call) cache protocol."""

    @abstractmethod
    def append_key(self, k: Any) -> None:
        """Append a new key vector, shape ``(d,)``."""

    @abstractmethod
    def append_value(self, v: Any) -> None:
        """Append the value vector that belongs to the key appended last, shape ``(d,)``."""

    @abstractmethod
    def attend(self, q: Any) -> Any:
        """Attention-weighted value for a query of shape ``(d,)``; returns ``(d,)``."""

    @abstractmethod
    def memory_bytes(self) -> int:
        """Current footprint of the stored tokens in bytes."""

    def reset(self) -> None:
        """Clear all stored tokens, keeping quantizer / calibration / configuration state.
        Not abstract (a decorator may give "reset" another meaning); the default raises."""
        raise NotImplementedError(f"{type(self).__name__} does not implement reset()")

    def append(self, k: Any, v: Any) -> None:
        """Append a key-value pair in one call."""
        self.append_key(k)
        self.append_value(v)

    def __len__(self) -> int:
        raise NotImplementedError

    def __repr__(self) -> str:
        return f"{self.__class__.__name__}(size={len(self)})"


class StandaloneProtocol(KVCache):
    """``KVCache`` on top of a batched cache (``update_and_fetch`` / ``fused_sdpa`` / ``offset`` /
    ``nbytes`` / ``_reset_tokens``). The key waits for its value: a token enters the store when
    both have arrived, so a query never sees a key without a value."""

    _pending_key = None

    @staticmethod
    def _as_row(x: Any, what: str) -> torch.Tensor:
        if not isinstance(x, torch.Tensor):
            x = torch.as_tensor(x)
        if x.ndim == 2 and x.shape[0] == 1:
            x = x[0]
        if x.ndim != 1:
            raise ValueError(f"{what}: expected a vector of shape (d,), got {tuple(x.shape)}")
        return x

    def append_key(self, k: Any) -> None:
        if self._pending_key is not None:
            raise RuntimeError(f"{type(self).__name__}.append_key: the previous key still waits for its value")
        k = self._as_row(k, f"{type(self).__name__}.append_key")
        if k.shape[0] != self._head_dim:
            raise ValueError(f"{type(self).__name__}.append_key: expected d={self._head_dim}, got {k.shape[0]}")
        self._pending_key = k

    def append_value(self, v: Any) -> None:
        if self._pending_key is None:
            raise RuntimeError(f"{type(self).__name__}.append_value: append_key comes first")
        v = self._as_row(v, f"{type(self).__name__}.append_value")
        k, self._pending_key = self._pending_key, None
        if v.shape != k.shape:
            raise ValueError(f"{type(self).__name__}.append_value: key has d={k.shape[0]}, value d={v.shape[0]}")
        d = k.shape[0]
        self.update_and_fetch(k.reshape(1, 1, 1, d), v.to(dtype=k.dtype, device=k.device).reshape(1, 1, 1, d))

    def attend(self, q: Any) -> torch.Tensor:
        q = self._as_row(q, f"{type(self).__name__}.attend")
        d = q.shape[0]
        if len(self) == 0:
            return torch.zeros_like(q)
        return self.fused_sdpa(q.reshape(1, 1, 1, d), 1.0 / math.sqrt(d)).reshape(d)

    def memory_bytes(self) -> int:
        return int(self.nbytes)

    def reset(self) -> None:
        self._pending_key = None
        self._reset_tokens()

    def __len__(self) -> int:
        return int(self.offset)


@dataclass
class EncodedVector:
    """Typed output of a quantizer's ``encode`` (reference: ``core/context.py:72-138``); different
    quantizers fill different fields. Arrays may be ``torch`` tensors or NumPy arrays."""

    quantizer_type: str
    batch_size: int
    dim: int
    indices: Any | None = None
    norm: Any | None = None
    signs: Any | None = None
    residual_norm: Any | None = None
    angles: list | None = None
    final_radius: Any | None = None
    outlier_idx: Any | None = None
    outlier_encoded: "EncodedVector | None" = None
    inlier_encoded: "EncodedVector | None" = None

    def memory_bytes(self) -> int:
        """Exact bytes of every stored array, nested encodings included."""

        def nbytes(a: Any) -> int:
            if a is None:
                return 0
            if isinstance(a, np.ndarray):
                return int(a.nbytes)
            if isinstance(a, torch.Tensor):
                return int(a.numel() * a.element_size())
            return int(getattr(a, "nbytes", 0))

        total = sum(nbytes(a) for a in (self.indices, self.norm, self.signs, self.residual_norm, self.final_radius,
                                        self.outlier_idx))
        for a in self.angles or ():
            total += nbytes(a)
        for nested in (self.outlier_encoded, self.inlier_encoded):
            if nested is not None:
                total += nested.memory_bytes()
        return total

    def __repr__(self) -> str:
        fields = [n for n in ("indices", "norm", "signs", "residual_norm", "angles", "final_radius", "outlier_idx",
                              "outlier_encoded", "inlier_encoded") if getattr(self, n) is not None]
        return (f"EncodedVector(type={self.quantizer_type!r}, batch={self.batch_size}, d={self.dim}, "
                f"fields={fields}, bytes={self.memory_bytes()})")


__all__ = ["KVCache", "StandaloneProtocol", "EncodedVector"]
