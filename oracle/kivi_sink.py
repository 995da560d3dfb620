"""Oracle: the sink-protected KIVI cache's dense view (test infrastructure only).

A NumPy restatement of ``SinkProtectedKVCache`` (``veloxquant_mlx/cache/sink_cache.py``):

* ``_update_sinks`` (``sink_cache.py:83-107``): per batch element a running top-``n_sink`` of
  token positions by key L2 norm (float32) averaged over the KV heads; pruned with a stable sort
  by descending norm whenever more than ``n_sink`` candidates are held.
* ``update_and_fetch`` (``sink_cache.py:112-190``): the block is appended to a dense buffer kept
  in the input dtype; the newly aged rows ``[n_quantized, boundary)`` are round-tripped through
  the KIVI group quantizer (keys per channel, values per token) after every row that is a sink
  *of its batch element* has been replaced by its nearest non-sink row (left first, then right),
  and the sink rows are then restored to their exact values.
* ``trim`` (``sink_cache.py:192-218``, buffer semantics of ``cache/kivi_cache.py:264-299``): the
  frontier snaps down to a group multiple; candidates at discarded positions are dropped.

Pinning: ``tests/golden/cache_traces.npz`` holds what the reference's own ``SinkProtectedKVCache``
and (with ``n_sink = 0``) ``KIVIKVCache`` classes return over a call script with a trim, executed
unmodified over NumPy stand-ins for ``mlx.core`` and their ``mlx_lm`` base class
(``tests/golden/make_golden.py``); this model reproduces every recorded tensor, the frontier and the
sink positions bit for bit (``tests/test_oracle_golden.py``). Also anchored by the properties the
reference's own tests assert (``veloxquant_mlx/tests/cache/test_sink_cache.py``), restated in
``tests/test_sink_cache_cpu.py``.
"""

from __future__ import annotations

import numpy as np

from . import kivi as o_kivi


def neighbour_sources(sink_local, n: int) -> dict:
    """For each sink row index of a block of ``n`` rows, the row it is neutralised with
    (``sink_cache.py:148-163``); a sink with no non-sink row on either side maps to itself."""
    sink_set = set(sink_local)
    out = {}
    for idx in sorted(sink_local):
        src = idx - 1
        while src in sink_set and src > 0:
            src -= 1
        if src < 0 or src in sink_set:
            src = idx + 1
            while src in sink_set and src < n - 1:
                src += 1
        out[idx] = src if (0 <= src < n and src not in sink_set) else idx
    return out


class SinkProtectedOracle:
    def __init__(self, head_dim: int, bits: int, group: int = 32, residual_length: int = 128, n_sink: int = 5):
        self.head_dim, self.bits, self.group, self.residual_length, self.n_sink = head_dim, bits, group, residual_length, n_sink
        self.levels = (1 << bits) - 1
        self.keys = self.values = None
        self.offset = 0
        self.n_quantized = 0
        self.sink_norms: list[dict[int, float]] = []

    # -- sink bookkeeping ----------------------------------------------------------------
    def _update_sinks(self, keys: np.ndarray, start: int):
        B = keys.shape[0]
        while len(self.sink_norms) < B:
            self.sink_norms.append({})
        if self.n_sink == 0:
            return [set() for _ in range(B)]
        norms = np.sqrt((keys.astype(np.float32) ** 2).sum(-1, dtype=np.float32))  # [B,H,S]
        per_tok = norms.mean(axis=1, dtype=np.float32)
        for b in range(B):
            nb = self.sink_norms[b]
            for i, v in enumerate(per_tok[b].tolist()):
                nb[start + i] = float(v)
            if len(nb) > self.n_sink:
                keep = sorted(nb.items(), key=lambda kv: -kv[1])  # (stable)
                self.sink_norms[b] = dict(keep[: self.n_sink])
        return [set(self.sink_norms[b].keys()) for b in range(B)]

    def sink_positions_for(self, b: int):
        if b >= len(self.sink_norms):
            return []
        return [p for p, _ in sorted(self.sink_norms[b].items(), key=lambda kv: -kv[1])]

    # -- protocol ------------------------------------------------------------------------
    def update_and_fetch(self, keys: np.ndarray, values: np.ndarray):
        B, H, S, D = keys.shape
        start = self.offset
        sinks = self._update_sinks(keys, start)
        if self.keys is None:
            self.keys, self.values = keys.copy(), values.copy()
        else:
            self.keys = np.concatenate([self.keys[:, :, : self.offset], keys], axis=2)
            self.values = np.concatenate([self.values[:, :, : self.offset], values], axis=2)
        self.offset += S
        boundary = o_kivi.quantization_boundary(self.offset, self.residual_length, self.group)
        if boundary > self.n_quantized:
            lo, hi = self.n_quantized, boundary
            n = hi - lo
            k_reg, v_reg = self.keys[:, :, lo:hi].copy(), self.values[:, :, lo:hi].copy()
            local = [sorted(p - lo for p in sinks[b] if lo <= p < hi) for b in range(B)]
            for b in range(B):
                for idx, src in neighbour_sources(local[b], n).items():
                    if src != idx:
                        k_reg[b, :, idx] = self.keys[b, :, lo + src]
                        v_reg[b, :, idx] = self.values[b, :, lo + src]
            k_q = o_kivi.quant_dequant_along(k_reg, -2, self.group, self.levels)
            v_q = o_kivi.quant_dequant_along(v_reg, -1, self.group, self.levels)
            for b in range(B):
                for idx in local[b]:
                    k_q[b, :, idx] = self.keys[b, :, lo + idx]
                    v_q[b, :, idx] = self.values[b, :, lo + idx]
            self.keys[:, :, lo:hi], self.values[:, :, lo:hi] = k_q, v_q
            self.n_quantized = boundary
        return self.keys[:, :, : self.offset], self.values[:, :, : self.offset]

    def trim(self, n: int) -> int:
        n = int(min(max(n, 0), self.offset))
        if n == 0:
            return 0
        self.offset -= n
        if self.offset < self.n_quantized:
            self.n_quantized = (self.offset // self.group) * self.group
        for b, nb in enumerate(self.sink_norms):
            self.sink_norms[b] = {p: v for p, v in nb.items() if p < self.offset}
        return n
