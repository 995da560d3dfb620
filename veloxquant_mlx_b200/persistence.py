"""Persistence of compressed caches and prefix-cache reuse.

The reference hands persistence to ``mlx_lm``: a cache exposes ``state`` (arrays) and
``meta_state`` (strings), ``mlx_lm.models.cache.save_prompt_cache`` writes them to one
safetensors file, and ``LRUPromptCache`` (wrapped by ``integration/prefix_cache.py``) reuses a
stored prompt's cache for a prompt that shares its prefix
(``cache/vecinfer_cache.py:542-609``, ``cache/turboquant_rvq_cache.py:380-425``,
``integration/prefix_cache.py``). ``mlx_lm`` is not available here, so this module provides
the same three pieces for the caches of this package:

* ``save_prompt_cache`` / ``load_prompt_cache`` -- one safetensors file for a list of per-layer
  caches. On-disk layout: tensor ``"<layer>.<j>"`` is element ``j`` of that cache's ``state``
  (only the LIVE rows: packed codes ``u8 [B,H,n_q,D*sb/8]``, fp32 scales / zero-points,
  the residual window in the activation dtype, index or sign-bit arrays), and the file's
  metadata holds, per layer, the cache method and its ``meta_state`` strings, plus the caller's
  own metadata. The live token count travels in ``meta_state`` and, as in the reference, in the
  array lengths.
* ``PrefixCache`` -- an LRU store keyed by token sequences: ``fetch(prompt)`` returns fresh caches
  restored from the longest stored prefix (a longer stored entry is cut back with ``trim``, which
  for KIVI re-opens the partly trimmed group exactly as the live cache would) and the tokens that
  still have to be prefilled.
"""

from __future__ import annotations

import json
from collections import OrderedDict
from typing import Any, Hashable, Sequence

import torch

from .cache import KVCacheConfig, KVCacheFactory, _CACHE_CLASS_BY_METHOD

_FORMAT = "veloxquant-b200-prompt-cache/1"


def _method_of(cache: Any) -> str:
    for name, cls in _CACHE_CLASS_BY_METHOD.items():
        if type(cache) is cls:
            return name
    raise TypeError(f"save_prompt_cache: {type(cache).__name__} is not a cache of this package")


def save_prompt_cache(path: str, caches: Sequence[Any], metadata: dict | None = None) -> None:
    """Write the per-layer ``caches`` (their ``state`` and ``meta_state``) to one safetensors file."""
    from safetensors.torch import save_file

    tensors: dict = {}
    layers = []
    for i, c in enumerate(caches):
        st = tuple(c.state)
        present = []
        for j, t in enumerate(st):
            if t is None:
                continue
            tensors[f"{i}.{j}"] = t.detach().contiguous().cpu()
            present.append(j)
        layers.append({"method": _method_of(c), "meta_state": list(c.meta_state), "n_state": len(st), "present": present})
    header = {"format": _FORMAT, "layers": json.dumps(layers), "user": json.dumps(metadata or {})}
    if not tensors:  # safetensors needs at least the header; an all-empty cache list still round-trips
        tensors["empty"] = torch.zeros(1, dtype=torch.uint8)
    save_file(tensors, path, metadata=header)


def load_prompt_cache(path: str, config: KVCacheConfig | Sequence[KVCacheConfig], device: Any = "cuda",
                      return_metadata: bool = False):
    """Rebuild the per-layer caches of ``save_prompt_cache``. ``config`` supplies what is not
    state (codebooks, smooth factors, flags): one config for all layers or one per layer; its
    ``method`` must match the stored one. Counters and the packed layout come from the file."""
    from safetensors import safe_open

    with safe_open(path, framework="pt", device="cpu") as f:
        header = f.metadata() or {}
        if header.get("format") != _FORMAT:
            raise ValueError(f"load_prompt_cache: {path} is not a {_FORMAT} file")
        layers = json.loads(header["layers"])
        configs = list(config) if isinstance(config, (list, tuple)) else [config] * len(layers)
        if len(configs) != len(layers):
            raise ValueError(f"load_prompt_cache: {len(layers)} layers stored, {len(configs)} configs given")
        caches = []
        for i, (rec, cfg) in enumerate(zip(layers, configs)):
            if cfg.method != rec["method"]:
                raise ValueError(f"load_prompt_cache: layer {i} was saved by method {rec['method']!r}, config says {cfg.method!r}")
            st = [None] * rec["n_state"]
            for j in rec["present"]:
                st[j] = f.get_tensor(f"{i}.{j}").to(device)
            c = KVCacheFactory.create(cfg)
            c.meta_state = tuple(rec["meta_state"])
            c.state = tuple(st)
            caches.append(c)
    if return_metadata:
        return caches, json.loads(header.get("user", "{}"))
    return caches


def clone_caches(caches: Sequence[Any], config: KVCacheConfig | Sequence[KVCacheConfig]) -> list:
    """Independent copies (fresh objects, cloned tensors) through ``state`` / ``meta_state``."""
    configs = list(config) if isinstance(config, (list, tuple)) else [config] * len(caches)
    out = []
    for c, cfg in zip(caches, configs):
        n = KVCacheFactory.create(cfg)
        n.meta_state = tuple(c.meta_state)
        n.state = tuple(None if t is None else t.clone() for t in c.state)
        out.append(n)
    return out


class PrefixCache:
    """LRU store of prompt caches keyed by ``(model_key, token sequence)``.

    ``insert(tokens, caches)`` stores a snapshot of ``caches`` as the state after ``tokens``.
    ``fetch(tokens)`` looks for the stored sequence with the longest common prefix with
    ``tokens``, returns copies of its caches cut back to that prefix (never the whole prompt: at
    least the last token stays to be fed to the model) and the remaining tokens; on a miss it
    returns fresh caches and the whole prompt. Mirrors the reference's ``PrefixCache``
    (``integration/prefix_cache.py``) with the LRU of ``mlx_lm`` written out.
    """

    def __init__(self, config: KVCacheConfig, n_layers: int, *, max_size: int = 10, max_bytes: int = 1 << 63,
                 factory=None, cloner=None) -> None:
        self._config, self._n_layers = config, int(n_layers)
        self._max_size, self._max_bytes = int(max_size), int(max_bytes)
        self._entries: "OrderedDict[tuple, tuple]" = OrderedDict()  # (model_key, tokens) -> (caches, nbytes)
        self._factory = factory or (lambda: [KVCacheFactory.create(config) for _ in range(self._n_layers)])
        self._cloner = cloner or (lambda caches: clone_caches(caches, config))
        self.hits = self.misses = 0

    def __len__(self) -> int:
        return len(self._entries)

    @property
    def nbytes(self) -> int:
        return sum(b for _, b in self._entries.values())

    @staticmethod
    def _common(a: Sequence[int], b: Sequence[int]) -> int:
        n = 0
        for x, y in zip(a, b):
            if x != y:
                break
            n += 1
        return n

    def fetch(self, prompt: Sequence[int], *, model_key: Hashable | None = None):
        """``(caches, rest)``: caches holding a prefix of ``prompt`` and the tokens still to feed."""
        prompt = list(prompt)
        best_key, best_len = None, 0
        for key in self._entries:
            if key[0] != model_key:
                continue
            n = self._common(key[1], prompt)
            if n > best_len:
                best_key, best_len = key, n
        usable = min(best_len, len(prompt) - 1)  # the model needs at least one input token
        if best_key is None or usable <= 0:
            self.misses += 1
            return self._factory(), prompt
        stored, _ = self._entries[best_key]
        self._entries.move_to_end(best_key)
        caches = self._cloner(stored)
        cut = len(best_key[1]) - usable
        if cut > 0:
            for c in caches:
                if hasattr(c, "is_trimmable") and not c.is_trimmable():
                    self.misses += 1
                    return self._factory(), prompt
                c.trim(cut)
        self.hits += 1
        return caches, prompt[usable:]

    def insert(self, tokens: Sequence[int], caches: Sequence[Any], *, model_key: Hashable | None = None) -> None:
        """Store a snapshot of ``caches`` as the state after the FULL sequence ``tokens`` (prompt
        plus generated tokens)."""
        key = (model_key, tuple(tokens))
        snap = self._cloner(caches)
        size = sum(int(getattr(c, "nbytes", 0)) for c in snap)
        self._entries.pop(key, None)
        self._entries[key] = (snap, size)
        while len(self._entries) > self._max_size or (self.nbytes > self._max_bytes and len(self._entries) > 1):
            self._entries.popitem(last=False)


__all__ = ["save_prompt_cache", "load_prompt_cache", "clone_caches", "PrefixCache"]
