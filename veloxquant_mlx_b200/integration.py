"""Model-level integration: per-layer caches for a model, attention dispatch to
``cache.fused_sdpa`` and the mask recogniser that guards it.

Reference counterparts: ``integration/mlx_lm_patch.py:25-80`` (``patch_model_kv_cache``: a
``make_cache`` hook that builds a FRESH per-layer cache list on every call),
``metal/fused_sdpa.py:399-416`` (the patched ``scaled_dot_product_attention``: a memory-bound
cache gets ``cache.fused_sdpa(q, scale=, causal=, sliding_window=)``, every other cache the
original attention) and ``metal/fused_sdpa.py:332-396`` (``_memory_bound_mask_parameters``).
The host framework here is PyTorch, so the model side is Hugging Face Transformers instead of
``mlx_lm``: ``VeloxQuantCacheLayer`` is a ``transformers`` cache layer around one cache of
this package, and ``veloxquant_attention`` is an attention function for Transformers'
attention interface. Everything in this module is host logic; the arithmetic stays in the
caches' native kernels.
"""

from __future__ import annotations

import math
from typing import Any, Callable

import torch

from .cache import KVCacheBuilder, KVCacheConfig

_MASK_ERROR = (
    "Memory-bound fused SDPA requires an unmasked, causal, or uniform sliding-window mask. "
    "This mask cannot be represented by the fused kernel. Set fused_sdpa_memory_bound=False to "
    "use standard SDPA."
)


def _memory_bound_mask_parameters(mask: Any, queries: torch.Tensor, kv_length: int) -> tuple[bool, int]:
    """``(causal, sliding_window)`` of a mask the fused kernels can represent; ``ValueError`` for
    every other mask.

    Accepted: ``None`` (all keys visible), the string ``"causal"``, or an array mask -- boolean,
    or additive with entries 0 / -inf -- of 1 to 4 dimensions broadcastable to
    ``[B, H, S_q, kv_length]`` that is uniform over batch and heads and is EXACTLY all-visible,
    or the tail-aligned causal mask (query row ``r`` sits at key ``kv_length - S_q + r``),
    optionally bounded by a uniform trailing window. Every entry is compared, nothing is
    inferred from the shape: padding, holes, per-head masks and biases raise instead of being
    ignored (reference: ``metal/fused_sdpa.py:332-396``).
    """
    if mask is None:
        return False, 0
    if isinstance(mask, str):
        if mask == "causal":
            return True, 0
        raise ValueError(_MASK_ERROR)
    if not isinstance(mask, torch.Tensor) or not 1 <= mask.ndim <= 4:
        raise ValueError(_MASK_ERROR)
    B, H, N, _ = queries.shape
    expected = (B, H, N, kv_length)
    padded = (1,) * (4 - mask.ndim) + tuple(mask.shape)
    if N < 1 or kv_length < N or any(a not in (1, e) for a, e in zip(padded, expected)):
        raise ValueError(_MASK_ERROR)
    if mask.dtype == torch.bool:
        visible = mask
        entries_ok = True
    elif mask.dtype.is_floating_point:
        visible = mask == 0
        entries_ok = bool((visible | (mask == float("-inf"))).all())
    else:
        raise ValueError(_MASK_ERROR)
    if not entries_ok:
        raise ValueError(_MASK_ERROR)
    shaped = visible.reshape(padded).expand(*padded[:-1], kv_length) if padded[-1] == 1 else visible.reshape(padded)
    # uniform over batch and heads: every [b, h] slice equals the first one
    first = shaped[:1, :1]
    if not bool((shaped == first).all()):
        raise ValueError(_MASK_ERROR)
    rows = first[0, 0]
    if rows.shape[0] == 1 and N > 1:
        rows = rows.expand(N, kv_length)
    if bool(rows.all()):
        return False, 0
    # The last query aligns with the last key; its visible count is the candidate window width,
    # verified by the full comparison.
    width = int(rows[-1].sum())
    dev = rows.device
    q_pos = torch.arange(kv_length - N, kv_length, device=dev)[:, None]
    k_pos = torch.arange(kv_length, device=dev)[None, :]
    candidate = (k_pos <= q_pos) & (k_pos > q_pos - width)
    if width > 0 and bool((rows == candidate).all()):
        return True, 0 if width == kv_length else width
    raise ValueError(_MASK_ERROR)


def fused_sdpa_dispatch(queries: torch.Tensor, keys: torch.Tensor, values: torch.Tensor, cache: Any, scale: float,
                        mask: Any, sinks: Any = None, original: Callable | None = None) -> torch.Tensor:
    """The attention call of a model layer, routed as the reference's patched SDPA routes it.

    A memory-bound cache returned sentinel K/V from ``update_and_fetch``: the call must either
    dispatch ``cache.fused_sdpa`` or raise -- never attend over the sentinels. Every other cache
    keeps real K/V and takes ``original(queries, keys, values, cache=, scale=, mask=, sinks=)``
    (default: PyTorch's ``scaled_dot_product_attention`` with grouped-query head repetition).
    """
    if getattr(cache, "_memory_bound", False):
        if sinks is not None:
            raise ValueError("Memory-bound fused SDPA does not support attention sinks. "
                             "Set fused_sdpa_memory_bound=False to use standard SDPA.")
        if not callable(getattr(cache, "fused_sdpa", None)):
            raise RuntimeError("Memory-bound cache requires a callable fused_sdpa method.")
        causal, window = _memory_bound_mask_parameters(mask, queries, int(cache.offset))
        return cache.fused_sdpa(queries, scale=scale, causal=causal, sliding_window=window)
    if original is not None:
        return original(queries, keys, values, cache=cache, scale=scale, mask=mask, sinks=sinks)
    return _dense_sdpa(queries, keys, values, scale, mask)


def _dense_sdpa(q, k, v, scale, mask):
    rep = q.shape[1] // k.shape[1]
    if rep > 1:
        k = k.repeat_interleave(rep, dim=1)
        v = v.repeat_interleave(rep, dim=1)
    if isinstance(mask, str):
        n, s = q.shape[2], k.shape[2]
        mask = torch.ones(n, s, dtype=torch.bool, device=q.device).tril(diagonal=s - n)
    return torch.nn.functional.scaled_dot_product_attention(q, k, v, attn_mask=mask, scale=scale)


# ----------------------------------------------------------------------------------------------
# Hugging Face Transformers
# ----------------------------------------------------------------------------------------------
def _cache_layer_base():
    from transformers.cache_utils import CacheLayerMixin

    return CacheLayerMixin


def make_cache_layer_class():
    """The ``transformers`` cache-layer class (built on first use, so that importing this module
    does not import ``transformers``)."""
    global _LAYER_CLASS
    if _LAYER_CLASS is not None:
        return _LAYER_CLASS
    Base = _cache_layer_base()

    class VeloxQuantCacheLayer(Base):
        """One attention layer's compressed cache behind Transformers' cache-layer interface.

        ``update`` appends through ``update_and_fetch``. A standard-mode cache returns the
        history as it would be after dequantization, which any attention implementation can
        consume; a memory-bound cache returns zero-length sentinels that carry a reference to
        the cache (``keys.velox_cache``), and ``veloxquant_attention`` attends over the packed
        store instead.
        """

        is_compileable = False
        is_sliding = False

        def __init__(self, cache: Any) -> None:
            super().__init__()
            self.cache = cache

        def lazy_initialization(self, key_states, value_states) -> None:
            self.dtype, self.device = key_states.dtype, key_states.device
            self.is_initialized = True

        def update(self, key_states, value_states, *args, **kwargs):
            if not self.is_initialized:
                self.lazy_initialization(key_states, value_states)
            k, v = self.cache.update_and_fetch(key_states, value_states)
            if getattr(self.cache, "_memory_bound", False):
                k = k.view(k.shape)  # a fresh tensor object: the attribute must not leak between layers
                k.velox_cache = self.cache
            self.keys, self.values = k, v
            return k, v

        def get_seq_length(self) -> int:
            return int(self.cache.offset)

        def get_mask_sizes(self, query_length) -> tuple[int, int]:
            q = int(query_length.shape[0]) if isinstance(query_length, torch.Tensor) else int(query_length)
            return int(self.cache.offset) + q, 0

        def get_max_cache_shape(self) -> int:
            return -1

        def reset(self) -> None:
            self.cache.reset()

        def crop(self, max_length: int) -> None:
            n = int(self.cache.offset)
            if max_length < 0:
                max_length = n + max_length
            if n > max_length:
                self.cache.trim(n - max_length)

        def reorder_cache(self, beam_idx) -> None:
            raise NotImplementedError("VeloxQuantCacheLayer: beam search reordering is not supported")

    _LAYER_CLASS = VeloxQuantCacheLayer
    return _LAYER_CLASS


_LAYER_CLASS = None


def make_hf_cache(model_or_n_layers: Any, config: KVCacheConfig):
    """A fresh ``transformers.Cache`` whose layers are caches of this package: for a model, what
    :meth:`KVCacheBuilder.for_model` plans for it (``integration/mlx_lm_patch.py:25-80`` builds its
    list the same way); for a layer count, that many caches of ``config`` with seeds ``config.seed + i``
    and a list-form ``bit_width_inlier`` spread over them."""
    from transformers.cache_utils import Cache

    Layer = make_cache_layer_class()
    if isinstance(model_or_n_layers, int):
        caches = KVCacheBuilder.for_layers(model_or_n_layers, config)
    else:   # per-layer head_dim from the model itself, a plain cache for a layer without attention
        caches = KVCacheBuilder.for_model(model_or_n_layers, config)
    return Cache(layers=[Layer(c) for c in caches])


def patch_model_kv_cache(model: Any, config: KVCacheConfig):
    """Give ``model`` a ``make_cache()`` hook that builds a FRESH compressed cache on every call
    (``model.generate(..., past_key_values=model.make_cache())``), and return the first one,
    which also validates ``config`` eagerly. Reference: ``integration/mlx_lm_patch.py:25-80``."""
    def _make_cache(*_a, **_k):
        return make_hf_cache(model, config)

    first = _make_cache()
    model.make_cache = _make_cache
    return first


def veloxquant_attention(module: Any, query: torch.Tensor, key: torch.Tensor, value: torch.Tensor,
                         attention_mask: Any, dropout: float = 0.0, scaling: float | None = None, **kwargs):
    """Attention function for Transformers' attention interface (``attn_implementation=
    "veloxquant"`` after :func:`register_attention`). ``key`` / ``value`` are what the layer's
    cache returned: sentinels of a memory-bound cache are dispatched to ``cache.fused_sdpa``
    (after the mask was recognised), real tensors go to PyTorch's dense attention."""
    scale = float(scaling) if scaling is not None else 1.0 / math.sqrt(query.shape[-1])
    cache = getattr(key, "velox_cache", None)
    mask = attention_mask
    # Transformers passes no mask when plain causal attention is meant (several query rows of a
    # causal module) or when nothing is masked (one query row)
    is_causal = kwargs.get("is_causal")
    if is_causal is None:
        is_causal = getattr(module, "is_causal", True)
    if mask is None and query.shape[2] > 1 and is_causal:
        mask = "causal"
    if cache is not None:
        out = fused_sdpa_dispatch(query, key, value, cache, scale, mask, sinks=kwargs.get("s_aux"))
    else:
        if key.shape[-2] == 0:
            # a memory-bound cache's sentinel that lost its reference to the cache (something copied
            # or reshaped the key tensor on the way here): there is nothing to attend over
            raise RuntimeError("veloxquant_attention: received zero-length keys without a cache reference; a "
                               "memory-bound cache must reach this function through VeloxQuantCacheLayer.update unchanged")
        out = _dense_sdpa(query, key, value, scale, mask)
    return out.transpose(1, 2).contiguous(), None


def register_attention(name: str = "veloxquant") -> str:
    """Register :func:`veloxquant_attention` (and the mask builder of the ``sdpa`` implementation)
    under ``name`` with Transformers; returns the name to use as ``attn_implementation``."""
    from transformers import AttentionInterface
    from transformers.masking_utils import AttentionMaskInterface, sdpa_mask

    AttentionInterface.register(name, veloxquant_attention)
    AttentionMaskInterface.register(name, sdpa_mask)
    return name


def patch_hf_for_fused_sdpa(model: Any, name: str = "veloxquant") -> None:
    """Route every attention layer of ``model`` through :func:`veloxquant_attention`."""
    register_attention(name)
    model.config._attn_implementation = name
    for m in model.modules():
        cfg = getattr(m, "config", None)
        if cfg is not None and hasattr(cfg, "_attn_implementation"):
            cfg._attn_implementation = name


__all__ = ["fused_sdpa_dispatch", "make_hf_cache", "patch_model_kv_cache", "veloxquant_attention", "register_attention",
           "patch_hf_for_fused_sdpa", "make_cache_layer_class"]
