"""Cache-level drop-in surface: ``KVCacheConfig`` / ``KVCacheFactory`` / ``KVCacheBuilder`` and
the packed KIVI cache.

Mirrors the reference's ``veloxquant_mlx/cache/base.py`` (config ``:473-864``, factory
``:974-1048``, builder ``:1242-1433``), ``cache/options.py:35-50`` and
``cache/kivi_cache.py`` for the methods on the compressed-KV hot path. Only the fields those
methods read exist here. Tensors are ``torch`` CUDA tensors; all arithmetic runs in the
native library (no CPU path).

Difference from the reference that is the point of this package: the reference's KIVI cache
quantizes and immediately dequantizes back into an fp16 buffer (``cache/kivi_cache.py:26-43``);
this one KEEPS the packed codes + fp32 (scale, zero) and attends over them directly with
:meth:`KIVIKVCache.fused_sdpa`. ``update_and_fetch`` still returns the reference's view of
the history (round-tripped quantized region followed by the exact residual window) unless
``fused_sdpa_memory_bound=True``, in which case it returns empty sentinels like the
reference's VecInfer memory-bound mode (``cache/vecinfer_cache.py:491-532``).
"""

from __future__ import annotations

import ctypes as C
import dataclasses
import functools
import math
import warnings
from dataclasses import dataclass, field
from typing import Any

import torch

from . import _lib, kernels
from .core import EncodedVector, KVCache, StandaloneProtocol


class QuantizerConfigError(ValueError):
    """Invalid cache / quantizer configuration (reference: ``core/exceptions.py:12``)."""


# ----------------------------------------------------------------------------------------
# options (reference: cache/options.py)
# ----------------------------------------------------------------------------------------
@dataclass
class VecInferOptions:
    key_sub_dim: int = 4
    value_sub_dim: int = 8
    key_codebook_bits: int = 12
    value_codebook_bits: int = 8
    residual_length: int = 128


@dataclass
class KIVIOptions:
    kivi_group_size: int = 32


@dataclass
class SKVQOptions:
    """SKVQ configuration (reference: ``cache/options.py:314-325``)."""

    skvq_bits_key: int = 4
    skvq_bits_value: int = 4
    skvq_group_size: int = 32
    skvq_window: int = 128
    skvq_n_sink: int = 5
    skvq_reorder: bool = True
    skvq_clip_search: bool = True
    skvq_clip_alpha: float = 1.0
    skvq_max_ctx: Any = None


@dataclass
class KittyOptions:
    """Kitty configuration (reference: ``cache/options.py:67-73``)."""

    kitty_hi_fraction: float = 0.25
    kitty_hi_bit: int = 4
    kitty_lo_bit: int = 2
    kitty_group_size: int = 32


@dataclass
class AgeTieredKVOptions:
    """AgeTieredKV configuration (reference: ``cache/options.py:496-505``)."""

    age_recent_boundary: int = 128
    age_mid_boundary: int = 1024
    age_bits_recent: int = 8
    age_bits_mid: int = 4
    age_bits_old: int = 2
    age_group_size: int = 32


_FIELD_TO_OPTIONS_CLASS = {
    "key_sub_dim": "VecInferOptions", "value_sub_dim": "VecInferOptions",
    "key_codebook_bits": "VecInferOptions", "value_codebook_bits": "VecInferOptions",
    "residual_length": "VecInferOptions", "kivi_group_size": "KIVIOptions",
    **{name: "SKVQOptions" for name in ("skvq_bits_key", "skvq_bits_value", "skvq_group_size", "skvq_window", "skvq_n_sink",
                                        "skvq_reorder", "skvq_clip_search", "skvq_clip_alpha", "skvq_max_ctx")},
    **{name: "KittyOptions" for name in ("kitty_hi_fraction", "kitty_hi_bit", "kitty_lo_bit", "kitty_group_size")},
    **{name: "AgeTieredKVOptions" for name in ("age_recent_boundary", "age_mid_boundary", "age_bits_recent", "age_bits_mid",
                                             "age_bits_old", "age_group_size")},
}

_CACHE_CLASS_BY_METHOD: dict = {}  # filled at the bottom of the module


@dataclass
class KVCacheConfig:
    """Configuration of one cache instance (hot-path subset of the reference's dataclass).

    ``use_metal_kernels`` is kept for source compatibility: ``None``/``True`` select the
    native kernels (the only implementation here); ``False`` asks for the reference's
    pure-MLX twin, which does not exist in this package, and is rejected.
    """

    method: str = "turboquant_rvq"   # (the reference's default, cache/base.py)
    head_dim: int = 128
    bit_width_inlier: Any = 2
    bit_width_outlier: Any = None
    seed: int = 42
    dtype: Any = None
    capacity: Any = None
    sliding_window: Any = None
    observers: list = field(default_factory=list)
    options: Any = None
    key_sub_dim: int = 4
    value_sub_dim: int = 8
    key_codebook_bits: int = 12
    value_codebook_bits: int = 8
    residual_length: int = 128
    kivi_group_size: int = 32
    smooth_factors: Any = None
    key_codebook: Any = None
    value_codebook: Any = None
    use_metal_kernels: Any = None
    fused_sdpa: Any = False
    fused_sdpa_max_ctx: Any = None
    fused_sdpa_memory_bound: bool = False
    n_sink_tokens: int = 5
    skvq_bits_key: int = 4
    skvq_bits_value: int = 4
    skvq_group_size: int = 32
    skvq_window: int = 128
    skvq_n_sink: int = 5
    skvq_reorder: bool = True
    skvq_clip_search: bool = True
    skvq_clip_alpha: float = 1.0
    skvq_max_ctx: Any = None
    kitty_hi_fraction: float = 0.25
    kitty_hi_bit: int = 4
    kitty_lo_bit: int = 2
    kitty_group_size: int = 32
    age_recent_boundary: int = 128
    age_mid_boundary: int = 1024
    age_bits_recent: int = 8
    age_bits_mid: int = 4
    age_bits_old: int = 2
    age_group_size: int = 32

    def __repr__(self) -> str:
        return (f"KVCacheConfig(method={self.method!r}, d={self.head_dim}, "
                f"b={self.bit_width_inlier}, seed={self.seed})")

    def __post_init__(self) -> None:
        # An `options` dataclass fills its flat fields unless the caller NAMED the flat
        # field (even with its default value): reference cache/base.py:872-888, :957-971.
        if self.options is not None and dataclasses.is_dataclass(self.options):
            explicit = getattr(self, "_explicit_fields", frozenset())
            for f in dataclasses.fields(self.options):
                if f.name in _FIELD_TO_OPTIONS_CLASS and f.name not in explicit:
                    object.__setattr__(self, f.name, getattr(self.options, f.name))
        _warn_inlier_bits_ignored(self, getattr(self, "_explicit_fields", frozenset()))
        object.__setattr__(self, "_post_init_done", True)

    def __setattr__(self, name: str, value: Any) -> None:
        if getattr(self, "_post_init_done", False) and name in _FIELD_TO_OPTIONS_CLASS:
            cls_name = _FIELD_TO_OPTIONS_CLASS[name]
            warnings.warn(
                f"KVCacheConfig.{name} is deprecated in favor of {cls_name} "
                f"(pass it via KVCacheConfig(options={cls_name}({name}=...))).",
                DeprecationWarning, stacklevel=2)
        object.__setattr__(self, name, value)


# the methods (of this package) whose caches read ``bit_width_inlier``
_INLIER_BITS_METHODS = frozenset({"kivi", "kivi_sink", "turboquant_rvq"})


def _warn_inlier_bits_ignored(config, explicit) -> None:
    """``UserWarning`` when the caller NAMED ``bit_width_inlier`` for a method that never reads it
    (reference: ``cache/base.py:930-955``). A copy made by ``dataclasses.replace`` names every field
    and is not the caller asking for a width: no warning then."""
    if "bit_width_inlier" not in explicit or config.method in _INLIER_BITS_METHODS:
        return
    init_names = {f.name for f in dataclasses.fields(config) if f.init}
    if explicit >= init_names:
        return
    own = sorted(f.name for f in dataclasses.fields(config)
                 if f.init and "bit" in f.name and f.name.startswith(f"{config.method}_"))
    hint = f"; this method's own bit-width field is {', '.join(own)}" if own else ""
    warnings.warn(f"KVCacheConfig(method={config.method!r}) ignores bit_width_inlier={config.bit_width_inlier!r}: only "
                  f"{', '.join(sorted(_INLIER_BITS_METHODS))} read it{hint}.", UserWarning, stacklevel=5)


def _track_explicit_fields(cls):
    init = cls.__init__
    names = [f.name for f in dataclasses.fields(cls) if f.init]

    @functools.wraps(init)
    def __init__(self, *args, **kwargs):
        object.__setattr__(self, "_explicit_fields", frozenset(names[: len(args)]) | kwargs.keys())
        init(self, *args, **kwargs)

    cls.__init__ = __init__
    return cls


_track_explicit_fields(KVCacheConfig)


class KVCacheFactory:
    """``KVCacheFactory.create(config)`` -> cache (reference: ``cache/base.py:974-1048``)."""

    @staticmethod
    def create(config: KVCacheConfig):
        b = config.bit_width_inlier
        if isinstance(b, list) and config.method != "vecinfer":
            raise QuantizerConfigError(
                "KVCacheFactory.create() requires bit_width_inlier to be a single int. "
                "List-form bit_width_inlier (per-layer allocation) is consumed by "
                "KVCacheBuilder.for_model(), which dispatches to create() once per layer.")
        if config.observers:
            raise QuantizerConfigError(
                "KVCacheFactory.create() received a non-empty config.observers, but no cache "
                "implementation emits QuantizationEvent -- remove `observers` from KVCacheConfig.")
        if config.bit_width_outlier is not None:
            raise QuantizerConfigError(
                f"KVCacheFactory.create() received config.bit_width_outlier={config.bit_width_outlier!r}, "
                "but no cache implementation reads this field. Remove `bit_width_outlier` from "
                "KVCacheConfig; it has no effect.")
        cls = _CACHE_CLASS_BY_METHOD.get(config.method)
        if cls is None:
            choices = ", ".join(_CACHE_CLASS_BY_METHOD)
            raise QuantizerConfigError(f"KVCacheFactory: unknown method '{config.method}'. Choices: {choices}.")
        if config.sliding_window is not None:
            raise QuantizerConfigError(
                f"KVCacheFactory: sliding_window is only compatible with standalone methods -- "
                f"method {config.method!r} implements the update_and_fetch protocol.")
        return cls(config)


class KVCacheBuilder:
    """Fluent builder (reference: ``cache/base.py:1050-1241``) for the fields the hot-path methods read;
    ``build()`` validates as the reference's does (power-of-two head_dim, bit widths >= 1) before the
    factory is called."""

    def __init__(self) -> None:
        self._config = KVCacheConfig()

    def _set(self, name: str, value) -> "KVCacheBuilder":
        object.__setattr__(self._config, name, value)
        return self

    def with_method(self, method: str) -> "KVCacheBuilder":
        return self._set("method", method)

    def with_head_dim(self, d: int) -> "KVCacheBuilder":
        return self._set("head_dim", d)

    def with_bit_width(self, inlier, outlier=None) -> "KVCacheBuilder":
        """``inlier``: an int, or a list with one entry per attention layer (then only
        :meth:`for_model` can consume the configuration)."""
        self._set("bit_width_inlier", inlier)
        return self._set("bit_width_outlier", outlier)

    def with_bits(self, inlier) -> "KVCacheBuilder":
        return self._set("bit_width_inlier", inlier)

    def with_seed(self, seed: int) -> "KVCacheBuilder":
        return self._set("seed", seed)

    def with_precision(self, dtype) -> "KVCacheBuilder":
        return self._set("dtype", dtype)

    def with_capacity(self, max_tokens: int) -> "KVCacheBuilder":
        return self._set("capacity", max_tokens)

    def with_observer(self, observer) -> "KVCacheBuilder":
        self._config.observers.append(observer)
        return self

    def with_sliding_window(self, window_size: int) -> "KVCacheBuilder":
        return self._set("sliding_window", window_size)

    def build(self):
        cfg = self._config
        d = cfg.head_dim
        if not (d >= 1 and (d & (d - 1)) == 0):
            raise QuantizerConfigError(f"KVCacheBuilder: head_dim={d} must be a power of 2.")
        if isinstance(cfg.bit_width_inlier, list):
            if not cfg.bit_width_inlier:
                raise QuantizerConfigError("KVCacheBuilder: bit_width_inlier list must not be empty.")
            if not all(isinstance(b, int) and b >= 1 for b in cfg.bit_width_inlier):
                raise QuantizerConfigError("KVCacheBuilder: every element of bit_width_inlier must be an int >= 1.")
        elif cfg.bit_width_inlier < 1:
            raise QuantizerConfigError(f"KVCacheBuilder: bit_width_inlier={cfg.bit_width_inlier} must be >= 1.")
        return KVCacheFactory.create(cfg)

    @staticmethod
    def for_layers(n_layers: int, config: KVCacheConfig, head_dims=None) -> list:
        """One cache per attention layer with ``seed + i`` and the layer's own bit-width
        (list-form ``bit_width_inlier``) and head_dim, as ``for_model`` does per layer."""
        caches = []
        bits = config.bit_width_inlier
        if isinstance(bits, list) and len(bits) != n_layers:
            raise QuantizerConfigError(
                f"KVCacheBuilder.for_model: bit_width_inlier list has {len(bits)} entries for {n_layers} layers")
        for i in range(n_layers):
            changes = {"seed": config.seed + i}
            if isinstance(bits, list):
                changes["bit_width_inlier"] = int(bits[i])
            if head_dims is not None:
                changes["head_dim"] = int(head_dims[i])
            caches.append(KVCacheFactory.create(dataclasses.replace(config, **changes)))
        return caches

    @staticmethod
    def for_model(model: Any, config: KVCacheConfig) -> list:
        """One cache per layer of ``model`` (``cache/base.py:1242-1433``): ``model.layers`` or
        ``model.model.layers``; a layer's head_dim comes from its ``self_attn`` / ``attn`` module, else
        from ``model.args`` (``model.config`` for a Transformers model): ``head_dim`` or
        ``hidden_size // num_attention_heads``; seeds are ``config.seed + layer index``; a list-form
        ``bit_width_inlier`` is spread over the attention layers. A layer without attention gets the
        slot of the model's own ``make_cache()`` (looked up on the class, so a patched instance hook is
        not called back) or a :class:`DenseKVCache`. A model that only carries
        ``config.num_hidden_layers`` gets that many caches of ``config`` as it stands."""
        layers = getattr(model, "layers", None) or getattr(getattr(model, "model", None), "layers", None)
        if layers is None:
            if hasattr(model, "config") and hasattr(model.config, "num_hidden_layers"):
                return KVCacheBuilder.for_layers(int(model.config.num_hidden_layers), config)
            raise QuantizerConfigError("KVCacheBuilder.for_model: cannot find the model's layers")
        native: list = []
        native_fn = None
        for klass in type(model).__mro__:
            candidate = klass.__dict__.get("make_cache")
            if candidate is not None:
                native_fn = candidate.__get__(model, type(model))
                break
        if callable(native_fn):
            try:
                built = native_fn()
                if isinstance(built, list) and len(built) == len(layers):
                    native = built
            except Exception as exc:
                warnings.warn(
                    f"KVCacheBuilder.for_model: {type(model).__name__}.make_cache() "
                    f"raised {type(exc).__name__}: {exc}. Falling back to a plain "
                    f"KVCache for any unquantized layer; recurrent/linear-attention "
                    f"layers on this model may not behave correctly.",
                    stacklevel=2,
                )
                native = []
        args = getattr(model, "args", None)
        if args is None:
            args = getattr(model, "config", None)
        if args is not None and not hasattr(args, "hidden_size"):
            lm = getattr(model, "language_model", None)
            if lm is not None:
                args = getattr(lm, "args", args)
        b_spec = config.bit_width_inlier
        if isinstance(b_spec, list):
            n_attn = sum(1 for layer in layers
                         if (getattr(layer, "self_attn", None) or getattr(layer, "attn", None)) is not None)
            if len(b_spec) != n_attn:
                raise QuantizerConfigError(
                    f"KVCacheBuilder.for_model: bit_width_inlier is a list of "
                    f"length {len(b_spec)}, but model has {n_attn} attention "
                    f"layers. The list must have one entry per attention layer.")
        caches = []
        attn_idx = 0
        for i, layer in enumerate(layers):
            hd = _resolve_head_dim(layer, args)
            if hd is None:
                caches.append(native[i] if i < len(native) else DenseKVCache())
                continue
            layer_b = b_spec[attn_idx] if isinstance(b_spec, list) else b_spec
            caches.append(KVCacheFactory.create(dataclasses.replace(config, head_dim=hd, bit_width_inlier=layer_b,
                                                                    seed=config.seed + i)))
            attn_idx += 1
        return caches


def _resolve_head_dim(layer: Any, args: Any):
    """A layer's attention head_dim, or ``None`` for a layer without attention
    (``cache/base.py:455-470``)."""
    attn = getattr(layer, "self_attn", None) or getattr(layer, "attn", None)
    if attn is None:
        return None
    hd = getattr(attn, "head_dim", None)
    if hd is None and args is not None:
        hd = getattr(args, "head_dim", None) or (args.hidden_size // args.num_attention_heads)
    return hd


class DenseKVCache:
    """Uncompressed keys and values for a layer this package does not quantize: the counterpart of
    the plain container the reference hands such layers (``cache/base.py:1284-1330``). Buffers grow
    in steps of 256 rows; ``update_and_fetch`` returns views of the live rows."""

    step = 256

    def __init__(self) -> None:
        self.keys = self.values = None
        self.offset = 0

    def update_and_fetch(self, keys: torch.Tensor, values: torch.Tensor):
        S = keys.shape[2]
        prev = self.offset
        if self.keys is None or prev + S > self.keys.shape[2]:
            rows = -(-(self.step + S - 1) // self.step) * self.step

            def grown(buf, new):
                fresh = new.new_zeros((*new.shape[:2], rows, new.shape[3]))
                return fresh if buf is None else torch.cat([buf[:, :, :prev], fresh], dim=2)

            self.keys, self.values = grown(self.keys, keys), grown(self.values, values)
        self.offset = prev + S
        self.keys[:, :, prev:self.offset] = keys
        self.values[:, :, prev:self.offset] = values
        return self.keys[:, :, :self.offset], self.values[:, :, :self.offset]

    def trim(self, n: int) -> int:
        n = int(min(self.offset, max(n, 0)))
        self.offset -= n
        return n

    def is_trimmable(self) -> bool:
        return True

    def empty(self) -> bool:
        return self.keys is None

    def size(self) -> int:
        return self.offset

    def reset(self) -> None:
        self.keys = self.values = None
        self.offset = 0

    @property
    def state(self):
        if self.keys is None:
            return (None, None)
        return self.keys[:, :, :self.offset], self.values[:, :, :self.offset]

    @state.setter
    def state(self, v) -> None:
        self.keys, self.values = v
        self.offset = 0 if self.keys is None else self.keys.shape[2]

    @property
    def nbytes(self) -> int:
        if self.keys is None:
            return 0
        k, v = self.state
        return k.numel() * k.element_size() + v.numel() * v.element_size()


def _native_only(config, who: str) -> None:
    if getattr(config, "use_metal_kernels", None) is False:
        raise RuntimeError(
            f"{who}: use_metal_kernels=False asks for the pure-framework twin, which this package "
            "does not have (native sm_100a kernels only, no fallback)")
    if not kernels.kivi_available():
        raise RuntimeError(f"{who}: the native library or a CUDA device is not available")


# ----------------------------------------------------------------------------------------
# KIVI
# ----------------------------------------------------------------------------------------
def _paired_view(keys: torch.Tensor, values: torch.Tensor):
    """``[2, *keys.shape]`` view over both tensors if ``values`` is ``keys`` shifted by a fixed
    positive offset inside one storage (two slices of one buffer), else ``None``."""
    if keys.dtype != values.dtype or keys.stride() != values.stride() or keys.shape != values.shape:
        return None
    if keys.untyped_storage().data_ptr() != values.untyped_storage().data_ptr():
        return None
    delta = values.storage_offset() - keys.storage_offset()
    if delta <= 0:
        return None
    return torch.as_strided(keys, (2, *keys.shape), (delta, *keys.stride()), keys.storage_offset())


class KIVIKVCache(StandaloneProtocol):
    """Packed KIVI cache: per-channel keys, per-token values, fp residual window.

    Storage (grown geometrically): packed codes ``u8 [B,H,cap,D*sb/8]``, key params
    ``f32 [B,H,cap/g,D]``, value params ``f32 [B,H,cap,D/g]``, residual ``[B,H,2(R+g)+g.., D]``
    in the activation dtype: the live rows are ``[_res_lo, _res_lo + _n_res)``; a flush
    quantizes the oldest rows where they lie and advances ``_res_lo``, and the live rows move
    back to the front (one copy, into rows they do not overlap) only when the buffer's end is
    reached, so a decode step allocates nothing. Quantization policy = ``KIVIKVCache._quantization_boundary``
    of the reference (``cache/kivi_cache.py:206-225``): after each append, tokens older than
    ``residual_length`` are flushed in whole ``group_size`` blocks, so one-shot prefill and
    token-by-token decode quantize identical groups. Never exposes ``.bits``.
    """

    def __init__(self, config: Any) -> None:
        _native_only(config, "KIVIKVCache")
        self._head_dim = int(config.head_dim)
        b = config.bit_width_inlier
        if isinstance(b, list):
            raise QuantizerConfigError(
                "KIVIKVCache: bit_width_inlier must be a single int; "
                "per-layer lists are dispatched by KVCacheBuilder.for_model().")
        self._b = int(b)
        if not 1 <= self._b <= 8:
            raise QuantizerConfigError(f"KIVIKVCache: bit_width_inlier={self._b} must be in [1, 8].")
        self._group_size = int(getattr(config, "kivi_group_size", 32))
        if self._group_size < 1:
            raise QuantizerConfigError(f"KIVIKVCache: kivi_group_size={self._group_size} must be >= 1.")
        self._residual_length = int(getattr(config, "residual_length", 128))
        self._levels = (1 << self._b) - 1
        self._sb = kernels.storage_bits(self._b)
        if (self._head_dim * self._sb) % 8:
            raise QuantizerConfigError("KIVIKVCache: head_dim * storage bits must be a multiple of 8")
        self._eps = 1e-8
        self._memory_bound = bool(getattr(config, "fused_sdpa_memory_bound", False))
        # `capacity` (tokens) pre-sizes the packed store at its first allocation, so that a serving
        # loop of known maximum length never reallocates; the store still doubles beyond it
        cap_hint = getattr(config, "capacity", None)
        self._capacity_hint = int(cap_hint) if cap_hint else 0
        self.offset = 0
        self._n_quantized = 0
        self._n_res = 0
        self._res_lo = 0
        self._cap = 0
        self._k_codes = self._v_codes = None
        self._k_scale = self._k_zero = self._v_scale = self._v_zero = None
        self._kv_res = self._k_res = self._v_res = None
        self._shape_bhd = (1, 1, self._head_dim)
        self._dtype = None
        # Host fast paths of the decode loop: the argument structure of the last attention call
        # and the layout of the last single-token append, reused while nothing they describe has
        # changed (`_version` moves whenever a buffer is replaced).
        self._version = 0
        self._just_flushed = False
        self._attend_plan = None
        self._append_plan = None
        self._quant_args = None
        self._sentinel = None
        # byte accounting (same definitions as the reference's properties)
        self._key_bytes_compressed = 0
        self._value_bytes_compressed = 0
        self._key_bytes_fp16 = 0
        self._value_bytes_fp16 = 0
        self._residual_fp16_bytes = 0
        self._tokens_seen = 0

    # -- policy ------------------------------------------------------------------------
    def _quantization_boundary(self) -> int:
        aged = max(0, self.offset - self._residual_length)
        return (aged // self._group_size) * self._group_size

    # -- storage -----------------------------------------------------------------------
    def _ensure_capacity(self, B, H, D, n_tokens, device, dtype) -> None:
        g = self._group_size
        if self._k_codes is not None and n_tokens <= self._cap:
            return
        new_cap = max(256, self._cap, self._capacity_hint)
        while new_cap < n_tokens:
            new_cap *= 2
        new_cap = ((new_cap + g - 1) // g) * g
        rb = D * self._sb // 8
        gv = (D + g - 1) // g

        def grow(old, shape, dt):
            t = torch.empty(shape, dtype=dt, device=device)
            if old is not None and old.shape[2] > 0:
                t[:, :, : old.shape[2]] = old
            return t

        self._k_codes = grow(self._k_codes, (B, H, new_cap, rb), torch.uint8)
        self._v_codes = grow(self._v_codes, (B, H, new_cap, rb), torch.uint8)
        self._k_scale = grow(self._k_scale, (B, H, new_cap // g, D), torch.float32)
        self._k_zero = grow(self._k_zero, (B, H, new_cap // g, D), torch.float32)
        self._v_scale = grow(self._v_scale, (B, H, new_cap, gv), torch.float32)
        self._v_zero = grow(self._v_zero, (B, H, new_cap, gv), torch.float32)
        self._cap = new_cap
        self._version += 1

    def _ensure_residual(self, B, H, D, n, device, dtype) -> None:
        """Room for ``n`` live rows starting at row 0 (a larger buffer is allocated, and the
        live rows are moved to its front, only when ``n`` exceeds the capacity)."""
        if self._k_res is not None and self._k_res.shape[2] >= n:
            return
        cap = max(2 * (self._residual_length + self._group_size) + self._group_size, n)
        # one allocation for both, so that a K/V pair that arrives as two slices of one tensor
        # (a fused QKV projection's output) is appended by a single copy
        kv = torch.empty((2, B, H, cap, D), dtype=dtype, device=device)
        if self._kv_res is not None and self._n_res:
            kv[:, :, :, : self._n_res] = self._kv_res[:, :, :, self._res_lo : self._res_lo + self._n_res]
        self._kv_res, self._k_res, self._v_res = kv, kv[0], kv[1]
        self._res_lo = 0
        self._version += 1

    def _make_room(self, B, H, D, S, device, dtype) -> None:
        """Make rows ``[_res_lo + _n_res, +S)`` of the residual buffer exist."""
        if self._k_res is None or self._n_res + S > self._k_res.shape[2]:
            self._ensure_residual(B, H, D, self._n_res + S, device, dtype)
        elif self._res_lo + self._n_res + S > self._k_res.shape[2]:
            lo, n = self._res_lo, self._n_res
            if n:
                if lo >= n:   # disjoint rows: a plain copy, nothing allocated
                    self._kv_res[:, :, :, :n] = self._kv_res[:, :, :, lo : lo + n]
                else:
                    self._kv_res[:, :, :, :n] = self._kv_res[:, :, :, lo : lo + n].clone()
            self._res_lo = 0

    def _store_block(self, keys, values, S, overlap=False) -> None:
        at = self._res_lo + self._n_res
        if not kernels.kivi_append(keys, values, self._k_res, self._v_res, at, overlap):
            pair = _paired_view(keys, values)
            if pair is not None:
                self._kv_res[:, :, :, at : at + S] = pair
            else:
                self._k_res[:, :, at : at + S] = keys
                self._v_res[:, :, at : at + S] = values
        self._n_res += S

    def _quantize_rows(self, src_k, src_v, n_flush) -> None:
        g = self._group_size
        B, H, _, D = src_k.shape
        s0, s1, s2, s3 = src_k.stride()
        if (src_k.is_cuda and src_k.dtype is src_v.dtype and src_k.shape == src_v.shape and src_v.stride() == (s0, s1, s2, s3)
                and s3 == 1 and s2 == D and (B == 1 or s0 == H * s1) and n_flush > 0
                and self._n_quantized + n_flush <= self._cap and self._n_quantized % g == 0):
            # Evenly spaced (batch, head) slabs of whole rows, into this cache's own buffers: the two
            # launches go straight to the library with argument blocks kept from the last flush
            # (what kernels.kivi_quantize_into would check about the destination holds by construction).
            qa = self._quant_args
            if qa is None or qa[0] != self._version:
                rb, gv = D * self._sb // 8, (D + g - 1) // g
                common = dict(n_bh=B * H, head_dim=D, levels=self._levels, store_bits=self._sb, group=g, eps=self._eps,
                              codes_stride_bh=self._cap * rb, recon=None, recon_stride_bh=0)
                qa = self._quant_args = (self._version, _lib.KiviQuantArgs(axis=0, param_stride_bh=(self._cap // g) * D, **common),
                                         _lib.KiviQuantArgs(axis=1, param_stride_bh=self._cap * gv, **common), rb, gv)
            _, ak, av, rb, gv = qa
            nq = self._n_quantized
            stride_bh = s1 if H > 1 else (s0 if B > 1 else src_k.shape[2] * D)
            dt = _lib.dtype_code(src_k.dtype)
            ak.x, ak.dtype, ak.n_tok, ak.x_stride_bh = src_k.data_ptr(), dt, n_flush, stride_bh
            ak.codes = self._k_codes.data_ptr() + nq * rb
            ak.scale = self._k_scale.data_ptr() + 4 * (nq // g) * D
            ak.zero = self._k_zero.data_ptr() + 4 * (nq // g) * D
            av.x, av.dtype, av.n_tok, av.x_stride_bh = src_v.data_ptr(), dt, n_flush, stride_bh
            av.codes = self._v_codes.data_ptr() + nq * rb
            av.scale = self._v_scale.data_ptr() + 4 * nq * gv
            av.zero = self._v_zero.data_ptr() + 4 * nq * gv
            lib, st = _lib.lib(), _lib.stream_ptr(src_k.device)
            with _lib.on_device(src_k.device):
                _lib.check(lib.vq_kivi_quantize_pack(C.byref(ak), st), "KIVIKVCache: quantize keys")
                _lib.check(lib.vq_kivi_quantize_pack(C.byref(av), st), "KIVIKVCache: quantize values")
            return
        kernels.kivi_quantize_into(src_k[:, :, :n_flush], -2, g, self._b, codes=self._k_codes,
                                   scale=self._k_scale, zero=self._k_zero, tok_offset=self._n_quantized,
                                   store_bits=self._sb, eps=self._eps)
        kernels.kivi_quantize_into(src_v[:, :, :n_flush], -1, g, self._b, codes=self._v_codes,
                                   scale=self._v_scale, zero=self._v_zero, tok_offset=self._n_quantized,
                                   store_bits=self._sb, eps=self._eps)

    # -- protocol ----------------------------------------------------------------------
    def update_and_fetch(self, keys: torch.Tensor, values: torch.Tensor, *, overlap_previous: bool = False):
        """Append ``keys/values [B,H,S,D]``; flush aged whole groups into the packed store.

        ``overlap_previous=True`` (an addition to the reference's protocol): the copy of a block
        that flushes nothing may start under the preceding work on the stream, so that a decode
        loop ``update_and_fetch -> fused_sdpa(overlap_previous=True)`` per layer streams from one
        layer into the next. Only pass it when ``keys`` / ``values`` are not produced by the kernels
        right before this call. A call that flushes a group ignores it, and so does the attention
        call that follows the flush."""
        ap = self._append_plan
        if (ap is not None and ap[0] == self._version and keys.shape == ap[1] and values.shape == ap[1]
                and keys.dtype is ap[2] and values.dtype is ap[2] and (self.offset + 1 - self._residual_length) % self._group_size
                and self._res_lo + self._n_res < ap[3] and keys.is_contiguous() and values.is_contiguous()
                and not (keys.data_ptr() | values.data_ptr()) & 15 and torch.cuda.current_device() == ap[9].index):
            # One token, no group ages out, room behind the live rows, same layout as last time:
            # straight to the copy kernel (the checks of the general path below were made then).
            _, shape, _, _, n_bh, res_stride, dt, k_ptr, v_ptr, dev = ap
            _lib.check(_lib.lib().vq_kivi_append(keys.data_ptr(), values.data_ptr(), shape[3], k_ptr, v_ptr, res_stride, n_bh, 1,
                                                 self._res_lo + self._n_res, shape[3], dt,
                                                 _lib.VQ_ATTEND_OVERLAP_PREVIOUS if overlap_previous else 0, _lib.stream_ptr(dev)),
                       "KIVIKVCache.update_and_fetch")
            self.offset += 1
            self._n_res += 1
            self._account_bytes(shape[0], shape[1], 1, shape[3], 0)
            if self._memory_bound:
                return self._sentinel, self._sentinel
            return self._materialize()
        if keys.ndim != 4 or keys.shape != values.shape:
            raise ValueError(f"KIVIKVCache.update_and_fetch: keys/values must be equal 4D shapes, got "
                             f"{tuple(keys.shape)} / {tuple(values.shape)}")
        B, H, S, D = keys.shape
        if D != self._head_dim:
            raise QuantizerConfigError(f"KIVIKVCache: expected head_dim {self._head_dim}, got {D}.")
        if self._dtype is None:
            self._dtype = keys.dtype
        self._shape_bhd = (B, H, D)
        dev = keys.device
        self.offset += S
        new_boundary = self._quantization_boundary()
        n_flush = new_boundary - self._n_quantized
        self._just_flushed = n_flush > 0
        if n_flush <= 0:
            self._make_room(B, H, D, S, dev, keys.dtype)
            self._store_block(keys, values, S, overlap_previous)
        elif self._n_res == 0:
            # A (prefill) block onto an empty residual: its head is quantized straight from the
            # caller's tensor, only its tail is copied into the residual buffer.
            self._ensure_capacity(B, H, D, new_boundary, dev, keys.dtype)
            self._quantize_rows(keys, values, n_flush)
            self._n_quantized = new_boundary
            keep = S - n_flush
            self._res_lo = 0
            self._ensure_residual(B, H, D, keep, dev, keys.dtype)
            if keep > 0:
                self._store_block(keys[:, :, n_flush:], values[:, :, n_flush:], keep)
        elif S <= self._residual_length + self._group_size:
            # Decode: the rows to flush are the oldest unquantized rows. The block is stored behind
            # the live rows, then the aged rows are quantized where they lie and the window's
            # start moves on: no concatenation, no shifting, no allocation.
            self._make_room(B, H, D, S, dev, keys.dtype)
            self._store_block(keys, values, S)
            self._ensure_capacity(B, H, D, new_boundary, dev, keys.dtype)
            lo = self._res_lo
            self._quantize_rows(self._k_res[:, :, lo : lo + n_flush], self._v_res[:, :, lo : lo + n_flush], n_flush)
            self._res_lo += n_flush
            self._n_res -= n_flush
            self._n_quantized = new_boundary
        else:
            # A long block onto a non-empty residual: the rows to flush span both.
            lo = self._res_lo
            src_k = torch.cat([self._k_res[:, :, lo : lo + self._n_res], keys], dim=2)
            src_v = torch.cat([self._v_res[:, :, lo : lo + self._n_res], values], dim=2)
            self._ensure_capacity(B, H, D, new_boundary, dev, keys.dtype)
            self._quantize_rows(src_k, src_v, n_flush)
            keep = src_k.shape[2] - n_flush
            self._n_res = 0
            self._res_lo = 0
            self._ensure_residual(B, H, D, keep, dev, keys.dtype)
            if keep > 0:
                self._store_block(src_k[:, :, n_flush:], src_v[:, :, n_flush:], keep)
            self._n_quantized = new_boundary
        self._account_bytes(B, H, S, D, max(n_flush, 0))
        if (S == 1 and keys.dtype is self._k_res.dtype and keys.is_cuda and (D * keys.element_size()) % 16 == 0
                and torch.cuda.current_device() == keys.device.index):
            es = keys.element_size()
            self._append_plan = (self._version, keys.shape, keys.dtype, self._k_res.shape[2], B * H,
                                 self._k_res.shape[2] * D, _lib.dtype_code(keys.dtype), self._k_res.data_ptr(),
                                 self._v_res.data_ptr(), keys.device)
            assert (self._k_res.shape[2] * D * es) % 16 == 0
        if self._memory_bound:
            if self._sentinel is None or self._sentinel.shape != (B, H, 0, D) or self._sentinel.dtype != keys.dtype:
                self._sentinel = keys.new_zeros((B, H, 0, D))
            return self._sentinel, self._sentinel
        return self._materialize()

    def _live_res(self):
        lo = self._res_lo
        return self._k_res[:, :, lo : lo + self._n_res], self._v_res[:, :, lo : lo + self._n_res]

    def _materialize(self):
        """The reference cache's view: round-tripped quantized rows, then the exact tail."""
        B, H, D = self._shape_bhd
        nq = self._n_quantized
        parts_k, parts_v = [], []
        if nq:
            g = self._group_size
            kq = kernels.scalar_decode_once(self._k_codes[:, :, :nq].contiguous(), self._k_scale[:, :, : nq // g].contiguous(),
                                            self._k_zero[:, :, : nq // g].contiguous(), g, "K", store_bits=self._sb,
                                            out_dtype=self._dtype)
            vq = kernels.scalar_decode_once(self._v_codes[:, :, :nq].contiguous(), self._v_scale[:, :, :nq].contiguous(),
                                            self._v_zero[:, :, :nq].contiguous(), g, "V", store_bits=self._sb,
                                            out_dtype=self._dtype)
            parts_k.append(kq)
            parts_v.append(vq)
        kr, vr = self._live_res()
        parts_k.append(kr)
        parts_v.append(vr)
        return torch.cat(parts_k, dim=2), torch.cat(parts_v, dim=2)

    def fused_sdpa(self, q: torch.Tensor, scale: float, *, causal: bool = True, sliding_window: int = 0,
                   out: torch.Tensor | None = None, overlap_previous: bool = False, gather=None) -> torch.Tensor:
        """Attention of ``q [B,H_q,S_q,D]`` over the packed store + residual, no dequantized
        copy of the history. With ``causal=True`` query row ``r`` of ``S_q`` sits at position
        ``offset - S_q + r`` and sees the slots up to its own (the tail-aligned mask of the
        reference's ``metal_fused_sdpa``, ``metal/fused_sdpa.py:200-299``); ``causal=False``
        lets every row see every slot, as the reference's ``scalar_fused_decode_attend`` does.

        ``overlap_previous`` / ``gather``: see :func:`kernels.kivi_decode_attend`."""
        plan = self._attend_plan
        if (plan is not None and out is not None and plan[0] == self._version and q.data_ptr() == plan[1]
                and out.data_ptr() == plan[2] and q.shape == plan[3] and q.dtype is plan[4] and out.dtype is plan[5]
                and out.shape == plan[3] and gather is plan[6] and not sliding_window and self._n_quantized > 0
                and torch.cuda.current_device() == plan[7]):
            # Same query / output buffers and cache buffers as the last call: only the counters,
            # the residual window's start and the flags are new.
            a, row_bytes, k_res_ptr, v_res_ptr, need = plan[8], plan[9], plan[10], plan[11], plan[12]
            lib = _lib.lib()
            a.n_quant, a.n_res, a.scale = self._n_quantized, self._n_res, scale
            a.flags = _lib.VQ_ATTEND_OVERLAP_PREVIOUS if overlap_previous else 0
            a.k_res = k_res_ptr + self._res_lo * row_bytes
            a.v_res = v_res_ptr + self._res_lo * row_bytes
            a.n_splits = 0
            key = (self._n_quantized, a.flags)
            if need[0] != key:
                need[0], need[1] = key, lib.vq_kivi_attend_workspace_bytes(C.byref(a))
            if self._just_flushed:
                # right after a flush the packed store was written by the kernels just before this
                # call: a plain launch, with the split plan (= summation order) the caller asked for
                if a.flags:
                    a.n_splits, a.flags = lib.vq_kivi_attend_splits(C.byref(a)), 0
                self._just_flushed = False
            ws = kernels._workspace(q.device, need[1])
            a.workspace, a.workspace_bytes = ws.data_ptr(), ws.numel()
            _lib.check(lib.vq_kivi_decode_attend(C.byref(a), _lib.stream_ptr(q.device)), "KIVIKVCache.fused_sdpa")
            return out
        if q.ndim != 4:
            raise ValueError(f"KIVIKVCache.fused_sdpa: q must be 4D, got {tuple(q.shape)}")
        if sliding_window:
            raise ValueError("KIVIKVCache.fused_sdpa: sliding_window is not supported")
        if self.offset == 0:
            raise RuntimeError("KIVIKVCache.fused_sdpa: the cache is empty")
        if q.shape[2] > self.offset and causal:
            raise ValueError(f"KIVIKVCache.fused_sdpa: {q.shape[2]} query rows but only {self.offset} cached tokens")
        has_q = self._n_quantized > 0
        plain_after_flush = bool(overlap_previous) and self._just_flushed
        self._just_flushed = False
        want_plan = (out is not None and has_q and self._n_res > 0 and q.shape[2] == 1 and q.is_contiguous()
                     and torch.cuda.current_device() == q.device.index)
        keep = [] if want_plan else None
        res = kernels.kivi_decode_attend(
            q, self._k_codes if has_q else None, self._k_scale, self._k_zero,
            self._v_codes if has_q else None, self._v_scale, self._v_zero, self._group_size, scale,
            store_bits=self._sb, n_quant=self._n_quantized,
            k_res=self._k_res if self._n_res else None, v_res=self._v_res if self._n_res else None,
            n_res=self._n_res, res_offset=self._res_lo, out=out, causal=bool(causal) and q.shape[2] > 1,
            overlap_previous=overlap_previous, gather=gather, sinks=self._attend_sinks() if has_q and q.shape[2] == 1 else None,
            _keep_args=keep, _plain_launch=plain_after_flush, _fn="KIVIKVCache.fused_sdpa")
        if want_plan and keep:
            # the validated argument structure, for the next call with the same buffers
            self._attend_plan = (self._version, q.data_ptr(), out.data_ptr(), q.shape, q.dtype, out.dtype, gather,
                                 q.device.index, keep[0], self._head_dim * self._k_res.element_size(),
                                 self._k_res.data_ptr(), self._v_res.data_ptr(), [None, 0])
        return res

    def _attend_sinks(self):
        """Protected tokens for the attention call (none in plain KIVI; see ``cache_sink``)."""
        return None

    def check_status(self) -> None:
        """Raise if a device-side bounded wait of an earlier attention call ran out (its output
        was then invalid). Synchronises the device; call it where a silent wrong result is not
        acceptable, e.g. once per decode step."""
        kernels.attend_status()

    # -- trim / state ------------------------------------------------------------------
    def trim(self, n: int) -> int:
        """Drop the last ``n`` tokens. The quantized frontier snaps DOWN to a group multiple;
        rows of a partly trimmed group return to the residual as their once-rounded values,
        so the next flush re-quantizes exactly what the reference's fp16 buffer would hold
        (``cache/kivi_cache.py:264-299``)."""
        n = int(min(max(n, 0), self.offset))
        if n == 0:
            return 0
        new_offset = self.offset - n
        g = self._group_size
        old_nq = self._n_quantized
        if new_offset >= old_nq:
            self._n_res -= n
            n_rolled = 0
        else:
            new_nq = (new_offset // g) * g
            n_rolled = old_nq - new_nq
            keep = new_offset - new_nq
            B, H, D = self._shape_bhd
            if keep > 0:
                lo_g, hi_g = new_nq // g, (new_offset + g - 1) // g
                kq = kernels.scalar_decode_once(self._k_codes[:, :, new_nq : hi_g * g].contiguous(),
                                                self._k_scale[:, :, lo_g:hi_g].contiguous(),
                                                self._k_zero[:, :, lo_g:hi_g].contiguous(), g, "K",
                                                store_bits=self._sb, out_dtype=self._dtype)
                vq = kernels.scalar_decode_once(self._v_codes[:, :, new_nq : hi_g * g].contiguous(),
                                                self._v_scale[:, :, new_nq : hi_g * g].contiguous(),
                                                self._v_zero[:, :, new_nq : hi_g * g].contiguous(), g, "V",
                                                store_bits=self._sb, out_dtype=self._dtype)
                self._n_res = 0
                self._ensure_residual(B, H, D, keep, kq.device, self._dtype)
                self._k_res[:, :, :keep] = kq[:, :, :keep]
                self._v_res[:, :, :keep] = vq[:, :, :keep]
            self._res_lo = 0
            self._n_res = keep
            self._n_quantized = new_nq
        self.offset = new_offset
        self._rollback_bytes(n, n_rolled)
        return n

    def is_trimmable(self) -> bool:
        return True

    def empty(self) -> bool:
        return self.offset == 0

    def size(self) -> int:
        return self.offset

    def _reset_tokens(self) -> None:
        """Forget every token; buffers, bit-width and group size stay (``KVCache.reset``)."""
        self.offset = self._n_quantized = self._n_res = self._res_lo = 0
        self._key_bytes_compressed = self._value_bytes_compressed = 0
        self._key_bytes_fp16 = self._value_bytes_fp16 = self._residual_fp16_bytes = self._tokens_seen = 0

    @property
    def state(self):
        """Live rows of every buffer plus the counters (checkpoint / prompt-cache reuse)."""
        nq, g = self._n_quantized, self._group_size
        if self._k_res is None:
            return ()
        pk = lambda t, n: None if t is None else t[:, :, :n].contiguous()  # noqa: E731
        return (pk(self._k_codes, nq), pk(self._k_scale, nq // g), pk(self._k_zero, nq // g),
                pk(self._v_codes, nq), pk(self._v_scale, nq), pk(self._v_zero, nq),
                *(t.contiguous() for t in self._live_res()),
                torch.tensor([self.offset, nq, self._n_res]))

    @state.setter
    def state(self, st) -> None:
        if not st:
            return
        kc, ks, kz, vc, vs, vz, kr, vr, counters = st
        self.offset, nq, n_res = (int(x) for x in counters.tolist())
        B, H, _, D = kr.shape
        self._shape_bhd, self._dtype = (B, H, D), kr.dtype
        self._k_codes = self._v_codes = None
        self._k_scale = self._k_zero = self._v_scale = self._v_zero = None
        self._cap = 0
        if nq:
            self._ensure_capacity(B, H, D, nq, kr.device, kr.dtype)
            g = self._group_size
            self._k_codes[:, :, :nq], self._v_codes[:, :, :nq] = kc, vc
            self._k_scale[:, :, : nq // g], self._k_zero[:, :, : nq // g] = ks, kz
            self._v_scale[:, :, :nq], self._v_zero[:, :, :nq] = vs, vz
        self._n_quantized = nq
        self._kv_res = self._k_res = self._v_res = None
        self._n_res = 0
        self._res_lo = 0
        self._ensure_residual(B, H, D, n_res, kr.device, kr.dtype)
        self._k_res[:, :, :n_res], self._v_res[:, :, :n_res] = kr, vr
        self._n_res = n_res

    @property
    def meta_state(self):
        """What ``state`` does not carry, as strings (the convention of the reference's caches,
        ``cache/turboquant_rvq_cache.py:396-405``): ``(head_dim, bits, group, residual_length,
        offset, n_quantized, n_residual)``."""
        return tuple(map(str, (self._head_dim, self._b, self._group_size, self._residual_length, self.offset,
                               self._n_quantized, self._n_res)))

    @meta_state.setter
    def meta_state(self, v) -> None:
        hd, b, g, r, off, nq, n_res = (int(x) for x in v)
        if not 1 <= b <= 8 or g < 1 or (hd * kernels.storage_bits(b)) % 8:
            raise QuantizerConfigError(f"KIVIKVCache.meta_state: unusable configuration {tuple(v)}")
        self._head_dim, self._b, self._group_size, self._residual_length = hd, b, g, r
        self._levels, self._sb = (1 << b) - 1, kernels.storage_bits(b)
        self.offset, self._n_quantized, self._n_res = off, nq, n_res
        if off == 0:
            self._reset_tokens()

    @classmethod
    def from_state(cls, state, meta_state=None, config=None):
        """A cache rebuilt from ``state`` and ``meta_state`` (``config`` supplies the flags that are
        neither: ``fused_sdpa_memory_bound``, ``capacity``)."""
        if meta_state is None:
            raise TypeError("KIVIKVCache.from_state() requires meta_state")
        hd, b, g, r = (int(x) for x in meta_state[:4])
        cfg = config if config is not None else KVCacheConfig(method="kivi")
        obj = cls(dataclasses.replace(cfg, method="kivi", head_dim=hd, bit_width_inlier=b, kivi_group_size=g, residual_length=r))
        obj.meta_state = meta_state
        obj.state = state
        return obj

    def merge(self, *a, **k):
        raise NotImplementedError("KIVIKVCache.merge: batched-cache merging is not supported")

    # -- accounting (reference: cache/kivi_cache.py:301-410) ---------------------------
    def _quantized_bytes(self, n, B, H, D):
        gs = self._group_size
        k = math.ceil(n * D * self._b / 8) * H * B + math.ceil(n / gs) * D * 2 * 2 * H * B
        v = math.ceil(n * D * self._b / 8) * H * B + n * math.ceil(D / gs) * 2 * 2 * H * B
        return k, v

    def _account_bytes(self, B, H, S, D, n_quant_now) -> None:
        if n_quant_now > 0:
            k, v = self._quantized_bytes(n_quant_now, B, H, D)
            self._key_bytes_compressed += k
            self._value_bytes_compressed += v
        self._residual_fp16_bytes = (self.offset - self._n_quantized) * D * 2 * 2 * H * B
        self._key_bytes_fp16 += H * B * S * D * 2
        self._value_bytes_fp16 += H * B * S * D * 2
        self._tokens_seen += S

    def _rollback_bytes(self, n_tokens, n_rolled) -> None:
        B, H, D = self._shape_bhd
        if n_rolled > 0:
            k, v = self._quantized_bytes(n_rolled, B, H, D)
            self._key_bytes_compressed = max(0, self._key_bytes_compressed - k)
            self._value_bytes_compressed = max(0, self._value_bytes_compressed - v)
        self._key_bytes_fp16 = max(0, self._key_bytes_fp16 - H * B * n_tokens * D * 2)
        self._value_bytes_fp16 = max(0, self._value_bytes_fp16 - H * B * n_tokens * D * 2)
        self._tokens_seen = max(0, self._tokens_seen - n_tokens)
        self._residual_fp16_bytes = (self.offset - self._n_quantized) * D * 2 * 2 * H * B

    @property
    def compressed_key_bytes(self) -> int:
        return self._key_bytes_compressed

    @property
    def compressed_value_bytes(self) -> int:
        return self._value_bytes_compressed

    @property
    def fp16_key_bytes(self) -> int:
        return self._key_bytes_fp16

    @property
    def fp16_value_bytes(self) -> int:
        return self._value_bytes_fp16

    @property
    def residual_fp16_bytes(self) -> int:
        return self._residual_fp16_bytes

    @property
    def assigned_avg_bits(self) -> float:
        return float(self._b)

    @property
    def effective_compression_ratio(self) -> float:
        total_fp16 = self._key_bytes_fp16 + self._value_bytes_fp16
        if total_fp16 == 0:
            return 1.0
        total = self._key_bytes_compressed + self._value_bytes_compressed + self._residual_fp16_bytes
        return total_fp16 / total if total else 1.0

    @property
    def nbytes(self) -> int:
        """True live footprint: packed codes + fp32 params of quantized rows + residual rows."""
        B, H, D = self._shape_bhd
        nq, g = self._n_quantized, self._group_size
        rb = D * self._sb // 8
        packed = 2 * nq * rb + (nq // g) * D * 8 + nq * ((D + g - 1) // g) * 8
        esz = 2 if self._dtype in (None, torch.float16, torch.bfloat16) else 4
        return B * H * (packed + 2 * self._n_res * D * esz)


_CACHE_CLASS_BY_METHOD["kivi"] = KIVIKVCache

from .cache_coded import RaBitQKVCache, VecInferKVCache  # noqa: E402  (registers "vecinfer", "rabitq")
from .cache_sink import SinkProtectedKVCache  # noqa: E402  (registers "kivi_sink")
from .cache_rvq import TurboQuantRVQKVCache  # noqa: E402  (registers "turboquant_rvq")
from .cache_skvq import SKVQKVCache  # noqa: E402  (registers "skvq")
from .cache_kitty import AgeTieredKVCache, KittyKVCache  # noqa: E402  (registers "kitty", "age_tiered")

__all__ = ["QuantizerConfigError", "VecInferOptions", "KIVIOptions", "SKVQOptions", "KVCacheConfig", "KVCacheFactory",
           "KVCacheBuilder", "DenseKVCache", "KIVIKVCache", "SinkProtectedKVCache", "TurboQuantRVQKVCache", "SKVQKVCache", "KittyKVCache",
           "AgeTieredKVCache", "KittyOptions", "AgeTieredKVOptions", "VecInferKVCache",
           "RaBitQKVCache", "KVCache", "EncodedVector"]
