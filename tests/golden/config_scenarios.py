"""Configuration scenarios run against BOTH the reference's ``cache/base.py`` (by make_golden.py, over
stand-ins for ``mlx_lm`` and the cache modules) and this package's ``cache.py`` (by
tests/test_cache_config.py): each returns a JSON-able record of what the configuration layer did
(field values, warnings, errors), so the two can be compared entry by entry."""

import dataclasses
import warnings

SHARED_FIELDS = ["method", "head_dim", "bit_width_inlier", "bit_width_outlier", "seed", "sliding_window", "key_sub_dim",
                 "value_sub_dim", "key_codebook_bits", "value_codebook_bits", "residual_length", "kivi_group_size",
                 "fused_sdpa", "fused_sdpa_max_ctx", "fused_sdpa_memory_bound", "n_sink_tokens", "skvq_bits_key",
                 "skvq_bits_value", "skvq_group_size", "skvq_window", "skvq_n_sink", "skvq_reorder", "skvq_clip_search",
                 "skvq_clip_alpha", "skvq_max_ctx", "kitty_hi_fraction", "kitty_hi_bit", "kitty_lo_bit", "kitty_group_size",
                 "age_recent_boundary", "age_mid_boundary", "age_bits_recent", "age_bits_mid", "age_bits_old", "age_group_size"]


def _fields(cfg):
    return {name: getattr(cfg, name) for name in SHARED_FIELDS}


def _record(fn):
    """Run ``fn``; report its result, the warnings it raised (category + the part of the message
    that names the field / method) and the exception (type name + first 60 characters, without the
    list of registered methods)."""
    with warnings.catch_warnings(record=True) as w:
        warnings.simplefilter("always")
        try:
            result, error = fn(), None
        except Exception as e:  # noqa: BLE001
            result, error = None, [type(e).__name__, str(e).split(" Choices:")[0][:60]]
    warns = sorted([x.category.__name__, str(x.message).split(" is deprecated")[0].split(": only")[0][:80]] for x in w
                   if issubclass(x.category, (DeprecationWarning, UserWarning)) and "random N(0,1)" not in str(x.message))
    return {"result": result, "warnings": warns, "error": error}


def scenarios(ns):
    """``ns``: an object with ``KVCacheConfig``, ``KVCacheFactory``, ``VecInferOptions``, ``KIVIOptions``,
    ``SKVQOptions``, ``KittyOptions``, ``AgeTieredKVOptions``. Returns ``{name: record}``."""
    C, F = ns.KVCacheConfig, ns.KVCacheFactory
    out = {}
    out["defaults"] = _record(lambda: _fields(C()))
    out["repr"] = _record(lambda: repr(C(method="kivi", head_dim=64, bit_width_inlier=4, seed=7)))
    out["options_read_through_skvq"] = _record(lambda: _fields(C(method="skvq", options=ns.SKVQOptions(skvq_window=64, skvq_bits_key=2))))
    out["explicit_kwarg_wins"] = _record(lambda: _fields(C(method="skvq", skvq_window=128, options=ns.SKVQOptions(skvq_window=64))))
    out["options_vecinfer"] = _record(lambda: _fields(C(method="vecinfer", options=ns.VecInferOptions(key_sub_dim=8, residual_length=32))))
    out["options_kivi_group"] = _record(lambda: _fields(C(method="kivi", options=ns.KIVIOptions(kivi_group_size=64))))
    out["options_kitty"] = _record(lambda: _fields(C(method="kitty", options=ns.KittyOptions(kitty_hi_bit=8))))
    out["options_age"] = _record(lambda: _fields(C(method="age_tiered", options=ns.AgeTieredKVOptions(age_mid_boundary=256))))
    out["foreign_options_fill_their_fields"] = _record(lambda: _fields(C(method="kivi", options=ns.SKVQOptions(skvq_n_sink=1))))

    def set_flat():
        c = C(method="skvq")
        c.skvq_window = 5
        c.head_dim = 32          # not an options-owned field: silent
        return [c.skvq_window, c.head_dim]

    out["setattr_deprecation"] = _record(set_flat)
    out["inlier_bits_named_for_skvq"] = _record(lambda: _fields(C(method="skvq", bit_width_inlier=2))["bit_width_inlier"])
    out["inlier_bits_named_for_vecinfer"] = _record(lambda: C(method="vecinfer", bit_width_inlier=3).bit_width_inlier)
    out["inlier_bits_named_for_kivi"] = _record(lambda: C(method="kivi", bit_width_inlier=3).bit_width_inlier)
    out["replace_does_not_warn"] = _record(lambda: dataclasses.replace(C(method="kitty"), head_dim=64).head_dim)
    out["positional_method"] = _record(lambda: _fields(C("kivi_sink", 64))["head_dim"])
    out["factory_unknown_method"] = _record(lambda: F.create(C(method="no_such_method")))
    out["factory_list_bits"] = _record(lambda: F.create(C(method="kivi", bit_width_inlier=[2, 4])))
    out["factory_observers"] = _record(lambda: F.create(C(method="kivi", observers=[object()])))
    out["factory_outlier_bits"] = _record(lambda: F.create(C(method="kivi", bit_width_outlier=3)))
    return out


def construction_scenarios(ns):
    """Scenarios that construct a cache (this package needs a CUDA device for them)."""
    C, F = ns.KVCacheConfig, ns.KVCacheFactory
    out = {}
    out["factory_sliding_window_on_protocol_cache"] = _record(lambda: type(F.create(C(method="kivi", head_dim=32, sliding_window=16))).__name__)
    for method, kw in (("kivi", {}), ("kivi_sink", {}), ("skvq", {}), ("kitty", {}), ("age_tiered", {})):
        out[f"factory_{method}"] = _record(lambda m=method, k=kw: type(F.create(C(method=m, head_dim=32, **k))).__name__)
    for method, kw, tag in (("kivi_sink", {"n_sink_tokens": -1}, "negative_sinks"), ("skvq", {"skvq_window": 1}, "window_1"),
                            ("skvq", {"skvq_n_sink": 200}, "sinks_past_window"), ("skvq", {"skvq_bits_key": 0}, "bits_0"),
                            ("skvq", {"skvq_clip_alpha": 1.5}, "alpha"), ("kitty", {"kitty_hi_fraction": 2.0}, "hi_fraction"),
                            ("age_tiered", {"age_recent_boundary": 0}, "recent_0"),
                            ("age_tiered", {"age_recent_boundary": 64, "age_mid_boundary": 32}, "mid_below_recent"),
                            ("age_tiered", {"age_bits_mid": 17}, "bits_17"), ("kivi", {"bit_width_inlier": [2]}, "kivi_list")):
        out[f"factory_{method}_{tag}"] = _record(lambda m=method, k=kw: type(F.create(C(method=m, head_dim=32, **k))).__name__)
    return out


def _record_full(fn):
    """As :func:`_record`, with whole messages."""
    with warnings.catch_warnings(record=True) as w:
        warnings.simplefilter("always")
        try:
            result, error = fn(), None
        except Exception as e:  # noqa: BLE001
            result, error = None, [type(e).__name__, str(e)]
    return {"result": result, "warnings": sorted([x.category.__name__, str(x.message)] for x in w), "error": error}


class _Attn:
    def __init__(self, head_dim=None):
        if head_dim is not None:
            self.head_dim = head_dim


class _Layer:
    def __init__(self, kind="self_attn", head_dim=None):
        if kind is not None:
            setattr(self, kind, _Attn(head_dim))


class _Args:
    def __init__(self, **kw):
        self.__dict__.update(kw)


def builder_scenarios(ns):
    """``KVCacheBuilder.for_model`` over stand-in models (``ns`` also carries ``KVCacheBuilder`` and
    ``PlainCache``, the class handed to layers without attention). ``KVCacheFactory.create`` is replaced
    for the duration of a scenario by a recorder, so a record is the per-layer plan: for an attention
    layer ``[method, head_dim, bit width, seed]``, otherwise ``"plain"`` or the model's own slot."""
    C, F, Bld = ns.KVCacheConfig, ns.KVCacheFactory, ns.KVCacheBuilder

    def plan(model, cfg):
        original = F.create
        F.create = staticmethod(lambda c: ("cache", [c.method, c.head_dim, c.bit_width_inlier, c.seed]))
        try:
            caches = Bld.for_model(model, cfg)
        finally:
            F.create = staticmethod(original)
        return [c[1] if isinstance(c, tuple) else "plain" if isinstance(c, ns.PlainCache) else str(c) for c in caches]

    class Flat:                                    # layers on the model itself, per-layer head_dim
        def __init__(self):
            self.layers = [_Layer(head_dim=64), _Layer(head_dim=32), _Layer("attn", head_dim=16)]

    class Nested:                                  # model.model.layers, head_dim from the arguments
        def __init__(self, args, layers=None):
            self.model = _Args(layers=layers or [_Layer(), _Layer()])
            self.args = args

    class Hybrid:                                  # attention, recurrent, attention; the model offers its own slots
        def __init__(self):
            self.layers = [_Layer(head_dim=64), _Layer(None), _Layer(head_dim=64)]

        def make_cache(self):
            return ["slot0", "slot1", "slot2"]

    class HybridNoHook(Hybrid):
        make_cache = None

    class HybridShortHook(Hybrid):
        def make_cache(self):
            return ["slot0"]

    class HybridFailingHook(Hybrid):
        def make_cache(self):
            raise RuntimeError("no cache today")

    class Patched(Hybrid):                         # an instance attribute must not be called back
        def __init__(self):
            super().__init__()
            self.make_cache = lambda: 1 / 0

    class Wrapped:                                 # arguments without hidden_size: the language model's are used
        def __init__(self):
            self.layers = [_Layer(), _Layer()]
            self.args = _Args(model_type="wrapper")
            self.language_model = _Args(args=_Args(hidden_size=512, num_attention_heads=4))

    class EmptyOuter:                              # an empty outer list falls through to model.model.layers
        def __init__(self):
            self.layers = []
            self.model = _Args(layers=[_Layer(head_dim=8)])

    out = {}
    kivi = C(method="kivi", bit_width_inlier=4, seed=10)
    out["flat_per_layer_head_dim"] = _record_full(lambda: plan(Flat(), kivi))
    out["nested_hidden_over_heads"] = _record_full(lambda: plan(Nested(_Args(hidden_size=256, num_attention_heads=4)), kivi))
    out["nested_args_head_dim_wins"] = _record_full(lambda: plan(Nested(_Args(head_dim=32, hidden_size=256, num_attention_heads=4)), kivi))
    out["nested_layer_head_dim_wins"] = _record_full(
        lambda: plan(Nested(_Args(head_dim=32), [_Layer(head_dim=128), _Layer()]), kivi))
    out["hybrid_native_slot"] = _record_full(lambda: plan(Hybrid(), kivi))
    out["hybrid_no_hook"] = _record_full(lambda: plan(HybridNoHook(), kivi))
    out["hybrid_short_hook"] = _record_full(lambda: plan(HybridShortHook(), kivi))
    out["hybrid_failing_hook"] = _record_full(lambda: plan(HybridFailingHook(), kivi))
    out["hybrid_patched_instance"] = _record_full(lambda: plan(Patched(), kivi))
    out["wrapped_language_model_args"] = _record_full(lambda: plan(Wrapped(), kivi))
    out["empty_outer_layers"] = _record_full(lambda: plan(EmptyOuter(), kivi))
    out["list_bits_over_attention_layers"] = _record_full(lambda: plan(Hybrid(), C(method="kivi", bit_width_inlier=[2, 4], seed=3)))
    out["list_bits_wrong_length"] = _record_full(lambda: plan(Hybrid(), C(method="kivi", bit_width_inlier=[2, 4, 8])))
    out["rvq_default_method"] = _record_full(lambda: plan(Flat(), C(head_dim=4)))
    out["no_head_dim_anywhere"] = _record_full(lambda: plan(Nested(None), kivi))

    # the fluent surface and build()'s own validation (the factory again replaced by the recorder)
    def built(make):
        original = F.create
        F.create = staticmethod(lambda c: [c.method, c.head_dim, c.bit_width_inlier, c.bit_width_outlier, c.seed, c.capacity,
                                           c.sliding_window, len(c.observers), str(c.dtype)])
        try:
            return make(Bld()).build()
        finally:
            F.create = staticmethod(original)

    out["fluent_defaults"] = _record_full(lambda: built(lambda b: b))
    out["fluent_every_setter"] = _record_full(lambda: built(
        lambda b: b.with_method("kivi").with_head_dim(64).with_bit_width(4).with_seed(7).with_precision("f16").with_capacity(4096)
        .with_sliding_window(512).with_observer("obs")))
    out["fluent_bit_width_pair"] = _record_full(lambda: built(lambda b: b.with_method("kivi").with_bit_width(inlier=2, outlier=3)))
    out["fluent_head_dim_96"] = _record_full(lambda: built(lambda b: b.with_head_dim(96)))
    out["fluent_head_dim_0"] = _record_full(lambda: built(lambda b: b.with_head_dim(0)))
    out["fluent_bits_0"] = _record_full(lambda: built(lambda b: b.with_method("kivi").with_bit_width(0)))
    out["fluent_bits_empty_list"] = _record_full(lambda: built(lambda b: b.with_method("kivi").with_bit_width([])))
    out["fluent_bits_list_with_zero"] = _record_full(lambda: built(lambda b: b.with_method("kivi").with_bit_width([2, 0])))
    out["fluent_bits_list_with_float"] = _record_full(lambda: built(lambda b: b.with_method("kivi").with_bit_width([2, 2.0])))
    out["fluent_bits_list_reaches_factory"] = _record_full(lambda: built(lambda b: b.with_method("kivi").with_bit_width([2, 4])))
    return out
